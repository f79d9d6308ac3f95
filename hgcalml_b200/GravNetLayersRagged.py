"""Host-side mirror of the two GravNet layers of HGCalML's ``modules/GravNetLayersRagged.py`` that sit
directly on the kNN + accumulation path: ``RaggedGravNet`` (:3102-3288) and
``DistanceWeightedMessagePassing`` (:3540-3612), as inference-time torch modules on CUDA tensors.

The dense layers are plain library GEMMs (``torch.nn.functional.linear``); everything between them --
neighbour search, the slice that drops the self slot, ``10.*distsq``, ``exp``, the weighted mean / max,
the subtraction of the hit's own features and the concatenation -- is the library's
``hgc_binned_select_knn_ragged`` and ``hgc_gravnet_collect``: the collected features are written
straight into their columns of the concatenation buffer."""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import _capi as C
from .binned_select_knn_op import BinnedSelectKnn

_ACTIVATIONS = {
    None: lambda t: t,
    "linear": lambda t: t,
    "relu": torch.relu,
    "elu": torch.nn.functional.elu,
    "tanh": torch.tanh,
    "sigmoid": torch.sigmoid,
    "selu": torch.selu,
    "gelu": torch.nn.functional.gelu,
}


def _activation(name):
    if callable(name):
        return name
    if name not in _ACTIVATIONS:
        raise ValueError(f"unsupported activation {name!r}")
    return _ACTIVATIONS[name]


def collect_neighbours(features, neighbour_indices, distancesq, *, first_slot: int = 0,
                       n_neighbours: Optional[int] = None, subtract_self: bool = False,
                       out: Optional[torch.Tensor] = None, out_column: int = 0,
                       order: Optional[torch.Tensor] = None, distance_scale: float = 10.,
                       with_max_idxs: bool = False):
    """``AccumulateKnn(10.*distancesq, features, neighbour_indices)`` of the GravNet layers
    (modules/GravNetLayersRagged.py:3264-3270, :3602-3609), optionally with the slice of the neighbour
    slots (``first_slot``, ``n_neighbours``), the subtraction ``features -= tile(prev_feat, [1, 2])``
    (:3202, :3597) and the placement into a wider row-major buffer (``out`` / ``out_column``) folded in.

    Returns ``(collected [N, 2F] (a view of ``out`` when given), max_idxs or None)``."""
    C.require_cuda(features, neighbour_indices, distancesq)
    feat, idx, dist = C.f32(features), C.i32(neighbour_indices), C.f32(distancesq)
    n, ld = idx.shape
    f = feat.shape[1]
    if dist.shape != idx.shape or feat.shape[0] != n:
        raise C.HgcError("collect_neighbours: distances, indices and features must agree in their first "
                         "dimensions and the first two in their second")
    k = ld - first_slot if n_neighbours is None else n_neighbours
    if out is None:
        out = torch.empty((n, 2 * f), dtype=torch.float32, device=feat.device)
        out_column = 0
    if out.dtype != torch.float32 or out.dim() != 2 or out.stride(1) != 1 or out.shape[0] != n or \
            out_column < 0 or out_column + 2 * f > out.shape[1]:
        raise C.HgcError("collect_neighbours: out must be a row-major float32 [N, >= out_column + 2F] buffer")
    maxidx = torch.empty((n, f), dtype=torch.int32, device=feat.device) if with_max_idxs else None
    if order is not None:
        C.require_cuda(order)
        order = C.i32(order)
    view = out[:, out_column:out_column + 2 * f]
    C.check(C.lib.hgc_gravnet_collect(C.ptr(dist), C.ptr(idx), ld, first_slot, k, C.ptr(feat),
                                      view.data_ptr() if n else None, out.stride(0), C.ptr(maxidx), n, f,
                                      float(distance_scale), int(bool(subtract_self)), C.ptr(order),
                                      C.stream_of(feat)), "gravnet_collect")
    return view, maxidx


class _Dense(torch.nn.Module):
    """``tf.keras.layers.Dense``: ``activation(x @ kernel + bias)`` with the kernel stored [in, out]."""

    def __init__(self, n_in: int, n_out: int, activation=None, use_bias: bool = True):
        super().__init__()
        self.kernel = torch.nn.Parameter(torch.empty(n_in, n_out))
        torch.nn.init.xavier_uniform_(self.kernel)  # Keras' default glorot_uniform
        self.bias = torch.nn.Parameter(torch.zeros(n_out)) if use_bias else None
        self.activation = _activation(activation)

    def forward(self, x):
        y = x @ self.kernel
        if self.bias is not None:
            y = y + self.bias
        return self.activation(y)

    def set_weights(self, weights: Sequence):
        """Keras order: ``[kernel [in, out], bias [out]]`` (bias absent when ``use_bias=False``)."""
        with torch.no_grad():
            self.kernel.copy_(torch.as_tensor(weights[0]))
            if self.bias is not None:
                self.bias.copy_(torch.as_tensor(weights[1]))


class RaggedGravNet(torch.nn.Module):
    """modules/GravNetLayersRagged.py:3102-3288, forward pass (``priv_call`` :3206-3224).

    Inputs ``[x [N, F_in], row_splits [E+1]]``; returns ``(outfeats [N, n_filters], coordinates
    [N, n_dimensions], neighbour_indices, distancesq)`` where the last two hold ``n_neighbours`` slots
    without the self slot, or ``n_neighbours + 1`` with it when ``return_self`` (:3218-3223)."""

    def __init__(self, n_neighbours: int, n_dimensions: int, n_filters: int, n_propagate: int, n_in: int,
                 return_self: bool = True, sumwnorm: bool = False, feature_activation="relu",
                 n_knn_bins: Optional[int] = None):
        super().__init__()
        assert n_neighbours > 1
        if sumwnorm:
            raise NotImplementedError("sumwnorm=True uses the op AccumulateKnnSumw, which is not part of this library")
        self.n_neighbours, self.n_dimensions, self.n_filters = n_neighbours, n_dimensions, n_filters
        self.n_propagate, self.return_self, self.n_knn_bins = n_propagate, return_self, n_knn_bins
        self.input_feature_transform = _Dense(n_in, n_propagate, feature_activation)
        self.input_spatial_transform = _Dense(n_in, n_dimensions, None, use_bias=False)
        self.output_feature_transform = _Dense(2 * n_propagate + n_in, n_filters, "relu")

    def forward(self, inputs):
        x, row_splits = inputs
        x = C.f32(x)
        n, f_in = x.shape
        coordinates = self.input_spatial_transform(x).contiguous()
        # compute_neighbours_and_distancesq (:3246-3261): the op is asked for the self slot as well
        idx, dist, sorting = BinnedSelectKnn(self.n_neighbours + 1, coordinates, row_splits,
                                             n_bins=self.n_knn_bins, return_sorting=True)
        # create_output_features (:3195-3204): [mean - own | max - own | x] in one buffer
        features = self.input_feature_transform(x).contiguous()
        p = self.n_propagate
        cat = torch.empty((n, 2 * p + f_in), dtype=torch.float32, device=x.device)
        collect_neighbours(features, idx, dist, first_slot=1, n_neighbours=self.n_neighbours,
                           subtract_self=True, out=cat, out_column=0, order=sorting)
        cat[:, 2 * p:] = x
        outfeats = self.output_feature_transform(cat)
        if self.return_self:
            return outfeats, coordinates, idx, dist
        return outfeats, coordinates, idx[:, 1:], dist[:, 1:]


class DistanceWeightedMessagePassing(torch.nn.Module):
    """modules/GravNetLayersRagged.py:3540-3612.  Inputs ``[x, neighbor_indices [N, K], distancesq
    [N, K]]``; returns ``[N, 2*sum(n_feature_transformation) + F_in]``: per pass the collected
    ``[mean - own | max - own]`` of the transformed features, then ``x`` (:3587-3600).  ``order``
    (optional) is a processing order for the accumulation, e.g. the sorting of ``BinnedSelectKnn``."""

    def __init__(self, n_feature_transformation: Sequence[int], n_in: int, sumwnorm: bool = False,
                 activation="relu"):
        super().__init__()
        if sumwnorm:
            raise NotImplementedError("sumwnorm=True uses the op AccumulateKnnSumw, which is not part of this library")
        self.n_feature_transformation = list(n_feature_transformation)
        widths = [n_in] + [2 * f for f in self.n_feature_transformation[:-1]]
        self.feature_tranformation_dense = torch.nn.ModuleList(
            _Dense(w, f, activation) for w, f in zip(widths, self.n_feature_transformation))

    def forward(self, inputs, order=None):
        x, neighbor_indices, distancesq = inputs
        x = C.f32(x)
        n, f_in = x.shape
        total = 2 * sum(self.n_feature_transformation)
        cat = torch.empty((n, total + f_in), dtype=torch.float32, device=x.device)
        features, col = x, 0
        for dense, f in zip(self.feature_tranformation_dense, self.n_feature_transformation):
            prev_feat = dense(features).contiguous()
            features, _ = collect_neighbours(prev_feat, neighbor_indices, distancesq, subtract_self=True,
                                             out=cat, out_column=col, order=order)
            col += 2 * f
        cat[:, total:] = x
        return cat
