"""Host-side mirror of HGCalML's ``modules/accknn_op.py`` on torch CUDA tensors."""
from __future__ import annotations

import torch

from . import _capi as C


def _prepare(weights, features, indices, mean_and_max, with_max_idxs):
    C.require_cuda(weights, features, indices)
    weights, features, indices = C.f32(weights), C.f32(features), C.i32(indices)
    n, k = indices.shape
    f = features.shape[1]
    if features.shape[0] != n or weights.shape[0] != n:
        raise C.HgcError("AccumulateKnnOp expects first dimensions of all inputs to match.")
    if weights.shape[1] != k:
        raise C.HgcError("AccumulateKnnOp expects second dimension of distance and neighbour index "
                         "tensor to match")
    n_out = 2 * f if mean_and_max else f
    out = torch.empty((n, n_out), dtype=torch.float32, device=features.device)
    maxidx = None
    if with_max_idxs:
        maxidx = torch.empty((n, f), dtype=torch.int32, device=features.device)
        if not mean_and_max:
            maxidx.zero_()
    return weights, features, indices, out, maxidx, n, k, f, n_out


def AccumulateLinKnn(weights, features, indices, mean_and_max=True, force_tf=False, with_max_idxs=True):
    """Accumulates neighbour features with linear weights: the registered op ``AccumulateKnn``
    as is (modules/accknn_op.py:17-36, modules/compiled/accumulate_knn_module.cc:7-14).
    Returns ``(out_features [N, 2F or F], out_max_idxs [N, F])``."""
    del force_tf
    w, feat, idx, out, maxidx, n, k, f, n_out = _prepare(weights, features, indices, mean_and_max,
                                                        with_max_idxs)
    C.check(C.lib.hgc_accumulate_knn(C.ptr(w), C.ptr(feat), C.ptr(idx), C.ptr(out), C.ptr(maxidx),
                                     n, k, f, n_out, 0, int(bool(mean_and_max)), C.stream_of(feat)),
            "AccumulateKnn")
    return out, maxidx


def AccumulateKnn(distances, features, indices, mean_and_max=True, force_tf=False, with_max_idxs=True,
                  order=None, distance_scale=1.):
    """modules/accknn_op.py:39-58: weights are ``exp(-distances)``, computed inside the kernel.

    Indices may be padded with trailing -1.  ``order`` (optional int32 permutation of the hits) only
    sets the order in which rows are processed; the bin-sorting permutation of BinnedSelectKnn keeps
    neighbouring hits together and makes the feature gather cache-friendly.  ``distance_scale`` is
    multiplied into the distances inside the kernel (``AccumulateKnn(10.*distsq, ..)`` of GravNet is
    ``distance_scale=10`` on the raw squared distances, without the extra elementwise pass)."""
    del force_tf
    d, feat, idx, out, maxidx, n, k, f, n_out = _prepare(distances, features, indices, mean_and_max,
                                                        with_max_idxs)
    if order is not None:
        C.require_cuda(order)
        order = C.i32(order)
    C.check(C.lib.hgc_accumulate_knn_exp(C.ptr(d), C.ptr(feat), C.ptr(idx), C.ptr(out), C.ptr(maxidx),
                                         n, k, f, n_out, int(bool(mean_and_max)), float(distance_scale),
                                         C.ptr(order),
                                         C.stream_of(feat)), "AccumulateKnn")
    return out, maxidx
