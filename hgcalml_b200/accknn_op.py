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


def AccumulateKnnGrad(grad_from_out_features, distances, features, neigh_indices, max_feat_indices, order=None):
    """The registered op ``AccumulateKnnGrad`` (modules/compiled/accumulate_knn_grad_module.cc:7-15), the
    gradient the reference attaches to the op ``AccumulateKnn`` (modules/accknn_op.py:71-90).
    ``distances`` are the forward op's weights.  ``order`` (optional int32 permutation of the hits, e.g.
    the sorting of ``BinnedSelectKnn``) only sets the order in which hits are processed.
    Returns ``(grad_distances [N,K], grad_features [N,F])``;
    mean-and-max mode is detected from the width of the incoming gradient, as in the reference."""
    C.require_cuda(grad_from_out_features, distances, features, neigh_indices)
    g, w, feat = C.f32(grad_from_out_features), C.f32(distances), C.f32(features)
    idx = C.i32(neigh_indices)
    n, k = idx.shape
    f = feat.shape[1]
    mean_and_max = g.shape[1] > f
    if mean_and_max:
        C.require_cuda(max_feat_indices)
        maxidx = C.i32(max_feat_indices)
    else:
        maxidx = None
    dev = feat.device
    gw = torch.empty((n, k), dtype=torch.float32, device=dev)
    gf = torch.empty((n, f), dtype=torch.float32, device=dev)
    ws = C.workspace(C.lib.hgc_knn_grad_workspace_bytes(n, k), dev)
    if order is not None:
        C.require_cuda(order)
        order = C.i32(order)
    C.check(C.lib.hgc_accumulate_knn_grad_ordered(C.ptr(g), C.ptr(w), C.ptr(feat), C.ptr(maxidx), C.ptr(idx),
                                                  C.ptr(gw), C.ptr(gf), n, k, f, g.shape[1], 0, int(mean_and_max),
                                                  C.ptr(order), C.ptr(ws), ws.numel(), C.stream_of(feat)),
            "AccumulateKnnGrad")
    return gw, gf


class _AccumulateLinKnnFunction(torch.autograd.Function):
    """AccumulateLinKnn with the reference's gradient wired into torch autograd."""

    @staticmethod
    def forward(ctx, weights, features, indices, mean_and_max, order):
        out, maxidx = AccumulateLinKnn(weights, features, indices, mean_and_max=mean_and_max)
        ctx.save_for_backward(weights, features, indices, maxidx)
        ctx.order = order
        ctx.mark_non_differentiable(maxidx)
        return out, maxidx

    @staticmethod
    def backward(ctx, grad_out, _grad_maxidx):
        weights, features, indices, maxidx = ctx.saved_tensors
        gw, gf = AccumulateKnnGrad(grad_out.contiguous(), weights, features, indices, maxidx, order=ctx.order)
        return gw, gf, None, None, None


def AccumulateKnnDifferentiable(distances, features, indices, mean_and_max=True, order=None):
    """``AccumulateKnn`` as the reference's training path sees it: ``exp(-distances)`` as a
    differentiable tensor op, then the op with its registered gradient (modules/accknn_op.py:52-57,71-90).
    ``order``: optional processing order for the backward pass (see ``AccumulateKnnGrad``)."""
    return _AccumulateLinKnnFunction.apply(torch.exp(-distances), features, indices, mean_and_max, order)
