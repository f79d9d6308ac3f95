"""Host-side mirror of HGCalML's ``modules/push_knn_op.py`` (forward op) on torch CUDA tensors."""
from __future__ import annotations

import torch

from . import _capi as C


def _push_knn(w, f, nidx):
    """The registered op ``PushKnn`` (modules/compiled/push_knn_module.cc:7-11): every hit adds its
    features, weighted per neighbour slot, to its neighbours: ``out[nidx[i,k]] += f[i] * w[i,k]``.
    Contributions are summed in (i, k) order, so the result does not change from run to run."""
    C.require_cuda(w, f, nidx)
    w, f, nidx = C.f32(w), C.f32(f), C.i32(nidx)
    n, k = nidx.shape
    if w.shape != nidx.shape or f.shape[0] != n:
        raise C.HgcError("PushKnn expects weights and indices of equal shape and one feature row per vertex")
    out = torch.empty_like(f)
    ws = C.workspace(C.lib.hgc_knn_grad_workspace_bytes(n, k), f.device)
    C.check(C.lib.hgc_push_knn(C.ptr(w), C.ptr(f), C.ptr(nidx), C.ptr(out), n, k, f.shape[1],
                               C.ptr(ws), ws.numel(), C.stream_of(f)), "PushKnn")
    return out


def PushKnnGrad(grad, weights, features, indices):
    """The registered op ``PushKnnGrad`` (modules/compiled/push_knn_grad_module.cc:7-13).
    Returns ``(weight_grad [N,K], feature_grad [N,F])``."""
    C.require_cuda(grad, weights, features, indices)
    g, w, f, idx = C.f32(grad), C.f32(weights), C.f32(features), C.i32(indices)
    n, k = idx.shape
    wg = torch.empty_like(w)
    fg = torch.empty_like(f)
    C.check(C.lib.hgc_push_knn_grad(C.ptr(g), C.ptr(w), C.ptr(f), C.ptr(idx), C.ptr(fg), C.ptr(wg),
                                    n, k, f.shape[1], C.stream_of(f)), "PushKnnGrad")
    return wg, fg


class _PushKnnFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, w, f, nidx):
        ctx.save_for_backward(w, f, nidx)
        return _push_knn(w, f, nidx)

    @staticmethod
    def backward(ctx, grad):
        w, f, nidx = ctx.saved_tensors
        wg, fg = PushKnnGrad(grad.contiguous(), w, f, nidx)
        return wg, fg, None


def PushKnn(w, f, nidx):
    """modules/push_knn_op.py:8-17 with its registered gradient (:19-37): pushes (sums) weighted
    features to the neighbours; -1 means no neighbour."""
    C.require_cuda(w, f, nidx)
    return _PushKnnFunction.apply(C.f32(w), C.f32(f), C.i32(nidx))
