"""Host-side mirror of HGCalML's ``modules/push_knn_op.py`` (forward op) on torch CUDA tensors."""
from __future__ import annotations

import torch

from . import _capi as C


def PushKnn(w, f, nidx):
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
