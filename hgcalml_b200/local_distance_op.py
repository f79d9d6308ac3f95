"""Host-side mirror of HGCalML's ``modules/local_distance_op.py`` on torch CUDA tensors."""
from __future__ import annotations

import torch

from . import _capi as C
from .binned_select_knn_op import SelectKnnGrad


def _local_distance(neighbour_idxs, coordinates):
    idx, coords = C.i32(neighbour_idxs), C.f32(coordinates)
    out = torch.empty(idx.shape, dtype=torch.float32, device=coords.device)
    C.check(C.lib.hgc_local_distance(C.ptr(idx), C.ptr(coords), C.ptr(out), coords.shape[1], coords.shape[0],
                                     idx.shape[0], idx.shape[1], C.stream_of(coords)), "LocalDistance")
    return out


class _LocalDistanceFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, coordinates, neighbour_idxs):
        dist = _local_distance(neighbour_idxs, coordinates)
        ctx.save_for_backward(coordinates, neighbour_idxs, dist)
        return dist

    @staticmethod
    def backward(ctx, grad_dist):
        coords, idx, dist = ctx.saved_tensors
        # the reference registers SelectKnnGrad as the gradient (modules/local_distance_op.py:27-40)
        return SelectKnnGrad(grad_dist.contiguous(), idx, dist, coords), None


def LocalDistance(coords, neighbour_idxs):
    """modules/local_distance_op.py:11-18: squared distances ``[V, K]`` from every hit to its listed
    neighbours (0 for -1 and for the hit itself), differentiable with respect to the coordinates
    through SelectKnnGrad as in the reference (:25-40)."""
    C.require_cuda(coords, neighbour_idxs)
    return _LocalDistanceFunction.apply(C.f32(coords), C.i32(neighbour_idxs))
