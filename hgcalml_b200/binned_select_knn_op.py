"""Host-side mirror of HGCalML's ``modules/binned_select_knn_op.py`` on torch CUDA tensors."""
from __future__ import annotations

import torch

from . import _capi as C


def _BinnedSelectKnn(K: int, coords, bin_idx, dim_bin_idx, bin_boundaries, n_bins, bin_width,
                     tf_compatible=False, direction=None):
    """The registered op ``BinnedSelectKnn`` on bin-sorted inputs
    (modules/binned_select_knn_op.py:9-30, modules/compiled/binned_select_knn_module.cc:8-20).
    Argument checks repeat the op's (modules/compiled/binned_select_knn_kernel.cc:336-352)."""
    C.require_cuda(coords, bin_idx, dim_bin_idx, bin_boundaries, n_bins, bin_width, direction)
    coords, bin_width = C.f32(coords), C.f32(bin_width)
    bin_idx, dim_bin_idx = C.i32(bin_idx), C.i32(dim_bin_idx)
    bin_boundaries, n_bins = C.i32(bin_boundaries), C.i32(n_bins)
    use_direction = direction is not None
    if use_direction:
        direction = C.i32(direction)
    n, c = coords.shape
    n_bin_dims = n_bins.shape[0]
    if n_bin_dims < 2:
        raise C.HgcError("BinnedSelectKnnOp expects at least 2 binning dimensions.")
    if n_bin_dims > 5:
        raise C.HgcError("BinnedSelectKnnOp expects maximum 5 binning dimensions.")
    if dim_bin_idx.shape[1] - 1 != n_bin_dims:
        raise C.HgcError("BinnedSelectKnnOp expects number of bin dimensions (including row splits) -1 "
                         "== number of total bin dimensions.")
    if c < 2:
        raise C.HgcError("BinnedSelectKnnOp expects at least 2 dimensions.")
    if bin_idx.shape[0] != n:
        raise C.HgcError("BinnedSelectKnnOp expects same first dimension for bin idx and coordinates.")
    if bin_width.numel() != 1:
        raise C.HgcError("BinnedSelectKnnOp expects singleton (dim(1)) for bin width.")
    if use_direction and direction.shape[0] != n:
        raise C.HgcError("BinnedSelectKnnOp needs a direction tensor with length nvert if use_direction=True.")
    dev = coords.device
    idx = torch.empty((n, K), dtype=torch.int32, device=dev)
    dist = torch.empty((n, K), dtype=torch.float32, device=dev)
    ws = C.workspace(C.lib.hgc_binned_select_knn_workspace_bytes(n, K, c, n_bin_dims), dev)
    C.check(C.lib.hgc_binned_select_knn(
        C.ptr(coords), C.ptr(bin_idx), C.ptr(direction), C.ptr(dim_bin_idx), C.ptr(bin_boundaries),
        C.ptr(n_bins), C.ptr(bin_width), C.ptr(idx), C.ptr(dist),
        n, K, c, n_bin_dims, bin_boundaries.shape[0], int(bool(tf_compatible)), int(use_direction),
        C.ptr(ws), ws.numel(), C.stream_of(coords)), "BinnedSelectKnn")
    return idx, dist


def BinnedSelectKnn(K: int, coords, row_splits, direction=None, n_bins=None, max_bin_dims=3,
                    tf_compatible=False, max_radius=None, name="", return_sorting=False):
    """modules/binned_select_knn_op.py:32-95: neighbour indices and squared distances, ``[N, K]``
    each, in the caller's order; slot 0 is the hit itself, missing neighbours are -1 / 0.

    One enqueue, no host synchronisation: grid derivation, binning, the stable sort by bin, the
    search and the mapping back all run in the library.  ``max_radius`` is accepted and ignored, as
    in the reference.  ``direction``: 0 can only be neighbour, 1 can only have neighbours, 2 neither.
    ``return_sorting=True`` also returns the bin-sorting permutation (useful as a cache-friendly
    processing order for AccumulateKnn)."""
    del max_radius, name
    C.require_cuda(coords, row_splits, direction)
    coords, row_splits = C.f32(coords), C.i32(row_splits)
    use_direction = direction is not None
    if use_direction:
        direction = C.i32(direction)
    n, c = coords.shape
    n_rs = row_splits.shape[0]
    nb = -1 if n_bins is None else int(n_bins)
    dev = coords.device
    idx = torch.empty((n, K), dtype=torch.int32, device=dev)
    dist = torch.empty((n, K), dtype=torch.float32, device=dev)
    sorting = torch.empty((n,), dtype=torch.int32, device=dev) if return_sorting else None
    nbytes = C.lib.hgc_binned_select_knn_ragged_workspace_bytes(n, K, c, n_rs, nb, max_bin_dims)
    if nbytes == 0:
        raise C.HgcError("BinnedSelectKnn: unsupported combination of sizes")
    ws = C.workspace(nbytes, dev)
    C.check(C.lib.hgc_binned_select_knn_ragged(
        C.ptr(coords), C.ptr(row_splits), C.ptr(direction), C.ptr(idx), C.ptr(dist), C.ptr(sorting),
        n, K, c, n_rs, nb, int(max_bin_dims), int(bool(tf_compatible)), int(use_direction),
        C.ptr(ws), ws.numel(), C.stream_of(coords)), "BinnedSelectKnn")
    if return_sorting:
        return idx, dist, sorting
    return idx, dist


def SelectKnnGrad(grad_distances, indices, distances, coordinates):
    """The registered op ``SelectKnnGrad`` (modules/compiled/select_knn_grad_module.cc), which the
    reference attaches as the gradient of ``BinnedSelectKnn`` (modules/binned_select_knn_op.py:107-118):
    gradient of the squared neighbour distances with respect to the coordinates, ``[N, C]``."""
    C.require_cuda(grad_distances, indices, coordinates)
    g, idx, coords = C.f32(grad_distances), C.i32(indices), C.f32(coordinates)
    d = None if distances is None else C.f32(distances)
    n, k = idx.shape
    out = torch.empty_like(coords)
    ws = C.workspace(C.lib.hgc_knn_grad_workspace_bytes(n, k), coords.device)
    C.check(C.lib.hgc_select_knn_grad(C.ptr(g), C.ptr(idx), C.ptr(d), C.ptr(coords), C.ptr(out),
                                      n, k, coords.shape[1], C.ptr(ws), ws.numel(), C.stream_of(coords)),
            "SelectKnnGrad")
    return out


class _BinnedSelectKnnFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, coords, row_splits, K, n_bins, max_bin_dims, tf_compatible):
        idx, dist = BinnedSelectKnn(K, coords, row_splits, n_bins=n_bins, max_bin_dims=max_bin_dims,
                                    tf_compatible=tf_compatible)
        ctx.save_for_backward(coords, idx, dist)
        ctx.mark_non_differentiable(idx)
        return idx, dist

    @staticmethod
    def backward(ctx, _grad_idx, grad_dist):
        coords, idx, dist = ctx.saved_tensors
        return SelectKnnGrad(grad_dist.contiguous(), idx, dist, coords), None, None, None, None, None


def BinnedSelectKnnDifferentiable(K, coords, row_splits, n_bins=None, max_bin_dims=3, tf_compatible=False):
    """``BinnedSelectKnn`` whose squared distances carry the reference's gradient to the coordinates."""
    return _BinnedSelectKnnFunction.apply(coords, row_splits, K, n_bins, max_bin_dims, tf_compatible)
