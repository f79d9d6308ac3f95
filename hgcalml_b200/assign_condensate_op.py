"""Host-side mirror of HGCalML's ``modules/assign_condensate_op.py`` on torch CUDA tensors."""
from __future__ import annotations

import ctypes
import math

import torch

from . import _capi as C
from .bin_by_coordinates_op import BinByCoordinates


def _BinnedAssignToCondensates(ccoords, dist, beta, no_condensation_mask, bins_flat, bin_splits,
                               indices_to_filtered, original_indices, row_splits, n_bins, bin_widths,
                               ccoords_h, dist_h, beta_h, no_condensation_mask_h, row_splits_h,
                               beta_threshold=0., assign_by_max_beta=True):
    """The registered op ``BinnedAssignToCondensates``
    (modules/compiled/binned_assign_to_condensates_module.cc:7-31), inputs in bin-sorted order.
    Returns ``assigned_h, assigned, alpha_indices, association, n_condensates``."""
    del beta_threshold, bins_flat  # attributes / inputs the reference kernel never reads
    C.require_cuda(ccoords, dist, beta, ccoords_h)
    ccoords, ccoords_h = C.f32(ccoords), C.f32(ccoords_h)
    dev = ccoords.device
    n, dims = ccoords.shape
    dist, dist_h, beta_h = C.f32(dist).reshape(-1), C.f32(dist_h).reshape(-1), C.f32(beta_h).reshape(-1)
    mask, mask_h = C.i32(no_condensation_mask).reshape(-1), C.i32(no_condensation_mask_h).reshape(-1)
    itf, orig_h = C.i32(indices_to_filtered), C.i32(original_indices)
    row_splits, row_splits_h = C.i32(row_splits, dev), C.i32(row_splits_h, dev)
    bin_splits, n_bins, bin_widths = C.i32(bin_splits), C.i32(n_bins, dev), C.f32(bin_widths, dev)
    nh = beta_h.shape[0]
    num_rows = row_splits.shape[0] - 1
    assigned_h = torch.empty((nh,), dtype=torch.int32, device=dev)
    assigned = torch.empty((n,), dtype=torch.int32, device=dev)
    alpha = torch.empty((nh,), dtype=torch.int32, device=dev)
    asso = torch.empty((n,), dtype=torch.int32, device=dev)
    ncond = torch.empty((num_rows + 1,), dtype=torch.int32, device=dev)
    ws = C.workspace(C.lib.hgc_binned_assign_to_condensates_workspace_bytes(n, nh, num_rows, dims), dev)
    C.check(C.lib.hgc_binned_assign_to_condensates(
        dims, n_bins.shape[0], C.ptr(ccoords_h), C.ptr(dist_h), C.ptr(beta_h), C.ptr(mask_h),
        C.ptr(assigned_h), C.ptr(orig_h), C.ptr(row_splits_h), C.ptr(ccoords), C.ptr(dist), C.ptr(mask),
        C.ptr(itf), C.ptr(assigned), C.ptr(asso), C.ptr(ncond), C.ptr(alpha), C.ptr(bin_splits),
        C.ptr(n_bins), C.ptr(bin_widths), C.ptr(row_splits), num_rows, n, nh,
        int(bool(assign_by_max_beta)), C.ptr(ws), ws.numel(), C.stream_of(ccoords)),
        "BinnedAssignToCondensates")
    return assigned_h, assigned, alpha, asso, ncond


def merge_noise_as_indiv_cp(assignment, asso_idx, alpha_idx, is_cond, n_condensates, row_splits):
    """modules/assign_condensate_op.py:16-44: every noise hit (assignment < 0) becomes a condensation
    point of its own.  Per event the noise hits take the shower numbers 0..n_noise-1 in hit order and
    the real showers are shifted up by n_noise; ``alpha_idx`` lists, per event, the noise hits first
    and then the condensates; noise hits are associated to themselves and flagged as condensates."""
    dev = assignment.device
    rs = row_splits.to(torch.int64)
    n = assignment.shape[0]
    num_rows = rs.shape[0] - 1
    a = assignment[:, 0].to(torch.int64)
    seg = torch.repeat_interleave(torch.arange(num_rows, device=dev), rs[1:] - rs[:-1])
    noise = a < 0
    csum = torch.cumsum(noise.to(torch.int64), 0)
    before_event = torch.cat([torch.zeros(1, dtype=torch.int64, device=dev), csum])[rs[:-1]]
    x = torch.where(noise, csum - before_event[seg], torch.zeros_like(csum))  # 1-based rank among the event's noise
    n_noise = torch.zeros(num_rows, dtype=torch.int64, device=dev).scatter_reduce(0, seg, x, "amax", include_self=True)
    new_assignment = torch.where(noise, x - 1, a + n_noise[seg]).to(torch.int32)

    allrange = torch.arange(n, device=dev)
    nc = n_condensates.to(torch.int64)
    cond_event = torch.repeat_interleave(torch.arange(num_rows, device=dev), nc[1:] - nc[:-1])
    noise_idx = allrange[noise]
    # per event: noise hits, then condensates -- a stable sort by (event, kind)
    keys = torch.cat([seg[noise] * 2, cond_event * 2 + 1])
    vals = torch.cat([noise_idx, alpha_idx.to(torch.int64)])
    new_alpha = vals[torch.sort(keys, stable=True).indices].to(torch.int32)

    cond = is_cond[:, 0].clone()
    cond[asso_idx < 0] = True
    new_asso = torch.where(asso_idx < 0, allrange.to(asso_idx.dtype), asso_idx)
    per_event = torch.zeros(num_rows, dtype=torch.int64, device=dev).scatter_add(0, seg, cond.to(torch.int64))
    new_ncond = torch.cat([n_condensates[0:1].to(torch.int64), torch.cumsum(per_event, 0)]).to(torch.int32)
    return new_assignment[:, None], new_asso, new_alpha, cond[:, None], new_ncond


def _segment_ids_to_row_splits(ids, num_segments):
    counts = torch.bincount(ids.to(torch.int64), minlength=num_segments)
    return torch.cat([torch.zeros(1, dtype=torch.int64, device=ids.device), counts.cumsum(0)]).to(torch.int32)


def BuildAndAssignCondensatesBinned(ccoords, betas, dist, row_splits, beta_threshold,
                                    no_condensation_mask=None, distance_threshold=1.,
                                    assign_by_max_beta=False, nbin_dims=3, keep_noise=False):
    """modules/assign_condensate_op.py:210-373.

    Returns ``assignment [N,1], association [N], alpha_idx, is_cond [N,1], n_condensates`` with the
    reference's meaning.  Everything up to ``keep_noise`` is one library call
    (``hgc_build_and_assign_condensates``: threshold scaling, shift, binning, stable sort by bin,
    high-beta filter, the op, mapping back); the ``keep_noise`` renumbering runs as tensor ops."""
    assert 1 <= nbin_dims <= 6
    assert 0. <= beta_threshold <= 1.
    assert distance_threshold > 0.
    ccoords = C.f32(ccoords)
    C.require_cuda(ccoords)
    dev = ccoords.device
    n, dims = ccoords.shape
    betas = C.f32(betas, dev).reshape(-1)
    dist = C.f32(dist, dev).reshape(-1)
    row_splits = C.i32(row_splits, dev)
    n_rs = row_splits.shape[0]
    if betas.shape[0] != n or dist.shape[0] != n:
        raise C.HgcError("BuildAndAssignCondensatesBinned: ccoords, betas and dist must have one row per hit")
    mask = None
    if no_condensation_mask is not None:
        mask = C.i32(no_condensation_mask, dev).reshape(-1)
    assignment = torch.empty((n,), dtype=torch.int32, device=dev)
    asso = torch.empty((n,), dtype=torch.int32, device=dev)
    alpha = torch.empty((n,), dtype=torch.int32, device=dev)
    is_cond = torch.empty((n,), dtype=torch.uint8, device=dev)
    n_condensates = torch.empty((n_rs,), dtype=torch.int32, device=dev)
    ws = C.workspace(C.lib.hgc_build_and_assign_condensates_workspace_bytes(n, dims, n_rs, nbin_dims), dev)
    n_alpha = ctypes.c_int(0)
    C.check(C.lib.hgc_build_and_assign_condensates(
        C.ptr(ccoords), C.ptr(betas), C.ptr(dist), C.ptr(mask), C.ptr(row_splits),
        C.ptr(assignment), C.ptr(asso), C.ptr(alpha), C.ptr(is_cond), C.ptr(n_condensates),
        ctypes.addressof(n_alpha), n, dims, n_rs, float(beta_threshold), float(distance_threshold),
        int(bool(assign_by_max_beta)), nbin_dims, C.ptr(ws), ws.numel(), C.stream_of(ccoords)),
        "BuildAndAssignCondensatesBinned")
    out = (assignment[:, None], asso, alpha[:n_alpha.value], is_cond.to(torch.bool)[:, None], n_condensates)
    if keep_noise:
        out = merge_noise_as_indiv_cp(*out, row_splits)
    return out


def BuildAndAssignCondensatesBinnedStepwise(ccoords, betas, dist, row_splits, beta_threshold,
                                            no_condensation_mask=None, distance_threshold=1.,
                                            assign_by_max_beta=False, nbin_dims=3, keep_noise=False):
    """The same function with the reference's tensor glue (modules/assign_condensate_op.py:245-310)
    spelled out step by step on CUDA tensors around the registered op ``_BinnedAssignToCondensates``;
    kept as the readable statement of what the one-call version does."""
    assert 1 <= nbin_dims <= 6
    assert 0. <= beta_threshold <= 1.
    assert distance_threshold > 0.
    ccoords = C.f32(ccoords)
    C.require_cuda(ccoords)
    dev = ccoords.device
    betas = C.f32(betas, dev).reshape(-1, 1)
    dist = C.f32(dist, dev).reshape(-1, 1) / distance_threshold
    row_splits = C.i32(row_splits, dev)
    num_rows = row_splits.shape[0] - 1
    n = ccoords.shape[0]
    if no_condensation_mask is None:
        no_condensation_mask = torch.zeros((n, 1), dtype=torch.int32, device=dev)
    mask = C.i32(no_condensation_mask, dev).reshape(-1, 1)

    rs_host = row_splits.cpu()
    nvertmax = int(rs_host[-1] - rs_host[0])
    n_bins_sc = max(4, min(int(math.ceil(math.pow(nvertmax / 5, 1 / 3))), 25))
    ccoords = ccoords - ccoords.min(dim=0, keepdim=True).values
    ccoords_2 = ccoords[:, 0:min(ccoords.shape[1], nbin_dims)].contiguous()
    _, bins_flat, n_bins, bin_width = BinByCoordinates(ccoords_2, row_splits, n_bins=n_bins_sc,
                                                       calc_n_per_bin=False, pre_normalized=True)
    sorting = torch.sort(bins_flat, stable=True).indices
    sorting_back = torch.empty_like(sorting)
    sorting_back[sorting] = torch.arange(n, device=dev)
    ccoords, betas, dist, mask = ccoords[sorting], betas[sorting], dist[sorting], mask[sorting]
    bins_flat = bins_flat[sorting]
    orig = sorting.to(torch.int32)
    total_bins = int(torch.prod(n_bins.cpu().to(torch.int64))) * num_rows
    bin_splits = _segment_ids_to_row_splits(bins_flat, total_bins)

    high = torch.logical_or(betas > beta_threshold, mask > 0)[:, 0]
    seg = torch.repeat_interleave(torch.arange(num_rows, device=dev),
                                  (row_splits[1:] - row_splits[:-1]).to(torch.int64))
    row_splits_h = _segment_ids_to_row_splits(seg[high], num_rows)
    betas_h, ccoords_h, dist_h = betas[high], ccoords[high], dist[high]
    mask_h, orig_h = mask[high], orig[high]
    nh = int(betas_h.shape[0])
    itf = torch.full((n,), -1, dtype=torch.int32, device=dev)
    itf[high] = torch.arange(nh, dtype=torch.int32, device=dev)

    _, assignment, alpha, asso, n_condensates = _BinnedAssignToCondensates(
        ccoords=ccoords, dist=dist, beta=betas, no_condensation_mask=mask, bins_flat=bins_flat,
        bin_splits=bin_splits, indices_to_filtered=itf, original_indices=orig_h, row_splits=row_splits,
        n_bins=n_bins, bin_widths=bin_width, ccoords_h=ccoords_h, dist_h=dist_h, beta_h=betas_h,
        no_condensation_mask_h=mask_h, row_splits_h=row_splits_h, beta_threshold=beta_threshold,
        assign_by_max_beta=assign_by_max_beta)

    assignment = assignment[sorting_back]
    asso = asso[sorting_back]
    alpha_idx = alpha[alpha != -1]
    is_cond = torch.zeros((n,), dtype=torch.bool, device=dev)
    is_cond[alpha_idx.to(torch.int64)] = True
    out = (assignment[:, None], asso, alpha_idx, is_cond[:, None], n_condensates)
    if keep_noise:
        out = merge_noise_as_indiv_cp(*out, row_splits)
    return out
