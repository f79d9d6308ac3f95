"""Host-side mirror of HGCalML's ``modules/bin_by_coordinates_op.py`` on torch CUDA tensors.

Same function name, arguments and return values as the reference wrapper; the op itself runs in
the CUDA library through the C ABI.
"""
from __future__ import annotations

import torch

from . import _capi as C


def _bin_by_coordinates(coordinates, row_splits, bin_width, nbins, calc_n_per_bin):
    """The registered op ``BinByCoordinates`` (modules/compiled/bin_by_coordinates_module.cc:7-15).
    The number of bins, which sizes the third output, is read on the host as the reference's
    NbinsHelper does (modules/compiled/bin_by_coordinates_kernel.cu.cc:18-36)."""
    C.require_cuda(coordinates, row_splits, bin_width, nbins)
    coordinates, bin_width = C.f32(coordinates), C.f32(bin_width)
    row_splits, nbins = C.i32(row_splits), C.i32(nbins)
    if bin_width.numel() != 1:
        raise C.HgcError("BinByCoordinatesOp expects singleton (dim: 1) for bin width.")
    n, c = coordinates.shape
    if nbins.numel() != c:
        raise C.HgcError("BinByCoordinatesOp expects coordinate dimension for number of bins.")
    n_rs = row_splits.numel()
    total = int(torch.prod(nbins.cpu().to(torch.int64))) * (n_rs - 1)
    dev = coordinates.device
    assigned = torch.empty((n, c + 1), dtype=torch.int32, device=dev)
    flat = torch.empty((n,), dtype=torch.int32, device=dev)
    nper = torch.empty((total,), dtype=torch.int32, device=dev)
    ws = C.workspace(C.lib.hgc_bin_by_coordinates_workspace_bytes(n, c, n_rs, total), dev)
    C.check(C.lib.hgc_bin_by_coordinates(
        C.ptr(coordinates), C.ptr(row_splits), C.ptr(bin_width), C.ptr(nbins),
        C.ptr(assigned), C.ptr(flat), C.ptr(nper), n, c, n_rs, total, int(bool(calc_n_per_bin)),
        C.ptr(ws), ws.numel(), C.stream_of(coordinates)), "BinByCoordinates")
    return assigned, flat, nper


def BinByCoordinates(coordinates, row_splits, bin_width=None, n_bins=None, calc_n_per_bin=True,
                     pre_normalized=False, name=""):
    """modules/bin_by_coordinates_op.py:14-88.

    Returns ``binass, flatbinass, n_bins, bin_width[, nperbin]`` like the reference.  The glue
    around the op (min shift, extent, bin width) is float32 tensor arithmetic, as it is there."""
    del name
    coordinates = C.f32(coordinates)
    C.require_cuda(coordinates)
    dev = coordinates.device
    if not torch.isfinite(coordinates).all():
        raise C.HgcError("BinByCoordinates: input coordinates : Tensor had NaN or Inf values")
    if not pre_normalized:
        coordinates = coordinates - coordinates.min(dim=0, keepdim=True).values
    dmax = coordinates.max(dim=0).values
    dmin = coordinates.min(dim=0).values
    dmax = torch.where(dmin == dmax, dmax + 1., dmax) + 1e-3
    dmax = torch.where(torch.isfinite(dmax), dmax, torch.ones_like(dmax))
    if bin_width is None:
        assert n_bins is not None
        bin_width = dmax / torch.as_tensor(n_bins, device=dev).to(torch.float32)
        n_bins = None
        bin_width = bin_width.max().reshape(1)
    else:
        bin_width = C.f32(bin_width, dev).reshape(1)
    if n_bins is None:
        n_bins = (dmax / bin_width + 1.).to(torch.int32)
    else:
        n_bins = C.i32(n_bins, dev)
    binass, flatbinass, nperbin = _bin_by_coordinates(coordinates, C.i32(row_splits, dev), bin_width,
                                                      n_bins, calc_n_per_bin)
    if calc_n_per_bin:
        return binass, flatbinass, n_bins, bin_width, nperbin
    return binass, flatbinass, n_bins, bin_width
