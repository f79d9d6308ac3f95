"""TEST INFRASTRUCTURE ONLY -- CPU checker for the CUDA library.

Two interchangeable back ends compute the op arithmetic:

* ``port``: ``oracle/_build/liboracle.so``, this repository's plain-C
  restatement (``hgc_oracle.c``);
* ``ref``:  ``oracle/_ref/libref.so``, the reference's own CPU kernels compiled
  from a cms-pepr/HGCalML checkout (only present where that was built).

On top of either, this module restates in numpy float32 the TensorFlow glue of
the reference's Python wrappers (min-shift, bin width, stable argsort, gathers,
cumsum, index remap, scatter back), citing the wrapper lines it follows.

Only ``tests/``, the smoke check and the CPU-baseline leg of ``bench.py`` may
import this module; the product never does.
"""
from __future__ import annotations

import ctypes
import math
import os
import subprocess
from ctypes import POINTER, c_float, c_int

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_PORT_SO = os.path.join(_HERE, "_build", "liboracle.so")
_REF_SO = os.path.join(_HERE, "_ref", "libref.so")
_REF_CUDA_SO = os.path.join(_HERE, "_ref", "libref_cuda.so")

_fp = POINTER(c_float)
_ip = POINTER(c_int)


def build(quiet: bool = True) -> None:
    """Compile the checker libraries (the reference one only where a checkout exists)."""
    subprocess.run(["make", "-C", _HERE, "all"], check=True,
                   stdout=subprocess.DEVNULL if quiet else None)


def _f(a):
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return a.ctypes.data_as(_fp)


def _i(a):
    assert a.dtype == np.int32 and a.flags.c_contiguous
    return a.ctypes.data_as(_ip)


def _c32f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _c32i(a):
    return np.ascontiguousarray(a, dtype=np.int32)


class _Lib:
    """ctypes view of one checker library; both export the same five routines."""

    def __init__(self, path: str, prefix: str):
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.path = path
        self.prefix = prefix
        self.dll = ctypes.CDLL(path)

    def fn(self, name):
        return getattr(self.dll, self.prefix + name)


_libs: dict = {}


def have(backend: str) -> bool:
    return os.path.exists(_REF_SO if backend == "ref" else _PORT_SO)


def lib(backend: str = "port") -> _Lib:
    if backend not in _libs:
        if backend == "port":
            if not os.path.exists(_PORT_SO):
                subprocess.run(["make", "-C", _HERE, "port"], check=True, stdout=subprocess.DEVNULL)
            _libs[backend] = _Lib(_PORT_SO, "oracle_")
        elif backend == "ref":
            _libs[backend] = _Lib(_REF_SO, "ref_")
        else:
            raise ValueError(backend)
    return _libs[backend]


# --------------------------------------------------------------------------
# op-level calls (raw functor semantics)
# --------------------------------------------------------------------------
def op_bin_by_coordinates(coords, row_splits, bin_width, n_bins, calc_n_per_bin=True, backend="port"):
    """Functor of bin_by_coordinates_kernel.cc:117-156. Returns (bin_assignment, flat, n_per_bin)."""
    coords = _c32f(coords)
    row_splits = _c32i(row_splits)
    bin_width = _c32f(bin_width).reshape(1)
    n_bins = _c32i(n_bins)
    n, c = coords.shape
    total = int(np.prod(n_bins.astype(np.int64))) * (len(row_splits) - 1)
    assigned = np.zeros((n, c + 1), np.int32)
    flat = np.zeros((n,), np.int32)
    nper = np.zeros((total,), np.int32)
    lib(backend).fn("bin_by_coordinates")(
        _f(coords), _i(row_splits), _f(bin_width), _i(n_bins), _i(assigned), _i(flat), _i(nper),
        c_int(n), c_int(c), c_int(len(row_splits)), c_int(total), c_int(int(calc_n_per_bin)))
    return assigned, flat, nper


def op_binned_select_knn(K, coords, bin_idx, dim_bin_idx, bin_boundaries, n_bins, bin_width,
                         tf_compatible=False, direction=None, backend="port"):
    """Kernel of binned_select_knn_kernel.cc:47-196 on bin-sorted inputs. Returns (idx, distsq)."""
    coords = _c32f(coords)
    bin_idx = _c32i(bin_idx)
    dim_bin_idx = _c32i(dim_bin_idx)
    bin_boundaries = _c32i(bin_boundaries)
    n_bins = _c32i(n_bins)
    bin_width = _c32f(bin_width).reshape(1)
    use_direction = direction is not None
    direction = _c32i(direction if use_direction else np.zeros((0,), np.int32))
    n, c = coords.shape
    idx = np.empty((n, K), np.int32)
    dist = np.empty((n, K), np.float32)
    rc = lib(backend).fn("binned_select_knn")(
        _f(coords), _i(bin_idx), _i(direction), _i(dim_bin_idx), _i(bin_boundaries), _i(n_bins),
        _f(bin_width), _i(idx), _f(dist),
        c_int(n), c_int(K), c_int(c), c_int(len(n_bins)), c_int(len(bin_boundaries)),
        c_int(int(tf_compatible)), c_int(int(use_direction)))
    if rc != 0:
        raise ValueError("unsupported number of binning dimensions")
    return idx, dist


def op_index_replacer(to_be_replaced, replacements, backend="port"):
    """Functor of index_replacer_kernel.cc:15-42."""
    tbr = _c32i(to_be_replaced)
    rep = _c32i(replacements)
    out = np.zeros_like(tbr)
    lib(backend).fn("index_replacer")(_i(tbr.reshape(-1)), _i(rep), _i(out.reshape(-1)),
                                      c_int(tbr.size), c_int(rep.shape[0]))
    return out


def op_accumulate_knn(weights, features, indices, mean_and_max=True, backend="port"):
    """Functor of accumulate_knn_kernel.cc:27-83 (weights are used verbatim)."""
    weights = _c32f(weights)
    features = _c32f(features)
    indices = _c32i(indices)
    n, k = indices.shape
    f = features.shape[1]
    n_out = 2 * f if mean_and_max else f
    out = np.zeros((n, n_out), np.float32)
    maxidx = np.zeros((n, f), np.int32)
    fn = lib(backend).fn("accumulate_knn")
    if backend == "ref":
        fn(_f(weights), _f(features), _i(indices), _f(out), _i(maxidx),
           c_int(n), c_int(k), c_int(f), c_int(n_out), c_int(0), c_int(int(mean_and_max)))
    else:
        fn(_f(weights), _f(features), _i(indices), _f(out), _i(maxidx),
           c_int(n), c_int(k), c_int(f), c_int(n_out), c_int(int(mean_and_max)))
    return out, maxidx


def op_accumulate_knn_grad(grad_out, weights, features, indices, max_idx, backend="port"):
    """Functor of accumulate_knn_grad_kernel.cc:166-221. Returns (grad_weights [N,K], grad_features [N,F])."""
    grad_out = _c32f(grad_out)
    weights = _c32f(weights)
    features = _c32f(features)
    indices = _c32i(indices)
    n, k = indices.shape
    f = features.shape[1]
    mean_and_max = grad_out.shape[1] > f  # the op detects it the same way (accumulate_knn_grad_kernel.cc:246)
    max_idx = _c32i(max_idx) if max_idx is not None else np.zeros((n, f), np.int32)
    gw = np.zeros((n, k), np.float32)
    gf = np.zeros((n, f), np.float32)
    lib(backend).fn("accumulate_knn_grad")(
        _f(grad_out), _f(weights), _f(features), _i(max_idx), _i(indices), _f(gw), _f(gf),
        c_int(n), c_int(k), c_int(f), c_int(grad_out.shape[1]), c_int(int(mean_and_max)))
    return gw, gf


def op_select_knn_grad(grad_dist, indices, coords):
    """Restatement of the reference's GPU kernels for SelectKnnGrad (its CPU functor is empty).
    Only the plain-C back end has it.  Returns grad_coords [N,C]."""
    grad_dist = _c32f(grad_dist)
    indices = _c32i(indices)
    coords = _c32f(coords)
    n, k = indices.shape
    out = np.zeros_like(coords)
    lib("port").fn("select_knn_grad")(_f(grad_dist), _i(indices), _f(coords), _f(out),
                                      c_int(n), c_int(k), c_int(coords.shape[1]))
    return out


def have_ref_cuda() -> bool:
    """True where the reference's GPU kernels of SelectKnnGrad were compiled (oracle/Makefile)."""
    return os.path.exists(_REF_CUDA_SO)


def op_select_knn_grad_ref_cuda(grad_dist, indices, dist, coords):
    """The reference's own GPU functor for SelectKnnGrad (select_knn_grad_kernel.cu.cc:81-216), its
    only implementation of the op, run on the current CUDA device; torch holds the device memory.
    The kernels scatter with float atomicAdd, so the result is reproducible only up to summation
    order.  Returns grad_coords [N,C] as a numpy array."""
    import torch
    dll = ctypes.CDLL(_REF_CUDA_SO)
    dev = torch.device("cuda", torch.cuda.current_device())
    t = [torch.as_tensor(_c32f(grad_dist), device=dev), torch.as_tensor(_c32i(indices), device=dev),
         torch.as_tensor(_c32f(dist), device=dev), torch.as_tensor(_c32f(coords), device=dev)]
    out = torch.zeros_like(t[3])
    torch.cuda.synchronize()  # the functor runs on the legacy default stream
    n, k = indices.shape
    rc = dll.ref_cuda_select_knn_grad(*[ctypes.c_void_p(x.data_ptr()) for x in t], ctypes.c_void_p(out.data_ptr()),
                                      c_int(n), c_int(k), c_int(coords.shape[1]))
    torch.cuda.synchronize()
    if rc != 0:
        raise RuntimeError(f"reference SelectKnnGrad kernels failed with CUDA error {rc}")
    return out.cpu().numpy()


def op_local_distance(coords, neigh_idxs, backend="port"):
    """Functor of local_distance_kernel.cc:47-70. Returns distsq [n_out_vert, K]."""
    coords = _c32f(coords)
    nidx = _c32i(neigh_idxs)
    out = np.zeros(nidx.shape, np.float32)
    lib(backend).fn("local_distance")(_i(nidx), _f(coords), _f(out), c_int(coords.shape[1]),
                                      c_int(coords.shape[0]), c_int(nidx.shape[0]), c_int(nidx.shape[1]))
    return out


def op_push_knn(weights, features, indices, backend="port"):
    """Functor of push_knn_kernel.cc:35-71. Returns out_features [N, F]."""
    weights = _c32f(weights)
    features = _c32f(features)
    indices = _c32i(indices)
    out = np.zeros_like(features)
    lib(backend).fn("push_knn")(_f(weights), _f(features), _i(indices), _f(out), c_int(features.shape[0]),
                                c_int(indices.shape[1]), c_int(features.shape[1]))
    return out


def op_push_knn_grad(grad, weights, features, indices, backend="port"):
    """Functor of push_knn_grad_kernel.cc:22-95. Returns (weight_grad [N,K], feature_grad [N,F])."""
    grad = _c32f(grad)
    weights = _c32f(weights)
    features = _c32f(features)
    indices = _c32i(indices)
    fg = np.zeros_like(features)
    wg = np.zeros_like(weights)
    lib(backend).fn("push_knn_grad")(_f(grad), _f(weights), _f(features), _i(indices), _f(fg), _f(wg),
                                     c_int(features.shape[0]), c_int(indices.shape[1]), c_int(features.shape[1]))
    return wg, fg


def op_binned_assign_to_condensates(ccoords, dist, beta, mask, bins_flat, bin_splits,
                                    indices_to_filtered, original_indices_h, row_splits, n_bins,
                                    bin_width, ccoords_h, dist_h, beta_h, mask_h, row_splits_h,
                                    assign_by_max_beta, backend="port"):
    """Functor of binned_assign_to_condensates_kernel.cc:128-241.
    Returns (assigned_h, assigned, alpha_indices, association, n_condensates)."""
    del bins_flat  # an op input the functor never receives
    ccoords = _c32f(ccoords)
    n, dims = ccoords.shape
    dist = _c32f(dist).reshape(-1)
    mask = _c32i(mask).reshape(-1)
    itf = _c32i(indices_to_filtered)
    orig_h = _c32i(original_indices_h)
    row_splits = _c32i(row_splits)
    n_bins = _c32i(n_bins)
    bin_width = _c32f(bin_width).reshape(1)
    bin_splits = _c32i(bin_splits)
    ccoords_h = _c32f(ccoords_h).reshape(-1, dims)
    dist_h = _c32f(dist_h).reshape(-1)
    beta_h = _c32f(beta_h).reshape(-1)
    mask_h = _c32i(mask_h).reshape(-1)
    row_splits_h = _c32i(row_splits_h)
    nh = beta_h.shape[0]
    # The pick loop reads mask_h[0] or mask_h[1] whatever the subset size; pad so it stays in bounds.
    mask_h_padded = np.concatenate([mask_h, np.zeros(2, np.int32)])
    claimed_h = np.zeros((nh,), np.int32)
    assigned_h = np.zeros((nh,), np.int32)
    assigned = np.zeros((n,), np.int32)
    asso = np.zeros((n,), np.int32)
    alpha = np.zeros((nh,), np.int32)
    ncond = np.zeros((len(row_splits),), np.int32)
    min_d = np.zeros((n,), np.float32)
    rc = lib(backend).fn("binned_assign_to_condensates")(
        c_int(dims), c_int(len(n_bins)), _i(claimed_h), _f(ccoords_h), _f(dist_h), _f(beta_h),
        _i(mask_h_padded), _i(assigned_h), _i(orig_h), _i(row_splits_h), _f(ccoords), _f(dist), _i(mask),
        _i(itf), None if assign_by_max_beta else _f(min_d), _i(assigned), _i(asso), _i(ncond),
        _i(alpha), _i(bin_splits), _i(n_bins), _f(bin_width), _i(row_splits),
        c_int(len(row_splits) - 1), c_int(int(assign_by_max_beta)))
    if rc != 0:
        raise RuntimeError("condensate search made no progress")
    return assigned_h, assigned, alpha, asso, ncond


# --------------------------------------------------------------------------
# wrapper-level restatements (TensorFlow glue in numpy float32)
# --------------------------------------------------------------------------
def BinByCoordinates(coordinates, row_splits, bin_width=None, n_bins=None, calc_n_per_bin=True,
                     pre_normalized=False, backend="port"):
    """modules/bin_by_coordinates_op.py:14-88."""
    coordinates = _c32f(coordinates)
    if not pre_normalized:
        coordinates = coordinates - coordinates.min(axis=0, keepdims=True)
    dmax = coordinates.max(axis=0)
    dmin = coordinates.min(axis=0)
    dmax = (np.where(dmin == dmax, dmax + np.float32(1.), dmax) + np.float32(1e-3)).astype(np.float32)
    dmax = np.where(np.isfinite(dmax), dmax, np.float32(1.)).astype(np.float32)
    if bin_width is None:
        assert n_bins is not None
        bin_width = (dmax / np.float32(n_bins)).astype(np.float32)
        n_bins = None
        bin_width = np.array([bin_width.max()], np.float32)
    else:
        bin_width = _c32f(bin_width).reshape(1)
    if n_bins is None:
        nb = (dmax / bin_width).astype(np.float32) + np.float32(1.)
        n_bins = nb.astype(np.int32)
    else:
        n_bins = _c32i(n_bins)
    binass, flat, nper = op_bin_by_coordinates(coordinates, row_splits, bin_width, n_bins,
                                               calc_n_per_bin, backend)
    if calc_n_per_bin:
        return binass, flat, n_bins, bin_width, nper
    return binass, flat, n_bins, bin_width


def default_n_bins(first_event_size: int, K: int, dims: int) -> int:
    """modules/binned_select_knn_op.py:59-63 (float32 pow, truncation, clamp to [5, 30])."""
    nb = np.power(np.float32(first_event_size) / np.float32(K / 32), np.float32(1 / dims), dtype=np.float32)
    return int(min(max(int(nb), 5), 30))


def BinnedSelectKnn(K, coords, row_splits, direction=None, n_bins=None, max_bin_dims=3,
                    tf_compatible=False, backend="port", return_sorting=False):
    """modules/binned_select_knn_op.py:32-95 with the TF-gradient branch off (globals.py:91)."""
    coords = _c32f(coords)
    row_splits = _c32i(row_splits)
    max_bin_dims = min(max_bin_dims, coords.shape[1])
    if n_bins is None:
        n_bins = default_n_bins(int(row_splits[1]), K, max_bin_dims)
    bin_coords = coords[:, :max_bin_dims]
    dbinning, binning, nb, bin_width, nper = BinByCoordinates(bin_coords, row_splits, n_bins=n_bins,
                                                              backend=backend)
    sorting = np.argsort(binning, kind="stable").astype(np.int32)
    scoords = coords[sorting]
    sbinning = binning[sorting]
    sdbinning = dbinning[sorting]
    sdirection = None if direction is None else _c32i(direction)[sorting]
    bin_boundaries = np.concatenate([np.zeros(1, np.int32), nper]).cumsum().astype(np.int32)
    idx_s, dist_s = op_binned_select_knn(K, scoords, sbinning, sdbinning, bin_boundaries, nb, bin_width,
                                         tf_compatible, sdirection, backend)
    idx_r = op_index_replacer(idx_s, sorting, backend)
    dist = np.zeros_like(dist_s)
    idx = np.zeros_like(idx_r)
    dist[sorting] = dist_s
    idx[sorting] = idx_r
    dist = np.where(idx < 0, np.float32(0.), dist).astype(np.float32)
    if return_sorting:
        return idx, dist, sorting
    return idx, dist


def AccumulateKnn(distances, features, indices, mean_and_max=True, backend="port"):
    """modules/accknn_op.py:39-58: weights = exp(-distances) in float32, then the op."""
    w = np.exp(-_c32f(distances)).astype(np.float32)
    return op_accumulate_knn(w, features, indices, mean_and_max, backend)


def AccumulateLinKnn(weights, features, indices, mean_and_max=True, backend="port"):
    """modules/accknn_op.py:17-36: the op on the weights as given."""
    return op_accumulate_knn(weights, features, indices, mean_and_max, backend)


_NP_ACT = {
    None: lambda t: t,
    "linear": lambda t: t,
    "relu": lambda t: np.maximum(t, np.float32(0.)),
    "tanh": np.tanh,
}


def _np_dense(x, weights, activation):
    """tf.keras.layers.Dense in float32: activation(x @ kernel [+ bias])."""
    y = _c32f(x) @ _c32f(weights[0])
    if len(weights) > 1:
        y = y + _c32f(weights[1])
    return _NP_ACT[activation](y).astype(np.float32)


def gravnet_collect(features, neighbour_indices, distancesq, backend="port"):
    """The collection step shared by the GravNet layers (modules/GravNetLayersRagged.py:3199-3202 with
    :3264-3270, and :3594-3597 with :3602-3609): AccumulateKnn(10.*distsq, features, idx), reshaped
    to [N, 2F], minus tile(features, [1, 2])."""
    features = _c32f(features)
    f, _ = AccumulateKnn(np.float32(10.) * _c32f(distancesq), features, neighbour_indices, backend=backend)
    f = f.reshape(-1, features.shape[1] * 2)
    return (f - np.tile(features, [1, 2])).astype(np.float32)


def RaggedGravNet(x, row_splits, weights, n_neighbours, n_knn_bins=None, feature_activation="relu",
                  return_self=True, dense=_np_dense, backend="port"):
    """Forward pass of RaggedGravNet (modules/GravNetLayersRagged.py:3206-3224 with :3195-3204 and
    :3246-3261).  weights = [[kernel, bias] of input_feature_transform, [kernel] of
    input_spatial_transform, [kernel, bias] of output_feature_transform]; `dense(x, weights, activation)`
    evaluates one dense layer (numpy by default; a test may hand in the very GEMM the other side uses so
    that only the ops are compared)."""
    x = _c32f(x)
    coordinates = dense(x, weights[1], None)
    idx, dist = BinnedSelectKnn(n_neighbours + 1, coordinates, row_splits, n_bins=n_knn_bins, backend=backend)
    dist = np.where(idx < 0, np.float32(0.), dist).astype(np.float32)
    nidx, ndist = idx[:, 1:], dist[:, 1:]
    features = dense(x, weights[0], feature_activation)
    collected = gravnet_collect(features, nidx, ndist, backend)
    out = dense(np.concatenate([collected, x], axis=-1), weights[2], "relu")
    if return_self:
        return out, coordinates, idx, dist
    return out, coordinates, nidx, ndist


def DistanceWeightedMessagePassing(x, neighbour_indices, distancesq, weights, activation="relu",
                                   dense=_np_dense, backend="port"):
    """modules/GravNetLayersRagged.py:3587-3600; weights = [[kernel, bias], ...] per pass."""
    x = _c32f(x)
    allfeat = []
    features = x
    for w in weights:
        prev_feat = dense(features, w, activation)
        features = gravnet_collect(prev_feat, neighbour_indices, distancesq, backend)
        allfeat.append(features)
    return np.concatenate(allfeat + [x], axis=-1)


def _segment_ids_to_row_splits(ids, num_segments):
    counts = np.bincount(ids, minlength=num_segments).astype(np.int64)
    return np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)


def merge_noise_as_indiv_cp(assignment, asso_idx, alpha_idx, is_cond, n_condensates, row_splits):
    """modules/assign_condensate_op.py:16-44, event by event in plain numpy."""
    assignment = np.array(assignment[:, 0], np.int64)
    asso_idx = np.array(asso_idx)
    is_cond = np.array(is_cond[:, 0], bool)
    new_alpha, new_ncond = [], [int(n_condensates[0])]
    for e in range(len(row_splits) - 1):
        lo, hi = int(row_splits[e]), int(row_splits[e + 1])
        a = assignment[lo:hi]
        noise = a < 0
        n_noise = int(noise.sum())
        a = np.where(noise, np.cumsum(noise) - 1, a + n_noise)
        assignment[lo:hi] = a
        new_alpha += list(np.nonzero(noise)[0] + lo) + list(alpha_idx[n_condensates[e]:n_condensates[e + 1]])
        is_cond[lo:hi] |= asso_idx[lo:hi] < 0
        new_ncond.append(new_ncond[-1] + int(is_cond[lo:hi].sum()))
    allrange = np.arange(len(asso_idx))
    asso_idx = np.where(asso_idx < 0, allrange, asso_idx).astype(asso_idx.dtype)
    return (assignment.astype(np.int32)[:, None], asso_idx, np.array(new_alpha, np.int32), is_cond[:, None],
            np.array(new_ncond, np.int32))


def BuildAndAssignCondensatesBinned(ccoords, betas, dist, row_splits, beta_threshold,
                                    no_condensation_mask=None, distance_threshold=1.,
                                    assign_by_max_beta=False, nbin_dims=3, backend="port",
                                    return_op_io=False, keep_noise=False):
    """modules/assign_condensate_op.py:210-333.
    Returns (assignment[N,1], association[N], alpha_idx, is_cond[N,1], n_condensates)."""
    ccoords = _c32f(ccoords)
    betas = _c32f(betas).reshape(-1, 1)
    dist = (_c32f(dist).reshape(-1, 1) / np.float32(distance_threshold)).astype(np.float32)
    row_splits = _c32i(row_splits)
    num_rows = len(row_splits) - 1
    n = ccoords.shape[0]
    if no_condensation_mask is None:
        no_condensation_mask = np.zeros((n, 1), np.int32)
    mask = _c32i(no_condensation_mask).reshape(-1, 1)

    nvertmax = int(row_splits[-1] - row_splits[0])
    n_bins_sc = max(4, min(int(math.ceil(math.pow(nvertmax / 5, 1 / 3))), 25))
    ccoords = ccoords - ccoords.min(axis=0, keepdims=True)
    cc2 = ccoords[:, :min(ccoords.shape[1], nbin_dims)]
    _, bins_flat, n_bins, bin_width = BinByCoordinates(cc2, row_splits, n_bins=n_bins_sc,
                                                       calc_n_per_bin=False, pre_normalized=True,
                                                       backend=backend)
    sorting = np.argsort(bins_flat, kind="stable").astype(np.int32)
    sorting_back = np.argsort(sorting, kind="stable")
    ccoords = ccoords[sorting]
    betas = betas[sorting]
    dist = dist[sorting]
    mask = mask[sorting]
    bins_flat = bins_flat[sorting]
    orig = np.arange(n, dtype=np.int32)[sorting]
    total_bins = int(np.prod(n_bins.astype(np.int64))) * num_rows
    bin_splits = _segment_ids_to_row_splits(bins_flat, total_bins)

    high = np.logical_or(betas > np.float32(beta_threshold), mask > 0)[:, 0]
    seg = np.repeat(np.arange(num_rows), np.diff(row_splits))
    row_splits_h = _segment_ids_to_row_splits(seg[high], num_rows)
    betas_h, ccoords_h, dist_h = betas[high], ccoords[high], dist[high]
    mask_h, orig_h = mask[high], orig[high]
    itf = np.full((n,), -1, np.int32)
    itf[np.nonzero(high)[0]] = np.arange(int(high.sum()), dtype=np.int32)

    op_in = dict(ccoords=ccoords, dist=dist, beta=betas, mask=mask, bins_flat=bins_flat,
                 bin_splits=bin_splits, indices_to_filtered=itf, original_indices_h=orig_h,
                 row_splits=row_splits, n_bins=n_bins, bin_width=bin_width, ccoords_h=ccoords_h,
                 dist_h=dist_h, beta_h=betas_h, mask_h=mask_h, row_splits_h=row_splits_h,
                 assign_by_max_beta=assign_by_max_beta)
    assigned_h, assignment_s, alpha, asso_s, ncond = op_binned_assign_to_condensates(**op_in, backend=backend)
    assignment = assignment_s[sorting_back]
    asso = asso_s[sorting_back]
    alpha_idx = alpha[alpha != -1]
    is_cond = np.zeros((n,), bool)
    is_cond[alpha_idx] = True
    out = (assignment[:, None], asso, alpha_idx, is_cond[:, None], ncond)
    if keep_noise:
        out = merge_noise_as_indiv_cp(*out, row_splits)
    if return_op_io:
        return out, op_in, (assigned_h, assignment_s, alpha, asso_s, ncond)
    return out


# --------------------------------------------------------------------------
# multi-threaded use of the single-threaded CPU ops (ctypes releases the GIL)
# --------------------------------------------------------------------------
def op_binned_select_knn_threaded(K, coords, bin_idx, dim_bin_idx, bin_boundaries, n_bins, bin_width,
                                  n_threads, pool, backend="port"):
    """The search op with its queries split over threads.  Each thread calls the unmodified op with
    the op's own `direction` input set to 0 ("may only be a neighbour") outside its slice of
    queries and 3 (no restriction) inside, and keeps its slice of the rows: identical to one call."""
    n = coords.shape[0]
    bounds = np.linspace(0, n, n_threads + 1).astype(np.int64)
    idx = np.empty((n, K), np.int32)
    dist = np.empty((n, K), np.float32)

    def work(t):
        lo, hi = bounds[t], bounds[t + 1]
        direction = np.zeros((n,), np.int32)
        direction[lo:hi] = 3
        i, d = op_binned_select_knn(K, coords, bin_idx, dim_bin_idx, bin_boundaries, n_bins, bin_width,
                                    direction=direction, backend=backend)
        idx[lo:hi] = i[lo:hi]
        dist[lo:hi] = d[lo:hi]
    list(pool.map(work, range(n_threads)))
    return idx, dist


def op_accumulate_knn_rows(weights, features, indices, lo, hi, backend="port"):
    """AccumulateKnn on rows [lo, hi): the functor only reaches features through the neighbour
    ids, so a row slice of weights / indices / outputs is a plain pointer offset."""
    k = indices.shape[1]
    f = features.shape[1]
    out = np.zeros((hi - lo, 2 * f), np.float32)
    maxidx = np.zeros((hi - lo, f), np.int32)
    fn = lib(backend).fn("accumulate_knn")
    args = [_f(weights[lo:hi]), _f(features), _i(indices[lo:hi]), _f(out), _i(maxidx),
            c_int(hi - lo), c_int(k), c_int(f), c_int(2 * f)]
    if backend == "ref":
        args.append(c_int(0))
    args.append(c_int(1))
    fn(*args)
    return out, maxidx


def knn_accumulate_path(K, coords, feats, row_splits, n_threads=1, pool=None, backend="port",
                        distance_scale=10., return_all=False):
    """The reference's CPU path for one batch -- BinnedSelectKnn wrapper, exp(-scale*d^2) weights,
    AccumulateKnn -- optionally with the per-query / per-row work spread over threads."""
    c = _c32f(coords)
    feats = _c32f(feats)
    row_splits = _c32i(row_splits)
    n = c.shape[0]
    mbd = min(3, c.shape[1])
    nb0 = default_n_bins(int(row_splits[1]), K, mbd)
    dbin, binning, nb, bw, nper = BinByCoordinates(c[:, :mbd], row_splits, n_bins=nb0, backend=backend)
    sorting = np.argsort(binning, kind="stable").astype(np.int32)
    sc, sb, sdb = c[sorting], binning[sorting], dbin[sorting]
    bb = np.concatenate([np.zeros(1, np.int32), nper]).cumsum().astype(np.int32)
    if n_threads <= 1:
        idx_s, dist_s = op_binned_select_knn(K, sc, sb, sdb, bb, nb, bw, backend=backend)
    else:
        idx_s, dist_s = op_binned_select_knn_threaded(K, sc, sb, sdb, bb, nb, bw, n_threads, pool, backend)
    idx_r = op_index_replacer(idx_s, sorting, backend)
    idx = np.empty_like(idx_r)
    dist = np.empty_like(dist_s)
    idx[sorting] = idx_r
    dist[sorting] = dist_s
    dist = np.where(idx < 0, np.float32(0), dist)
    w = np.exp(-(np.float32(distance_scale) * dist)).astype(np.float32)
    if n_threads <= 1:
        out, maxidx = op_accumulate_knn(w, feats, idx, backend=backend)
    else:
        bounds = np.linspace(0, n, n_threads + 1).astype(np.int64)
        out = np.empty((n, 2 * feats.shape[1]), np.float32)
        maxidx = np.empty((n, feats.shape[1]), np.int32)

        def work(t):
            lo, hi = bounds[t], bounds[t + 1]
            out[lo:hi], maxidx[lo:hi] = op_accumulate_knn_rows(w, feats, idx, lo, hi, backend)
        list(pool.map(work, range(n_threads)))
    if return_all:
        return idx, dist, out, maxidx
    return out


# --------------------------------------------------------------------------
# parity helpers
# --------------------------------------------------------------------------
def canonical_knn(idx, dist):
    """Row-wise canonical order: slot 0 stays (the query itself), the other slots are sorted by
    (distance, index) ascending with the -1 padding last.  The reference's own comparison op
    treats rows as sets (compare_knn_outputs_kernel.cc:42-60)."""
    idx = np.asarray(idx)
    dist = np.asarray(dist)
    n, k = idx.shape
    if k <= 1:
        return idx.copy(), dist.copy()
    pad = idx[:, 1:] < 0
    bits = dist[:, 1:].astype(np.float32).view(np.uint32).astype(np.uint64)
    key = (bits << np.uint64(32)) | idx[:, 1:].astype(np.int64).astype(np.uint64) & np.uint64(0xFFFFFFFF)
    key = np.where(pad, np.uint64(0xFFFFFFFFFFFFFFFF), key)
    order = np.argsort(key, axis=1, kind="stable")
    ci = np.concatenate([idx[:, :1], np.take_along_axis(idx[:, 1:], order, axis=1)], axis=1)
    cd = np.concatenate([dist[:, :1], np.take_along_axis(dist[:, 1:], order, axis=1)], axis=1)
    return ci, cd


def brute_force_knn(K, coords, row_splits, max_rows=None, rows=None):
    """Definitional kNN (float32, the reference's distance expression and summation order,
    ties broken by index) for the given query rows; canonical row order."""
    coords = _c32f(coords)
    row_splits = np.asarray(row_splits)
    n = coords.shape[0]
    if rows is None:
        rows = np.arange(n)
        if max_rows is not None and n > max_rows:
            rows = np.random.default_rng(0).choice(n, max_rows, replace=False)
    out_i = np.full((len(rows), K), -1, np.int32)
    out_d = np.zeros((len(rows), K), np.float32)
    ev = np.searchsorted(row_splits, rows, side="right") - 1
    for r, (q, e) in enumerate(zip(rows, ev)):
        lo, hi = int(row_splits[e]), int(row_splits[e + 1])
        d = np.zeros((hi - lo,), np.float32)
        for c in range(coords.shape[1]):
            t = coords[q, c] - coords[lo:hi, c]
            d = d + t * t
        ids = np.arange(lo, hi)
        keep = ids != q
        d, ids = d[keep], ids[keep]
        order = np.lexsort((ids, d))[:K - 1]
        out_i[r, 0] = q
        out_i[r, 1:1 + len(order)] = ids[order]
        out_d[r, 1:1 + len(order)] = d[order]
    return rows, out_i, out_d
