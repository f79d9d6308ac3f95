"""GPU parity tests at the sizes of the benchmark configurations (seeded synthetic inputs with the
configurations' shapes and distributions).  The CPU side is the checker's restatement of the
reference path, run on several host threads where the event is large."""
import os
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import pytest
import torch

from conftest import bits, assert_knn_equal
from hgcalml_b200 import synth
from test_ops_gpu import T, N, exp_weighted_tolerance, COND_KEYS

pytestmark = pytest.mark.gpu

N_THREADS = max(1, min(len(os.sched_getaffinity(0)), 32))


@pytest.fixture(scope="module")
def pool():
    with ThreadPoolExecutor(N_THREADS) as p:
        yield p


def _check_knn_and_accumulate(oracle, pool, cuda, K, c, f, rs, n_bins=None):
    from hgcalml_b200.binned_select_knn_op import BinnedSelectKnn
    from hgcalml_b200.accknn_op import AccumulateKnn, AccumulateLinKnn
    if n_bins is None:
        ri, rd, ro, rm = oracle.knn_accumulate_path(K, c, f, rs, n_threads=N_THREADS, pool=pool, return_all=True)
    else:
        ri, rd = oracle.BinnedSelectKnn(K, c, rs, n_bins=n_bins)
        ro, rm = oracle.AccumulateKnn(np.float32(10.) * rd, f, ri)
    kw = {} if n_bins is None else dict(n_bins=n_bins)
    gi, gd, sorting = BinnedSelectKnn(K, T(c, cuda), T(rs, cuda), return_sorting=True, **kw)
    ties = assert_knn_equal(N(gi), N(gd), ri, rd, what="config")
    assert ties <= 5
    # AccumulateKnn on the REFERENCE's neighbour rows, so that slot order (and with it the float sum) is
    # the same on both sides: linear weights bit-exact, exp weights within 1e-5
    w = np.exp(-(np.float32(10.) * rd)).astype(np.float32)
    go, gm = AccumulateLinKnn(T(w, cuda), T(f, cuda), T(ri, cuda))
    assert np.array_equal(bits(N(go)), bits(ro)) and np.array_equal(N(gm), rm)
    ge, _ = AccumulateKnn(T(rd, cuda), T(f, cuda), T(ri, cuda), distance_scale=10.)
    assert (np.abs(N(ge) - ro) <= exp_weighted_tolerance(np.float32(10.) * rd, f, ri, ro)).all()
    # and the library's own chain (its rows are sorted differently): 1e-5 on the mean, max identical
    gc, _ = AccumulateKnn(gd, T(f, cuda), gi, order=sorting, distance_scale=10.)
    gc = N(gc)
    F = f.shape[1]
    tol = exp_weighted_tolerance(np.float32(10.) * rd, f, ri, ro)
    ok_rows = (np.sort(N(gi), axis=1) == np.sort(ri, axis=1)).all(axis=1)  # rows without a boundary tie
    assert (np.abs(gc - ro) <= tol)[ok_rows].all()
    return ties


def test_config1_uniform_20k(cuda, oracle, pool):
    """One event, N=20000 uniform in [0,1)^3, n_bins=10, K=16, F=32."""
    c, f, rs = synth.uniform_event(20000, 3, 32, seed=101)
    _check_knn_and_accumulate(oracle, pool, cuda, 16, c, f, rs, n_bins=10)


def test_config2_ragged_showers(cuda, oracle, pool):
    """Four ragged events of 50k-150k hits, 4 coordinates, showers + noise, K=64, F=64."""
    c, f, rs = synth.ragged_shower_batch(4, 50000, 150000, dims=4, n_feat=64, seed=200)
    assert 200000 <= len(c) <= 600000
    _check_knn_and_accumulate(oracle, pool, cuda, 64, c, f, rs)


def test_config3_gravnet_stack(cuda, oracle, pool):
    """GravNet-style stack on one 200k-hit event: 4 x (dense 64->4 coordinates, BinnedSelectKnn K=64,
    AccumulateKnn mean+max over F=64, dense 192->64 + ReLU).  The dense layers run in torch on both
    sides' behalf; each block's ops are compared on identical op inputs."""
    from hgcalml_b200.binned_select_knn_op import BinnedSelectKnn
    from hgcalml_b200.accknn_op import AccumulateKnn
    n, K, F = 200000, 64, 64
    rs = np.array([0, n], np.int32)
    x = torch.as_tensor(np.random.default_rng(300).standard_normal((n, F), dtype=np.float32), device=cuda)
    rst = T(rs, cuda)
    for block in range(4):
        wc, wo = synth.gravnet_weights(block)
        coords = (x @ T(wc, cuda)).contiguous()
        gi, gd, sorting = BinnedSelectKnn(K, coords, rst, return_sorting=True)
        go, _ = AccumulateKnn(gd, x, gi, order=sorting, distance_scale=10.)
        # checker on the very same op inputs
        cn, xn = N(coords), N(x)
        ri, rd, ro, _ = oracle.knn_accumulate_path(K, cn, xn, rs, n_threads=N_THREADS, pool=pool, return_all=True)
        ties = assert_knn_equal(N(gi), N(gd), ri, rd, what=f"block {block}")
        assert ties <= 5
        tol = exp_weighted_tolerance(np.float32(10.) * rd, xn, ri, ro)
        ok_rows = (np.sort(N(gi), axis=1) == np.sort(ri, axis=1)).all(axis=1)
        assert (np.abs(N(go) - ro) <= tol)[ok_rows].all()
        x = torch.relu(torch.cat([x, go], dim=1) @ T(wo, cuda)).contiguous()
    assert torch.isfinite(x).all()


@pytest.mark.parametrize("amb", [True, False])
def test_config4_condensates_4x200k(cuda, oracle, amb):
    """Four events of 200k hits, 500 Gaussian blobs each, beta ~ Beta(0.5,5) with promoted seeds,
    t_b = 0.1, t_d = 0.5: all outputs identical to the checker."""
    from hgcalml_b200.assign_condensate_op import BuildAndAssignCondensatesBinned
    cc, beta, rs = synth.condensation_batch(4, 200000, 500, 3, 0.1, seed=400)
    d = np.full_like(beta, 0.5)
    ref = oracle.BuildAndAssignCondensatesBinned(cc, beta, d, rs, 0.1, assign_by_max_beta=amb)
    got = BuildAndAssignCondensatesBinned(T(cc, cuda), T(beta, cuda), T(d, cuda), T(rs, cuda), 0.1,
                                          assign_by_max_beta=amb)
    for r, g, key in zip(ref, got, COND_KEYS):
        assert np.array_equal(N(g), r), key
    assert 4 * 300 < ref[4][-1] < 4 * 700


def test_sharded_batch_equals_whole_batch_on_gpu(cuda):
    """The multi-GPU split, on the library itself: BinnedSelectKnn + AccumulateKnn on the two shards
    of ``shard_events(rs, 2)`` (each with its own binning grid, as on two ranks) against one call
    over the whole batch.  Neighbour rows must be identical in canonical order with bit-identical
    distances; the accumulated features agree within 1e-5 of the summed terms (rows of a shard are
    summed in the same slot order unless an exact distance tie reorders two slots)."""
    from hgcalml_b200.binned_select_knn_op import BinnedSelectKnn
    from hgcalml_b200.accknn_op import AccumulateKnn
    from hgcalml_b200.sharding import shard_events, local_row_splits, merge_indices
    K = 32
    c, f, rs = synth.shower_batch([30000, 500, 0, 42000, 20, 17000, 26000], dims=4, n_feat=16, seed=61)
    wi, wd, wsort = BinnedSelectKnn(K, T(c, cuda), T(rs, cuda), return_sorting=True)
    wo, _ = AccumulateKnn(wd, T(f, cuda), wi, order=wsort, distance_scale=10.)
    parts_i, parts_d, parts_o = [], [], []
    shards = shard_events(rs, 2)
    assert all(b > a for a, b in shards)
    for a, b in shards:
        lrs, off = local_row_splits(rs, a, b)
        n_local = int(lrs[-1])
        li, ld, lsort = BinnedSelectKnn(K, T(c[off:off + n_local], cuda), T(lrs, cuda), return_sorting=True)
        lo, _ = AccumulateKnn(ld, T(f[off:off + n_local], cuda), li, order=lsort, distance_scale=10.)
        parts_i.append(merge_indices(N(li), off))
        parts_d.append(N(ld))
        parts_o.append(N(lo))
    si, sd = np.concatenate(parts_i), np.concatenate(parts_d)
    # rows may differ only where candidates tie exactly at the K-th distance (none expected here)
    assert assert_knn_equal(si, sd, N(wi), N(wd), what="shards vs whole batch") <= 2
    same_rows = (np.sort(si, axis=1) == np.sort(N(wi), axis=1)).all(axis=1)
    got, want = np.concatenate(parts_o), N(wo)
    tol = exp_weighted_tolerance(np.float32(10.) * N(wd), f, N(wi), want)
    assert (np.abs(got - want) <= tol)[same_rows].all()
    # the max does not depend on slot order
    assert np.array_equal(bits(got[same_rows, 16:]), bits(want[same_rows, 16:]))
