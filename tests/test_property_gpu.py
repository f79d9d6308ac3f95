"""Property-based GPU parity: random small ragged batches (duplicate points, events smaller than K,
empty events, any supported dimensionality) against the CPU checker."""
import os

import numpy as np
import pytest
import torch
from hypothesis import given, settings, strategies as st, HealthCheck

from conftest import bits, assert_knn_equal
from test_ops_gpu import T, N

pytestmark = pytest.mark.gpu

SETTINGS = dict(max_examples=int(os.environ.get("HGC_PROPERTY_EXAMPLES", "40")), deadline=None,
                suppress_health_check=[HealthCheck.function_scoped_fixture, HealthCheck.too_slow])


@st.composite
def ragged_points(draw):
    dims = draw(st.integers(2, 6))
    sizes = draw(st.lists(st.integers(0, 300), min_size=1, max_size=4))
    if sum(sizes) == 0:
        sizes[0] = 5
    seed = draw(st.integers(0, 2 ** 31 - 1))
    style = draw(st.sampled_from(["uniform", "clustered", "lattice", "identical"]))
    rng = np.random.default_rng(seed)
    n = sum(sizes)
    if style == "uniform":
        c = rng.random((n, dims), dtype=np.float32)
    elif style == "clustered":
        c = (rng.integers(0, 3, (n, dims)) + 0.01 * rng.standard_normal((n, dims))).astype(np.float32)
    elif style == "lattice":      # many exactly equal distances
        c = rng.integers(0, 4, (n, dims)).astype(np.float32)
    else:                          # every hit at the same place
        c = np.full((n, dims), 0.25, np.float32)
    rs = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int32)
    return c, rs, rng


@settings(**SETTINGS)
@given(data=ragged_points(), K=st.integers(1, 40), mbd=st.integers(2, 5), nb=st.sampled_from([None, 3, 7]),
       tf_compat=st.booleans())
def test_binned_select_knn_random(cuda, oracle, data, K, mbd, nb, tf_compat):
    from hgcalml_b200.binned_select_knn_op import BinnedSelectKnn
    c, rs, _ = data
    kw = dict(max_bin_dims=mbd, tf_compatible=tf_compat)
    if nb is not None:
        kw["n_bins"] = nb
    ri, rd = oracle.BinnedSelectKnn(K, c, rs, **kw)
    gi, gd = BinnedSelectKnn(K, T(c, cuda), T(rs, cuda), **kw)
    gi, gd = N(gi), N(gd)
    if tf_compat:
        own = (np.arange(K)[None] > 0)
        rows = np.arange(len(c))[:, None]
        ri = np.where((ri == rows) & own, -1, ri)
        gi = np.where((gi == rows) & own, -1, gi)
    # lattices and identical points tie everywhere: distances must still agree bit for bit and every
    # differing row must differ only among candidates at the row's largest kept distance
    assert_knn_equal(gi, gd, ri, rd, what="random")
    assert ((gi >= 0).sum(axis=1) == (ri >= 0).sum(axis=1)).all()


@settings(**SETTINGS)
@given(n=st.integers(1, 400), K=st.integers(1, 70), F=st.integers(1, 70), mm=st.booleans(),
       seed=st.integers(0, 2 ** 31 - 1), pad=st.booleans())
def test_accumulate_knn_random(cuda, oracle, n, K, F, mm, seed, pad):
    from hgcalml_b200.accknn_op import AccumulateLinKnn, AccumulateKnnGrad
    rng = np.random.default_rng(seed)
    feat = rng.standard_normal((n, F), dtype=np.float32)
    w = rng.random((n, K), dtype=np.float32)
    idx = rng.integers(0, n, (n, K)).astype(np.int32)
    if pad:
        idx[rng.random((n, K)) < 0.3] = -1
    ro, ra = oracle.op_accumulate_knn(w, feat, idx, mean_and_max=mm)
    go, ga = AccumulateLinKnn(T(w, cuda), T(feat, cuda), T(idx, cuda), mean_and_max=mm)
    assert np.array_equal(bits(N(go)), bits(ro))
    if mm:
        assert np.array_equal(N(ga), ra)
    g = rng.standard_normal(ro.shape).astype(np.float32)
    rw, rf = oracle.op_accumulate_knn_grad(g, w, feat, idx, ra)
    gw, gf = AccumulateKnnGrad(T(g, cuda), T(w, cuda), T(feat, cuda), T(idx, cuda), T(ra, cuda))
    assert np.array_equal(bits(N(gw)), bits(rw)) and np.array_equal(bits(N(gf)), bits(rf))


@settings(**SETTINGS)
@given(sizes=st.lists(st.integers(0, 400), min_size=1, max_size=4), dims=st.integers(1, 8),
       nbin_dims=st.integers(1, 4), seed=st.integers(0, 2 ** 31 - 1), amb=st.booleans(),
       beta_style=st.sampled_from(["continuous", "few_levels", "all_equal"]),
       mask_frac=st.sampled_from([0.0, 0.05, 0.6]), radius=st.sampled_from([0.05, 0.3, 2.0]),
       thr=st.sampled_from([1.0, 0.6]))
def test_condensates_one_call_random(cuda, oracle, sizes, dims, nbin_dims, seed, amb, beta_style, mask_frac,
                                     radius, thr):
    """Random small ragged batches with tied betas (the priority order then falls back on the position
    after the bin sort), masks of both signs, radii from tiny to covering everything: all five outputs
    identical to the checker."""
    from hgcalml_b200.assign_condensate_op import BuildAndAssignCondensatesBinned
    if sum(sizes) == 0:
        sizes = [7] + list(sizes[1:])
    n = sum(sizes)
    rng = np.random.default_rng(seed)
    cc = rng.random((n, dims), dtype=np.float32)
    if beta_style == "continuous":
        beta = rng.random((n, 1), dtype=np.float32)
    elif beta_style == "few_levels":
        beta = (rng.integers(0, 5, (n, 1)) / 4.).astype(np.float32)
    else:
        beta = np.full((n, 1), 0.5, np.float32)
    d = np.full((n, 1), radius, np.float32) * rng.uniform(0.5, 1.5, (n, 1)).astype(np.float32)
    mask = None
    if mask_frac > 0:
        mask = np.where(rng.random((n, 1)) < mask_frac, rng.integers(-1, 3, (n, 1)), 0).astype(np.int32)
    rs = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int32)
    kw = dict(distance_threshold=thr, assign_by_max_beta=amb, nbin_dims=nbin_dims)
    ref = oracle.BuildAndAssignCondensatesBinned(cc, beta, d, rs, 0.1, no_condensation_mask=mask, **kw)
    got = BuildAndAssignCondensatesBinned(T(cc, cuda), T(beta, cuda), T(d, cuda), T(rs, cuda), 0.1,
                                          no_condensation_mask=None if mask is None else T(mask, cuda), **kw)
    for r, g, key in zip(ref, got, ("assignment", "association", "alpha_idx", "is_cond", "n_condensates")):
        assert np.array_equal(N(g), r), key


@settings(**SETTINGS)
@given(n=st.integers(1, 300), K=st.integers(1, 40), F=st.integers(1, 40), first=st.integers(0, 2),
       seed=st.integers(0, 2 ** 31 - 1), pad=st.booleans(), sub=st.booleans(), col=st.integers(0, 5))
def test_gravnet_collect_random(cuda, n, K, F, first, seed, pad, sub, col):
    """The one-call collection step equals slice + scale + AccumulateKnn + subtraction + placement done
    with separate tensor ops, bit for bit, for any shape, slot offset and target column."""
    from hgcalml_b200.GravNetLayersRagged import collect_neighbours
    from hgcalml_b200.accknn_op import AccumulateKnn
    rng = np.random.default_rng(seed)
    feat = T(rng.standard_normal((n, F), dtype=np.float32), cuda)
    ld = first + K
    dist = T(rng.random((n, ld), dtype=np.float32), cuda)
    idx_np = rng.integers(0, n, (n, ld)).astype(np.int32)
    if pad:
        idx_np[rng.random((n, ld)) < 0.3] = -1
    idx = T(idx_np, cuda)
    sep, sep_arg = AccumulateKnn(10. * dist[:, first:].contiguous(), feat, idx[:, first:].contiguous())
    if sub:
        sep = sep - feat.repeat(1, 2)
    buf = torch.full((n, col + 2 * F + 3), 7., device=cuda)
    view, arg = collect_neighbours(feat, idx, dist, first_slot=first, subtract_self=sub, out=buf, out_column=col,
                                   with_max_idxs=True)
    assert torch.equal(view, sep) and torch.equal(arg, sep_arg)
    assert (buf[:, :col] == 7.).all() and (buf[:, col + 2 * F:] == 7.).all()
