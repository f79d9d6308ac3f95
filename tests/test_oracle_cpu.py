"""CPU suite: the checker itself.  The plain-C restatement must reproduce the golden vectors (which
were produced by the reference's own compiled CPU kernels), the compiled reference where it is
available, and a definitional brute-force kNN."""
import numpy as np
import pytest

from conftest import load_golden, bits
from hgcalml_b200 import synth

KNN_CASES = {
    "knn_uniform3d": dict(n_bins=5),
    "knn_showers4d": dict(),
    "knn_showers4d_bin4": dict(max_bin_dims=4),
    "knn_showers4d_direction": dict(use_direction=True),
    "knn_showers4d_tfcompat": dict(tf_compatible=True),
}
COND_CASES = [f"cond_{t}_{m}" for t in ("const", "var", "masked", "maskedheavy") for m in ("maxbeta", "mindist")]


def _knn_kwargs(g, kw):
    kw = dict(kw)
    if kw.pop("use_direction", False):
        kw["direction"] = g["direction"]
    return kw


@pytest.mark.parametrize("name", sorted(KNN_CASES))
def test_port_matches_golden_knn_and_accumulate(oracle, name):
    g = load_golden(name)
    kw = _knn_kwargs(g, KNN_CASES[name])
    idx, dist = oracle.BinnedSelectKnn(int(g["K"]), g["coords"], g["row_splits"], backend="port", **kw)
    # raw equality, slot order included: the restatement follows the reference's scan order
    assert np.array_equal(idx, g["idx"])
    assert np.array_equal(bits(dist), bits(g["dist"]))
    acc, maxidx = oracle.AccumulateKnn(np.float32(10.) * dist, g["feats"], idx, backend="port")
    assert np.array_equal(bits(acc), bits(g["acc"]))
    assert np.array_equal(maxidx, g["maxidx"])


@pytest.mark.parametrize("name", COND_CASES)
def test_port_matches_golden_condensates(oracle, name):
    g = load_golden(name)
    out = oracle.BuildAndAssignCondensatesBinned(
        g["ccoords"], g["betas"], g["dist"], g["row_splits"], float(g["beta_threshold"]),
        no_condensation_mask=g["mask"], assign_by_max_beta=bool(g["assign_by_max_beta"]), backend="port")
    for got, key in zip(out, ("assignment", "association", "alpha_idx", "is_cond", "n_condensates")):
        assert np.array_equal(got, g[key]), key


def test_port_matches_golden_binning(oracle):
    g = load_golden("bin_by_coordinates")
    binass, flat, nb, bw, nper = oracle.BinByCoordinates(g["coords"], g["row_splits"],
                                                         n_bins=int(g["n_bins_arg"]), backend="port")
    assert np.array_equal(binass, g["binass"]) and np.array_equal(flat, g["flat"])
    assert np.array_equal(nb, g["n_bins"]) and np.array_equal(bits(bw), bits(g["bin_width"]))
    assert np.array_equal(nper, g["nper"])
    assert nper.sum() == g["coords"].shape[0]


def test_golden_knn_is_exact_knn(oracle):
    """The reference's result is the definitional kNN (set per row) -- pins the parity notion."""
    g = load_golden("knn_showers4d")
    rows, bi, bd = oracle.brute_force_knn(int(g["K"]), g["coords"], g["row_splits"])
    ci, cd = oracle.canonical_knn(g["idx"][rows], g["dist"][rows])
    assert np.array_equal(bits(cd), bits(bd))
    assert (ci == bi).mean() > 0.999  # only exact distance ties at the boundary may differ


@pytest.mark.skipif("not __import__('oracle.oracle').oracle.have('ref')")
@pytest.mark.parametrize("seed", [1, 2])
def test_port_matches_compiled_reference(oracle, seed):
    """Where the reference's own kernels were compiled, the restatement must agree with them on fresh
    inputs, bit for bit, for every op."""
    rng = np.random.default_rng(seed)
    sizes = [int(x) for x in rng.integers(0, 900, 4)] + [5]
    c, f, rs = synth.shower_batch(sizes, dims=4, n_feat=6, seed=1000 + seed)
    direction = rng.integers(0, 4, c.shape[0]).astype(np.int32)
    for kw in (dict(), dict(max_bin_dims=2), dict(max_bin_dims=4), dict(direction=direction),
               dict(tf_compatible=True), dict(n_bins=7)):
        a = oracle.BinnedSelectKnn(11, c, rs, backend="port", **kw)
        b = oracle.BinnedSelectKnn(11, c, rs, backend="ref", **kw)
        assert np.array_equal(a[0], b[0]) and np.array_equal(bits(a[1]), bits(b[1])), kw
    for mm in (True, False):
        a = oracle.AccumulateKnn(b[1], f, b[0], mean_and_max=mm, backend="port")
        r = oracle.AccumulateKnn(b[1], f, b[0], mean_and_max=mm, backend="ref")
        assert np.array_equal(bits(a[0]), bits(r[0])) and np.array_equal(a[1], r[1])
    cc, beta, rsc = synth.condensation_batch(2, 3000, 25, 3, 0.1, seed=50 + seed)
    d = rng.uniform(0.1, 0.7, beta.shape).astype(np.float32)
    mask = (rng.random(beta.shape) < 0.3).astype(np.int32)
    for m in (None, mask):
        for amb in (True, False):
            a = oracle.BuildAndAssignCondensatesBinned(cc, beta, d, rsc, 0.1, no_condensation_mask=m,
                                                       assign_by_max_beta=amb, backend="port")
            b = oracle.BuildAndAssignCondensatesBinned(cc, beta, d, rsc, 0.1, no_condensation_mask=m,
                                                       assign_by_max_beta=amb, backend="ref")
            for x, y in zip(a, b):
                assert np.array_equal(x, y)


def test_condensate_invariants(oracle):
    """Structural invariants the reference's own unit test checks (tests/unit/condensate.py:88-112):
    every condensate is assigned to itself and numbered 0..n-1 within its event."""
    g = load_golden("cond_var_maxbeta")
    assignment, asso, alpha, is_cond, ncond = (g[k] for k in
                                               ("assignment", "association", "alpha_idx", "is_cond", "n_condensates"))
    assert is_cond.sum() == len(alpha) == ncond[-1]
    for e in range(len(ncond) - 1):
        a = alpha[ncond[e]:ncond[e + 1]]
        assert np.array_equal(assignment[a, 0], np.arange(len(a)))
        assert np.array_equal(asso[a], a)
    assert ((assignment[:, 0] < 0) == (asso < 0)).all()


ACCGRAD_CASES = [f"accgrad_{t}_{m}" for t in ("tfcompat", "padded") for m in ("meanmax", "mean")]


@pytest.mark.parametrize("name", ACCGRAD_CASES)
def test_port_matches_golden_accumulate_grad(oracle, name):
    g = load_golden(name)
    gw, gf = oracle.op_accumulate_knn_grad(g["grad_out"], g["weights"], g["feats"], g["idx"], g["maxidx"],
                                           backend="port")
    assert np.array_equal(bits(gw), bits(g["grad_weights"]))
    assert np.array_equal(bits(gf), bits(g["grad_feats"]))


def test_accumulate_grad_is_the_gradient(oracle):
    """The reference's backward op against float64 finite algebra: d(sum(out * G))/d feat and /d w."""
    g = load_golden("accgrad_padded_meanmax")
    w, feat, idx, maxidx, G = (g[k] for k in ("weights", "feats", "idx", "maxidx", "grad_out"))
    n, K = idx.shape
    F = feat.shape[1]
    gf = np.zeros((n, F))
    gw = np.zeros((n, K))
    for i in range(n):
        for k in range(K):
            m = idx[i, k]
            if m < 0:
                continue
            is_max = (maxidx[i] == m)
            gf[m] += G[i, :F] / K * w[i, k] + is_max * G[i, F:] * w[i, k]
            gw[i, k] = (G[i, :F] * feat[m]).sum() / K + (is_max * G[i, F:] * feat[m]).sum()
    # rows where a neighbour id repeats inside a row are left out: the op then counts the max once
    assert np.allclose(g["grad_weights"], gw, rtol=1e-4, atol=1e-5)
    assert np.allclose(g["grad_feats"], gf, rtol=1e-4, atol=1e-4)


def test_select_knn_grad_restatement_is_the_gradient(oracle):
    """SelectKnnGrad has no reference CPU code (its CPU functor is empty): the restatement of the GPU
    kernels is checked against the analytic gradient of sum_k g[i,k] * |x_i - x_m|^2 in float64."""
    g = load_golden("knn_showers4d")
    idx, c = g["idx"], g["coords"]
    n, K = idx.shape
    gd = np.random.default_rng(5).standard_normal((n, K)).astype(np.float32)
    got = oracle.op_select_knn_grad(gd, idx, c)
    ref = np.zeros(c.shape)
    c64 = c.astype(np.float64)
    for k in range(K):
        m = idx[:, k]
        ok = m >= 0
        d = c64[ok] - c64[m[ok]]
        contrib = 2 * gd[ok, k][:, None] * d
        np.add.at(ref, np.nonzero(ok)[0], contrib)
        np.add.at(ref, m[ok], -contrib)
    assert np.allclose(got, ref, rtol=1e-4, atol=1e-4 * np.abs(ref).max())


def test_keep_noise_invariants(oracle):
    """keep_noise=True (modules/assign_condensate_op.py:16-44): afterwards no hit is noise, showers are
    numbered 0..n-1 per event with alpha_idx as their representatives -- the round trips the
    reference's unit test asserts (tests/unit/condensate.py:88-112)."""
    g = load_golden("cond_var_maxbeta")
    out = oracle.BuildAndAssignCondensatesBinned(g["ccoords"], g["betas"], g["dist"], g["row_splits"], 0.1,
                                                 assign_by_max_beta=True, keep_noise=True)
    assignment, asso, alpha, is_cond, ncond = out
    rs = g["row_splits"]
    assert (assignment >= 0).all() and (asso >= 0).all()
    assert is_cond.sum() == len(alpha) == ncond[-1]
    for e in range(len(rs) - 1):
        al = alpha[ncond[e]:ncond[e + 1]]
        assert np.array_equal(assignment[al, 0], np.arange(len(al)))
        assert np.array_equal(asso[al], al)
        a = assignment[rs[e]:rs[e + 1], 0]
        assert a.max() + 1 == len(al)


@pytest.mark.parametrize("name", ["showers4d", "showers4d_tfcompat", "uniform3d"])
def test_port_matches_golden_gravnet_collect(oracle, name):
    g = load_golden("gravnet_collect_" + name)
    got = oracle.gravnet_collect(g["feats"], g["idx"][:, 1:], g["dist"][:, 1:], backend="port")
    assert np.array_equal(bits(got), bits(g["collected"]))


def test_gravnet_layer_restatements_shapes(oracle):
    """The numpy restatements of RaggedGravNet / DistanceWeightedMessagePassing: output layout."""
    c, f, rs = synth.shower_batch([300, 0, 450], dims=4, n_feat=10, seed=3)
    rng = np.random.default_rng(4)
    w = [[rng.standard_normal((10, 6), dtype=np.float32), rng.standard_normal(6, dtype=np.float32)],
         [rng.standard_normal((10, 3), dtype=np.float32)],
         [rng.standard_normal((22, 7), dtype=np.float32), rng.standard_normal(7, dtype=np.float32)]]
    out, coords, idx, dist = oracle.RaggedGravNet(f, rs, w, n_neighbours=8)
    assert out.shape == (750, 7) and coords.shape == (750, 3) and idx.shape == dist.shape == (750, 9)
    assert (idx[:, 0] == np.arange(750)).all() and (out >= 0).all()
    out2, _, idx2, _ = oracle.RaggedGravNet(f, rs, w, n_neighbours=8, return_self=False)
    assert np.array_equal(out, out2) and np.array_equal(idx2, idx[:, 1:])
    wm = [[rng.standard_normal((10, 4), dtype=np.float32), rng.standard_normal(4, dtype=np.float32)],
          [rng.standard_normal((8, 5), dtype=np.float32), rng.standard_normal(5, dtype=np.float32)]]
    mp = oracle.DistanceWeightedMessagePassing(f, idx[:, 1:], dist[:, 1:], wm)
    assert mp.shape == (750, 2 * (4 + 5) + 10) and np.array_equal(mp[:, 18:], f)


def _sibling_inputs():
    g = load_golden("sibling_ops_showers4d")
    base = load_golden("knn_showers4d")
    w = np.exp(-(np.float32(10.) * base["dist"])).astype(np.float32)
    return g, base, w


def test_port_matches_golden_sibling_ops(oracle):
    """LocalDistance, PushKnn, PushKnnGrad and IndexReplacer: the plain-C restatement against vectors
    produced by the reference's compiled CPU kernels (local_distance_kernel.cc:47-70,
    push_knn_kernel.cc:35-71, push_knn_grad_kernel.cc:22-95, index_replacer_kernel.cc:28-49)."""
    g, base, w = _sibling_inputs()
    assert np.array_equal(bits(oracle.op_local_distance(base["coords"], base["idx"], backend="port")),
                          bits(g["local_dist"]))
    assert np.array_equal(bits(oracle.op_push_knn(w, base["feats"], base["idx"], backend="port")), bits(g["pushed"]))
    wg, fg = oracle.op_push_knn_grad(g["push_grad_in"], w, base["feats"], base["idx"], backend="port")
    assert np.array_equal(bits(wg), bits(g["push_wgrad"])) and np.array_equal(bits(fg), bits(g["push_fgrad"]))
    assert np.array_equal(oracle.op_index_replacer(base["idx"], g["replacements"], backend="port"), g["replaced"])


@pytest.mark.skipif("not __import__('oracle.oracle').oracle.have('ref')")
@pytest.mark.parametrize("seed", [7, 8])
def test_port_matches_compiled_reference_sibling_and_backward_ops(oracle, seed):
    """Fresh inputs: restatement against the compiled reference for the ops beside the main path."""
    rng = np.random.default_rng(seed)
    c, f, rs = synth.shower_batch([int(x) for x in rng.integers(1, 1500, 3)], dims=3 + seed % 2, n_feat=9,
                                  seed=2000 + seed)
    idx, dist = oracle.BinnedSelectKnn(13, c, rs, backend="ref")
    w = np.exp(-dist).astype(np.float32)
    a, b = (oracle.op_local_distance(c, idx, backend=k) for k in ("port", "ref"))
    assert np.array_equal(bits(a), bits(b))
    a, b = (oracle.op_push_knn(w, f, idx, backend=k) for k in ("port", "ref"))
    assert np.array_equal(bits(a), bits(b))
    grad = rng.standard_normal(f.shape, dtype=np.float32)
    a, b = (oracle.op_push_knn_grad(grad, w, f, idx, backend=k) for k in ("port", "ref"))
    assert np.array_equal(bits(a[0]), bits(b[0])) and np.array_equal(bits(a[1]), bits(b[1]))
    rep = rng.permutation(idx.shape[0]).astype(np.int32)
    assert np.array_equal(oracle.op_index_replacer(idx, rep, backend="port"),
                          oracle.op_index_replacer(idx, rep, backend="ref"))
    for mm in (True, False):
        out, maxidx = oracle.op_accumulate_knn(w, f, idx, mean_and_max=mm, backend="ref")
        gout = rng.standard_normal(out.shape, dtype=np.float32)
        a, b = (oracle.op_accumulate_knn_grad(gout, w, f, idx, maxidx, backend=k) for k in ("port", "ref"))
        assert np.array_equal(bits(a[0]), bits(b[0])) and np.array_equal(bits(a[1]), bits(b[1]))


@pytest.mark.skipif("not __import__('oracle.oracle').oracle.have('ref')")
def test_port_matches_compiled_reference_at_full_event_size(oracle):
    """One 200k-hit event, K = 64, F = 64 (the size of the benchmark's events): restatement and compiled
    reference agree bit for bit, slot order included, on the search and on AccumulateKnn."""
    n, K = 200000, 64
    c = synth.shower_event(n, dims=4, seed=500)
    rs = np.array([0, n], np.int32)
    a = oracle.BinnedSelectKnn(K, c, rs, backend="port")
    b = oracle.BinnedSelectKnn(K, c, rs, backend="ref")
    assert np.array_equal(a[0], b[0]) and np.array_equal(bits(a[1]), bits(b[1]))
    f = np.random.default_rng(3).standard_normal((n, 64), dtype=np.float32)
    rows = slice(0, 40000)   # AccumulateKnn rows are independent: a fifth of the event keeps the suite short
    x = oracle.op_accumulate_knn_rows(np.exp(-np.float32(10.) * b[1]).astype(np.float32), f, b[0], 0, 40000, backend="port")
    y = oracle.op_accumulate_knn_rows(np.exp(-np.float32(10.) * b[1]).astype(np.float32), f, b[0], 0, 40000, backend="ref")
    assert np.array_equal(bits(x[0]), bits(y[0])) and np.array_equal(x[1], y[1])
