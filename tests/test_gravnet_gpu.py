"""GPU parity of the GravNet layers' collection step (hgc_gravnet_collect) and of the two layer mirrors
against the checker's restatement of modules/GravNetLayersRagged.py."""
import numpy as np
import pytest
import torch

from conftest import load_golden, assert_knn_equal
from hgcalml_b200 import synth
from test_ops_gpu import T, N, exp_weighted_tolerance

pytestmark = pytest.mark.gpu


def collect_tolerance(feats, idx, dist):
    """Tolerance of the collected [mean - own | max - own]: that of the exp-weighted accumulation
    (1e-5 of the summed terms) -- the subtraction adds one rounding of a number of that size."""
    d = np.float32(10.) * dist
    w = np.exp(-d).astype(np.float32)
    nb = np.where(idx < 0, 0, idx)
    terms = feats[nb] * w[:, :, None] * (idx >= 0)[:, :, None]
    ref = np.concatenate([terms.sum(axis=1) / np.float32(idx.shape[1]), terms.max(axis=1)], axis=1)
    tol = exp_weighted_tolerance(d, feats, idx, ref)
    return tol + 1e-5 * np.abs(np.tile(feats, [1, 2]))


@pytest.mark.parametrize("name", ["showers4d", "showers4d_tfcompat", "uniform3d"])
def test_gravnet_collect_golden(cuda, name):
    from hgcalml_b200.GravNetLayersRagged import collect_neighbours
    g = load_golden("gravnet_collect_" + name)
    feats, idx, dist = g["feats"], g["idx"], g["dist"]
    got, _ = collect_neighbours(T(feats, cuda), T(idx, cuda), T(dist, cuda), first_slot=1, subtract_self=True)
    tol = collect_tolerance(feats, idx[:, 1:], dist[:, 1:])
    assert (np.abs(N(got) - g["collected"]) <= tol).all()


@pytest.mark.parametrize("f,k,width,col", [(64, 64, 200, 8), (12, 9, 40, 5), (32, 16, 64, 0), (6, 5, 12, 0)])
def test_gravnet_collect_equals_separate_steps(cuda, f, k, width, col):
    """Slice + scale + AccumulateKnn + subtraction + placement as separate tensor ops give bit-identical
    results to the one call (vector and scalar kernels, aligned and unaligned target columns)."""
    from hgcalml_b200.GravNetLayersRagged import collect_neighbours
    from hgcalml_b200.accknn_op import AccumulateKnn
    from hgcalml_b200.binned_select_knn_op import BinnedSelectKnn
    c, feats, rs = synth.shower_batch([900, 3, 0, 2000], dims=4, n_feat=f, seed=60 + f)
    idx, dist, sorting = BinnedSelectKnn(k + 1, T(c, cuda), T(rs, cuda), return_sorting=True)
    ft = T(feats, cuda)
    sep, sep_arg = AccumulateKnn(10. * dist[:, 1:].contiguous(), ft, idx[:, 1:].contiguous())
    sep = sep - ft.repeat(1, 2)
    buf = torch.full((len(c), width), 7., device=cuda)
    view, arg = collect_neighbours(ft, idx, dist, first_slot=1, subtract_self=True, out=buf, out_column=col,
                                   order=sorting, with_max_idxs=True)
    assert torch.equal(view, sep) and torch.equal(buf[:, col:col + 2 * f], sep)
    assert torch.equal(arg, sep_arg)
    untouched = torch.ones(width, dtype=torch.bool)
    untouched[col:col + 2 * f] = False
    assert (buf[:, untouched] == 7.).all()


def _torch_dense(dev):
    """Dense layers for the checker evaluated by the same library GEMM the modules use, so that the
    comparison is about the ops between them."""
    def dense(x, weights, activation):
        y = T(x, dev) @ T(weights[0], dev)
        if len(weights) > 1:
            y = y + T(weights[1], dev)
        if activation == "relu":
            y = torch.relu(y)
        elif activation is not None:
            raise ValueError(activation)
        return N(y)
    return dense


@pytest.mark.parametrize("return_self", [True, False])
def test_ragged_gravnet_layer_vs_checker(cuda, oracle, return_self):
    from hgcalml_b200.GravNetLayersRagged import RaggedGravNet
    _, x, rs = synth.shower_batch([2500, 40, 0, 4000], dims=4, n_feat=32, seed=71)
    rng = np.random.default_rng(72)
    K, S, P, FO = 24, 4, 16, 48
    w = [[(rng.standard_normal((32, P)) / 6).astype(np.float32), rng.standard_normal(P).astype(np.float32) / 10],
         [(rng.standard_normal((32, S)) / 6).astype(np.float32)],
         [(rng.standard_normal((2 * P + 32, FO)) / 8).astype(np.float32), rng.standard_normal(FO).astype(np.float32) / 10]]
    layer = RaggedGravNet(K, S, FO, P, n_in=32, return_self=return_self).to(cuda)
    layer.input_feature_transform.set_weights(w[0])
    layer.input_spatial_transform.set_weights(w[1])
    layer.output_feature_transform.set_weights(w[2])
    with torch.no_grad():
        out, coords, idx, dist = layer([T(x, cuda), T(rs, cuda)])
    ro, rc, ri, rd = oracle.RaggedGravNet(x, rs, w, K, return_self=return_self, dense=_torch_dense(cuda))
    assert np.array_equal(N(coords), rc)
    assert N(idx).shape == ri.shape == (len(x), K + 1 if return_self else K)
    if return_self:
        ties = assert_knn_equal(N(idx), N(dist), ri, rd, what="RaggedGravNet")
        assert ties <= 2
    # output features: rows whose neighbour sets agree, at the accumulated tolerance carried through
    # the last dense layer (|W| columns sum the per-input tolerances)
    same = (np.sort(N(idx), axis=1) == np.sort(ri, axis=1)).all(axis=1)
    assert same.mean() > 0.999
    feats = _torch_dense(cuda)(x, w[0], "relu")
    full_i, full_d = (ri, rd) if return_self else (None, None)
    if full_i is None:
        _, _, full_i, full_d = oracle.RaggedGravNet(x, rs, w, K, return_self=True, dense=_torch_dense(cuda))
    tol_in = collect_tolerance(feats, full_i[:, 1:], full_d[:, 1:])
    tol_out = tol_in @ np.abs(w[2][0][:2 * P]) + 1e-5 * np.abs(ro) + 1e-6
    assert (np.abs(N(out) - ro) <= tol_out)[same].all()


def test_distance_weighted_message_passing_vs_checker(cuda, oracle):
    from hgcalml_b200.GravNetLayersRagged import DistanceWeightedMessagePassing
    from hgcalml_b200.binned_select_knn_op import BinnedSelectKnn
    c, x, rs = synth.shower_batch([3000, 0, 1500], dims=3, n_feat=20, seed=81)
    rng = np.random.default_rng(82)
    nft = [16, 16, 8]
    widths = [20, 32, 32]
    w = [[(rng.standard_normal((wi, fo)) / np.sqrt(wi)).astype(np.float32),
          (rng.standard_normal(fo) / 10).astype(np.float32)] for wi, fo in zip(widths, nft)]
    idx, dist, sorting = BinnedSelectKnn(17, T(c, cuda), T(rs, cuda), return_sorting=True)
    nidx, ndist = idx[:, 1:].contiguous(), dist[:, 1:].contiguous()
    layer = DistanceWeightedMessagePassing(nft, n_in=20).to(cuda)
    for d, wi in zip(layer.feature_tranformation_dense, w):
        d.set_weights(wi)
    with torch.no_grad():
        got = N(layer([T(x, cuda), nidx, ndist], order=sorting))
    ref = oracle.DistanceWeightedMessagePassing(x, N(nidx), N(ndist), w, dense=_torch_dense(cuda))
    assert got.shape == ref.shape == (len(x), 2 * sum(nft) + 20)
    assert np.array_equal(got[:, 2 * sum(nft):], x)
    # pass 0 sees identical inputs on both sides: op-level tolerance; later passes inherit the
    # differences of the earlier ones through a dense layer, so they are checked at 1e-4 of the scale
    feats0 = _torch_dense(cuda)(x, w[0], "relu")
    tol0 = collect_tolerance(feats0, N(nidx), N(ndist))
    assert (np.abs(got[:, :32] - ref[:, :32]) <= tol0).all()
    scale = np.abs(ref[:, 32:80]).mean()
    assert np.abs(got[:, 32:80] - ref[:, 32:80]).max() <= 1e-4 * max(scale, 1.)
