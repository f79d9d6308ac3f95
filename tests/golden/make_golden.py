"""Generates the golden vectors in this directory from the REFERENCE's own CPU kernels.

Run in a container that has a cms-pepr/HGCalML checkout (see oracle/Makefile: ``make -C oracle ref``
builds oracle/_ref/libref.so from it).  The op arithmetic in the stored outputs is the reference's
compiled code; only the TensorFlow glue of its Python wrappers is restated in numpy
(oracle/oracle.py).  Inputs are seeded synthetic data.

    python tests/golden/make_golden.py            # every fixture
    python tests/golden/make_golden.py siblings   # only the LocalDistance / PushKnn / IndexReplacer fixture
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402
from hgcalml_b200 import synth  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))
BACKEND = "ref"


def knn_case(name, K, coords, feats, row_splits, **kw):
    idx, dist = O.BinnedSelectKnn(K, coords, row_splits, backend=BACKEND, **kw)
    acc, maxidx = O.AccumulateKnn(np.float32(10.) * dist, feats, idx, backend=BACKEND)
    extra = {k: np.asarray(v) for k, v in kw.items() if v is not None}
    np.savez_compressed(os.path.join(OUT, name + ".npz"), K=np.int32(K), coords=coords, feats=feats,
                        row_splits=row_splits, idx=idx, dist=dist, acc=acc, maxidx=maxidx, **extra)
    print(name, coords.shape, "K", K, "rows with padding", int((idx < 0).any(axis=1).sum()))


def sibling_cases():
    """LocalDistance, PushKnn, PushKnnGrad and IndexReplacer on the neighbour rows of a golden kNN case
    (rows with -1 padding included)."""
    base = "knn_showers4d"
    case = dict(np.load(os.path.join(OUT, base + ".npz")))
    idx, feats, coords = case["idx"], case["feats"], case["coords"]
    rng = np.random.default_rng(13)
    w = np.exp(-(np.float32(10.) * case["dist"])).astype(np.float32)
    local_dist = O.op_local_distance(coords, idx, backend=BACKEND)
    pushed = O.op_push_knn(w, feats, idx, backend=BACKEND)
    grad = rng.standard_normal(feats.shape, dtype=np.float32)
    push_wgrad, push_fgrad = O.op_push_knn_grad(grad, w, feats, idx, backend=BACKEND)
    replacements = rng.permutation(idx.shape[0]).astype(np.int32)
    replaced = O.op_index_replacer(idx, replacements, backend=BACKEND)
    np.savez_compressed(os.path.join(OUT, "sibling_ops_showers4d.npz"), base=np.array(base),  # weights = exp(-10 dist)
                        local_dist=local_dist, pushed=pushed, push_grad_in=grad, push_wgrad=push_wgrad,
                        push_fgrad=push_fgrad, replacements=replacements, replaced=replaced)
    print("sibling ops", local_dist.shape, pushed.shape, push_wgrad.shape, replaced.shape)


def main():
    assert O.have("ref"), "build oracle/_ref/libref.so first (make -C oracle ref)"
    if sys.argv[1:] == ["siblings"]:
        sibling_cases()
        return
    # uniform 3-D event, explicit number of bins (small sibling of the 20k-hit CPU configuration)
    c, f, rs = synth.uniform_event(1500, 3, 8, seed=101)
    knn_case("knn_uniform3d", 16, c, f, rs, n_bins=5)
    # ragged shower batch in 4-D incl. an empty event and events smaller than K
    c, f, rs = synth.shower_batch([700, 9, 0, 1100, 30], dims=4, n_feat=12, seed=210)
    knn_case("knn_showers4d", 24, c, f, rs)
    knn_case("knn_showers4d_bin4", 24, c, f, rs, max_bin_dims=4)
    direction = np.random.default_rng(5).integers(0, 4, c.shape[0]).astype(np.int32)
    knn_case("knn_showers4d_direction", 10, c, f, rs, direction=direction)
    knn_case("knn_showers4d_tfcompat", 40, c, f, rs, tf_compatible=True)

    # condensates: two events of blobs, both assignment modes, and a masked variant
    cc, beta, rs = synth.condensation_batch(2, 2500, 30, 3, 0.1, seed=400)
    dist = np.full_like(beta, 0.5)
    rng = np.random.default_rng(9)
    dist_var = rng.uniform(0.2, 0.8, beta.shape).astype(np.float32)
    mask = (rng.random(beta.shape) < 0.01).astype(np.int32)
    mask_heavy = (rng.random(beta.shape) < 0.5).astype(np.int32)  # sets mask_h[0] / mask_h[1] as well
    for tag, d, m in (("const", dist, None), ("var", dist_var, None), ("masked", dist_var, mask),
                      ("maskedheavy", dist_var, mask_heavy)):
        for amb in (True, False):
            out = O.BuildAndAssignCondensatesBinned(cc, beta, d, rs, 0.1, no_condensation_mask=m,
                                                    assign_by_max_beta=amb, backend=BACKEND)
            name = f"cond_{tag}_{'maxbeta' if amb else 'mindist'}"
            np.savez_compressed(os.path.join(OUT, name + ".npz"), ccoords=cc, betas=beta, dist=d,
                                row_splits=rs, mask=np.zeros_like(beta, dtype=np.int32) if m is None else m,
                                beta_threshold=np.float32(0.1), assign_by_max_beta=np.int32(amb),
                                assignment=out[0], association=out[1], alpha_idx=out[2],
                                is_cond=out[3], n_condensates=out[4])
            print(name, "condensates", out[4].tolist(), "noise", int((out[0] < 0).sum()))

    # AccumulateKnnGrad on the neighbour rows of a golden kNN case (padding and repeated self included)
    g = dict(np.load(os.path.join(OUT, "knn_showers4d_tfcompat.npz")))
    g2 = dict(np.load(os.path.join(OUT, "knn_showers4d.npz")))
    for tag, case, base in (("tfcompat", g, "knn_showers4d_tfcompat"), ("padded", g2, "knn_showers4d")):
        w = np.exp(-(np.float32(10.) * case["dist"])).astype(np.float32)
        rng = np.random.default_rng(11)
        for mm in (True, False):
            out, maxidx = O.op_accumulate_knn(w, case["feats"], case["idx"], mean_and_max=mm, backend=BACKEND)
            grad_out = rng.standard_normal(out.shape, dtype=np.float32)
            gw, gf = O.op_accumulate_knn_grad(grad_out, w, case["feats"], case["idx"], maxidx, backend=BACKEND)
            name = f"accgrad_{tag}_{'meanmax' if mm else 'mean'}"
            # features and neighbour indices are those of the base case file
            np.savez_compressed(os.path.join(OUT, name + ".npz"), base=np.array(base), weights=w,
                                maxidx=maxidx, grad_out=grad_out, grad_weights=gw, grad_feats=gf)
            print(name, gw.shape, gf.shape)

    # the GravNet layers' collection step on the neighbour rows of two golden kNN cases: self slot
    # sliced off, AccumulateKnn(10 d^2), own features subtracted (modules/GravNetLayersRagged.py:3199-3202)
    for base in ("knn_showers4d", "knn_showers4d_tfcompat", "knn_uniform3d"):
        case = dict(np.load(os.path.join(OUT, base + ".npz")))
        collected = O.gravnet_collect(case["feats"], case["idx"][:, 1:], case["dist"][:, 1:], backend=BACKEND)
        np.savez_compressed(os.path.join(OUT, "gravnet_collect_" + base[4:] + ".npz"), base=np.array(base),
                            collected=collected)
        print("gravnet_collect", base, collected.shape)

    sibling_cases()

    # bin_by_coordinates op outputs
    c, _, rs = synth.shower_batch([400, 0, 650], dims=3, n_feat=1, seed=77)
    binass, flat, nb, bw, nper = O.BinByCoordinates(c, rs, n_bins=6, backend=BACKEND)
    np.savez_compressed(os.path.join(OUT, "bin_by_coordinates.npz"), coords=c, row_splits=rs,
                        n_bins_arg=np.int32(6), binass=binass, flat=flat, n_bins=nb, bin_width=bw, nper=nper)
    print("bin_by_coordinates", nb, bw)


if __name__ == "__main__":
    main()
