"""GPU test of hgc_binned_select_knn_static, the BinnedSelectKnn entry for callers that cannot
provide device memory (a bare C job without an allocator, a server whose framework owns the GPU's
memory).  It must give exactly what the workspace-taking entry gives -- indices equal, distances
bit-identical -- also on a second call, which finds the built-in scratch full of the first call's
data; both must agree with the CPU checker; its status reader must report a clean run; and it must
refuse problems larger than that scratch.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test."""
import ctypes

import numpy as np
import pytest
import torch

from hgcalml_b200 import synth

pytestmark = pytest.mark.gpu


def _sorted_inputs(oracle, K, c, rs):
    nb0 = oracle.default_n_bins(int(rs[1]), K, 3)
    dbin, binning, nb, bw, nper = oracle.BinByCoordinates(c[:, :3], rs, n_bins=nb0)
    s = np.argsort(binning, kind="stable")
    bb = np.concatenate([[0], nper]).cumsum().astype(np.int32)
    return c[s], binning[s], dbin[s], bb, nb, bw


def _call_static(C, dev, K, sc, sb, sdb, bb, nb, bw, direction=None, tf_compat=False):
    t = [torch.as_tensor(np.ascontiguousarray(x), device=dev) for x in (sc, sb, sdb, bb, nb, bw)]
    d = None if direction is None else torch.as_tensor(np.ascontiguousarray(direction), device=dev)
    n, c = sc.shape
    idx = torch.full((n, K), -7, dtype=torch.int32, device=dev)
    dist = torch.full((n, K), -7., dtype=torch.float32, device=dev)
    rc = C.lib.hgc_binned_select_knn_static(
        C.ptr(t[0]), C.ptr(t[1]), C.ptr(d), C.ptr(t[2]), C.ptr(t[3]), C.ptr(t[4]), C.ptr(t[5]),
        C.ptr(idx), C.ptr(dist), n, K, c, len(nb), len(bb), int(tf_compat), int(d is not None),
        C.stream_of(idx))
    return rc, idx, dist


def _static_status(C, like):
    out = ctypes.c_uint(77)
    rc = C.lib.hgc_binned_select_knn_static_status(C.stream_of(like), ctypes.byref(out))
    return rc, out.value


def test_static_scratch_entry_matches_workspace_entry(cuda, oracle):
    from conftest import assert_knn_equal
    from hgcalml_b200 import _capi as C
    from hgcalml_b200.binned_select_knn_op import _BinnedSelectKnn
    # two different problems back to back: the second call meets the first call's leftovers
    for seed, sizes, K in ((3, [9000, 30, 4000], 24), (4, [2000, 6000], 40)):
        c, _, rs = synth.shower_batch(sizes, dims=4, n_feat=1, seed=seed)
        sc, sb, sdb, bb, nb, bw = _sorted_inputs(oracle, K, c, rs)
        rc, idx, dist = _call_static(C, cuda, K, sc, sb, sdb, bb, nb, bw)
        assert rc == 0, C.lib.hgc_strerror(rc)
        T = lambda a: torch.as_tensor(np.ascontiguousarray(a), device=cuda)  # noqa: E731
        ridx, rdist = _BinnedSelectKnn(K, T(sc), T(sb), T(sdb), T(bb), T(nb), T(bw))
        assert torch.equal(idx, ridx)
        assert torch.equal(dist.view(torch.int32), rdist.view(torch.int32))
        # ... and both against the CPU checker, so that an error common to the two entries shows
        ci, cd = oracle.op_binned_select_knn(K, sc, sb, sdb, bb, nb, bw)
        assert_knn_equal(idx.cpu().numpy(), dist.cpu().numpy(), ci, cd, what="static entry")
        assert _static_status(C, idx) == (0, 0)


def test_static_scratch_entry_direction_and_tf_compat(cuda, oracle):
    """The attributes of the op pass through the entry unchanged: direction codes and self-padding."""
    from conftest import assert_knn_equal
    from hgcalml_b200 import _capi as C
    K = 12
    c, _, rs = synth.shower_batch([3000, 7, 1500], dims=4, n_feat=1, seed=6)
    sc, sb, sdb, bb, nb, bw = _sorted_inputs(oracle, K, c, rs)
    direction = np.random.default_rng(2).integers(0, 4, sc.shape[0]).astype(np.int32)
    for kw in (dict(direction=direction), dict(tf_compat=True)):
        rc, idx, dist = _call_static(C, cuda, K, sc, sb, sdb, bb, nb, bw, **kw)
        assert rc == 0, C.lib.hgc_strerror(rc)
        ci, cd = oracle.op_binned_select_knn(K, sc, sb, sdb, bb, nb, bw, direction=kw.get("direction"),
                                             tf_compatible=kw.get("tf_compat", False))
        assert_knn_equal(idx.cpu().numpy(), dist.cpu().numpy(), ci, cd, what=f"static entry {sorted(kw)}")
        assert _static_status(C, idx) == (0, 0)


def test_static_scratch_status_reports_device_flags(cuda, oracle):
    """A bin table shorter than the bins the hits refer to makes the search flag a flat-bin overflow;
    the status reader of this entry must report it (and the call itself still returns)."""
    from hgcalml_b200 import _capi as C
    K = 8
    c, _, rs = synth.shower_batch([2000], dims=4, n_feat=1, seed=8)
    sc, sb, sdb, bb, nb, bw = _sorted_inputs(oracle, K, c, rs)
    short = bb[: len(bb) // 2].copy()
    rc, idx, dist = _call_static(C, cuda, K, sc, sb, sdb, short, nb, bw)
    assert rc == 0
    rc, status = _static_status(C, idx)
    assert rc == -5 and status & 2
    # a clean call afterwards starts from a cleared status word
    rc, idx, dist = _call_static(C, cuda, K, sc, sb, sdb, bb, nb, bw)
    assert rc == 0 and _static_status(C, idx) == (0, 0)


def test_static_scratch_entry_rejects_oversized_problems(cuda):
    from hgcalml_b200 import _capi as C
    nul = ctypes.c_void_p(None)
    too_many = 262144 + 1
    assert C.lib.hgc_binned_select_knn_static(nul, nul, nul, nul, nul, nul, nul, nul, nul,
                                              too_many, 8, 4, 3, 10, 0, 0, nul) == -6
    assert C.lib.hgc_binned_select_knn_static(nul, nul, nul, nul, nul, nul, nul, nul, nul,
                                              1000, 8, 5, 3, 10, 0, 0, nul) == -6
    assert b"scratch" in C.lib.hgc_strerror(-6)
