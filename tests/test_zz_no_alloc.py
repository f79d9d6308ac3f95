"""GPU test of hgc_binned_select_knn_static, the BinnedSelectKnn entry for callers that cannot
provide device memory (a bare C job without an allocator, a server whose framework owns the GPU's
memory).  It must give exactly what the workspace-taking entry gives -- indices equal, distances
bit-identical -- also on a second call, which finds the built-in scratch full of the first call's
data, and it must refuse problems larger than that scratch.

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


def _call_static(C, dev, K, sc, sb, sdb, bb, nb, bw):
    t = [torch.as_tensor(np.ascontiguousarray(x), device=dev) for x in (sc, sb, sdb, bb, nb, bw)]
    n, c = sc.shape
    idx = torch.full((n, K), -7, dtype=torch.int32, device=dev)
    dist = torch.full((n, K), -7., dtype=torch.float32, device=dev)
    rc = C.lib.hgc_binned_select_knn_static(
        C.ptr(t[0]), C.ptr(t[1]), None, C.ptr(t[2]), C.ptr(t[3]), C.ptr(t[4]), C.ptr(t[5]),
        C.ptr(idx), C.ptr(dist), n, K, c, len(nb), len(bb), 0, 0, C.stream_of(idx))
    return rc, idx, dist


def test_static_scratch_entry_matches_workspace_entry(cuda, oracle):
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


def test_static_scratch_entry_rejects_oversized_problems(cuda):
    from hgcalml_b200 import _capi as C
    nul = ctypes.c_void_p(None)
    too_many = 262144 + 1
    assert C.lib.hgc_binned_select_knn_static(nul, nul, nul, nul, nul, nul, nul, nul, nul,
                                              too_many, 8, 4, 3, 10, 0, 0, nul) == -6
    assert C.lib.hgc_binned_select_knn_static(nul, nul, nul, nul, nul, nul, nul, nul, nul,
                                              1000, 8, 5, 3, 10, 0, 0, nul) == -6
    assert b"scratch" in C.lib.hgc_strerror(-6)
