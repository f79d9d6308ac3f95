import functools
import inspect
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def load_golden(name):
    with np.load(os.path.join(GOLDEN, name + ".npz")) as z:
        g = {k: z[k] for k in z.files}
    if "base" in g:  # features / neighbour indices shared with another fixture
        base = load_golden(str(g.pop("base")))
        g.setdefault("feats", base["feats"])
        g.setdefault("idx", base["idx"])
        g.setdefault("dist", base["dist"])
    return g


class _Checker:
    """The checker module with a default back end: every routine that takes ``backend=`` gets the
    compiled reference (``oracle/_ref/libref.so``) where that library is present, else the plain-C
    restatement; a test that names a back end itself keeps it."""

    def __init__(self, module, backend):
        self._module = module
        self.backend = backend

    def __getattr__(self, name):
        attr = getattr(self._module, name)
        if callable(attr):
            try:
                takes_backend = "backend" in inspect.signature(attr).parameters
            except (TypeError, ValueError):
                takes_backend = False
            if takes_backend:
                return functools.partial(attr, backend=self.backend)
        return attr


@pytest.fixture(scope="session")
def oracle():
    """The CPU checker: the reference's own compiled CPU kernels where they were built, else the
    plain-C restatement (built on first use)."""
    from oracle import oracle as O
    O.lib("port")
    return _Checker(O, "ref" if O.have("ref") else "port")


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def assert_knn_equal(got_idx, got_dist, ref_idx, ref_dist, coords=None, what=""):
    """kNN parity: rows are compared in canonical order (slot 0 = the query, then ascending
    (distance, index)); distances must be bit-identical.  A row may differ in its last kept
    neighbours only when candidates tie exactly at the row's largest kept distance: there the
    reference keeps whichever its replacement history produced, the library the lower index.
    Such rows must still carry bit-identical distances.  Returns the number of such rows."""
    from oracle import oracle as O
    gi, gd = O.canonical_knn(got_idx, got_dist)
    ri, rd = O.canonical_knn(ref_idx, ref_dist)
    assert np.array_equal(bits(gd), bits(rd)), f"{what}: distances differ"
    same = (gi == ri).all(axis=1)
    tie_rows = 0
    for r in np.nonzero(~same)[0]:
        diff = gi[r] != ri[r]
        worst = rd[r, 1:][ri[r, 1:] >= 0].max()
        assert (rd[r][diff] == worst).all(), f"{what}: row {r} differs away from a boundary tie"
        tie_rows += 1
    return tie_rows
