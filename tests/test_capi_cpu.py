"""CPU suite: the C-ABI library loads without a GPU, exports every symbol the public header declares,
and rejects malformed arguments on the host before touching the device."""
import ctypes
import os
import re

import pytest

from conftest import ROOT


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "hgcalml_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hgc_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    from hgcalml_b200 import _capi
    names = _declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(_capi.lib, n), f"{n} declared in include/hgcalml_b200.h but not exported"


def test_error_strings_and_version():
    from hgcalml_b200 import _capi
    assert _capi.lib.hgc_version() >= 100
    assert _capi.lib.hgc_strerror(0) == b"ok"
    for code in (-1, -2, -3, -4, -5):
        assert _capi.lib.hgc_strerror(code) not in (b"ok", b"unknown error code")


def test_host_side_validation_needs_no_gpu():
    from hgcalml_b200 import _capi
    L = _capi.lib
    nul = ctypes.c_void_p(None)
    # op shape rules (binned_select_knn_kernel.cc:336-352): 2..5 binning dims, >= 2 coordinates
    assert L.hgc_binned_select_knn(nul, nul, nul, nul, nul, nul, nul, nul, nul,
                                   10, 4, 3, 1, 5, 0, 0, nul, 0, nul) == -1
    assert L.hgc_binned_select_knn(nul, nul, nul, nul, nul, nul, nul, nul, nul,
                                   10, 4, 3, 6, 5, 0, 0, nul, 0, nul) == -1
    assert L.hgc_binned_select_knn(nul, nul, nul, nul, nul, nul, nul, nul, nul,
                                   10, 4, 1, 3, 5, 0, 0, nul, 0, nul) == -1
    # beyond the library's limits
    assert L.hgc_binned_select_knn(nul, nul, nul, nul, nul, nul, nul, nul, nul,
                                   10, 1000, 3, 3, 5, 0, 0, nul, 0, nul) == -3
    # null tensors
    assert L.hgc_binned_select_knn(nul, nul, nul, nul, nul, nul, nul, nul, nul,
                                   10, 4, 3, 3, 5, 0, 0, nul, 0, nul) == -1
    # AccumulateKnn: output width must be F or 2F
    assert L.hgc_accumulate_knn(nul, nul, nul, nul, nul, 10, 4, 8, 9, 0, 1, nul) == -1
    # empty inputs are fine and launch nothing
    assert L.hgc_accumulate_knn(nul, nul, nul, nul, nul, 0, 4, 8, 16, 0, 1, nul) == 0
    assert L.hgc_index_replacer(nul, nul, nul, 0, 0, nul, nul) == 0
    # workspace queries are pure host arithmetic and grow with the problem
    a = L.hgc_binned_select_knn_ragged_workspace_bytes(1000, 16, 4, 2, -1, 3)
    b = L.hgc_binned_select_knn_ragged_workspace_bytes(100000, 16, 4, 2, -1, 3)
    assert 0 < a < b
    assert L.hgc_binned_select_knn_ragged_workspace_bytes(1000, 16, 12, 2, -1, 9) == 0


def test_no_cpu_fallback_in_python_layer():
    import torch
    from hgcalml_b200 import _capi
    from hgcalml_b200.accknn_op import AccumulateKnn
    with pytest.raises(_capi.HgcError):
        AccumulateKnn(torch.zeros(4, 2), torch.zeros(4, 4), torch.zeros(4, 2, dtype=torch.int32))


def test_product_does_not_import_checker():
    """Nothing under hgcalml_b200/ may import or load the CPU checker."""
    pkg = os.path.join(ROOT, "hgcalml_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cc")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src, os.path.join(dirpath, f)


def test_tf_shims_type_check_against_api_stub():
    """TensorFlow is not installed where this suite runs; the shims are at least parsed and
    type-checked against declarations of the custom-op API they use and against the C header."""
    import shutil
    import subprocess
    gxx = shutil.which("g++")
    cuda_inc = "/usr/local/cuda/include"
    if gxx is None or not os.path.exists(os.path.join(cuda_inc, "cuda_runtime.h")):
        pytest.skip("needs g++ and the CUDA headers")
    r = subprocess.run([gxx, "-std=c++17", "-fsyntax-only", "-I" + os.path.join(ROOT, "tests", "tf_api_stub"),
                        "-I" + os.path.join(ROOT, "include"), "-I" + cuda_inc,
                        os.path.join(ROOT, "hgcalml_b200", "tf_shims", "hgc_tf_ops.cc")],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]


def test_host_side_validation_of_wrapper_level_entries():
    """Argument rules of the wrapper-level entries are checked on the host, before any CUDA call."""
    from hgcalml_b200 import _capi
    L = _capi.lib
    nul = ctypes.c_void_p(None)
    f = ctypes.c_float
    # gravnet collect: the slice must fit the rows, the output row must hold 2F columns
    assert L.hgc_gravnet_collect(nul, nul, 8, 1, 8, nul, nul, 64, nul, 10, 16, f(10.), 1, nul, nul) == -1
    assert L.hgc_gravnet_collect(nul, nul, 9, 1, 8, nul, nul, 31, nul, 10, 16, f(10.), 1, nul, nul) == -1
    assert L.hgc_gravnet_collect(nul, nul, 9, -1, 8, nul, nul, 32, nul, 10, 16, f(10.), 1, nul, nul) == -1
    assert L.hgc_gravnet_collect(nul, nul, 9, 1, 8, nul, nul, 32, nul, 0, 16, f(10.), 1, nul, nul) == 0  # no hits
    # condensate wrapper: assert-rules of modules/assign_condensate_op.py:245-247
    args = lambda **kw: [nul] * 11 + [kw.get("n", 10), kw.get("dims", 3), kw.get("n_rs", 2), f(kw.get("bt", 0.1)),
                                      f(kw.get("dt", 1.0)), 1, kw.get("nbd", 3), nul, 0, nul]
    assert L.hgc_build_and_assign_condensates(*args(nbd=0)) == -1
    assert L.hgc_build_and_assign_condensates(*args(nbd=7)) == -1
    assert L.hgc_build_and_assign_condensates(*args(bt=1.5)) == -1
    assert L.hgc_build_and_assign_condensates(*args(dt=0.0)) == -1
    assert L.hgc_build_and_assign_condensates(*args(dims=9)) == -3
    assert L.hgc_build_and_assign_condensates(*args()) == -1           # null outputs
    assert L.hgc_build_and_assign_condensates_workspace_bytes(1000, 3, 3, 3) > 0
    assert L.hgc_build_and_assign_condensates_workspace_bytes(1000, 9, 3, 3) == 0


def test_gravnet_layer_mirrors_construct_without_gpu():
    import torch
    from hgcalml_b200 import _capi
    from hgcalml_b200.GravNetLayersRagged import RaggedGravNet, DistanceWeightedMessagePassing, collect_neighbours
    layer = RaggedGravNet(n_neighbours=8, n_dimensions=3, n_filters=12, n_propagate=6, n_in=10)
    assert layer.output_feature_transform.kernel.shape == (2 * 6 + 10, 12)
    mp = DistanceWeightedMessagePassing([4, 5], n_in=10)
    assert [tuple(d.kernel.shape) for d in mp.feature_tranformation_dense] == [(10, 4), (8, 5)]
    with pytest.raises(NotImplementedError):
        RaggedGravNet(8, 3, 12, 6, n_in=10, sumwnorm=True)
    with pytest.raises(_capi.HgcError):  # CPU tensors: no fallback
        collect_neighbours(torch.zeros(4, 4), torch.zeros(4, 3, dtype=torch.int32), torch.zeros(4, 3))


def _build_c_user(out_path):
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    cuda = "/usr/local/cuda"
    if gcc is None or not os.path.exists(os.path.join(cuda, "include", "cuda_runtime_api.h")):
        pytest.skip("needs gcc and the CUDA runtime headers")
    pkg = os.path.join(ROOT, "hgcalml_b200")
    r = subprocess.run([gcc, "-std=c11", "-O2", "-ffp-contract=off", "-I" + os.path.join(ROOT, "include"),
                        "-I" + os.path.join(cuda, "include"), os.path.join(ROOT, "tests", "c_abi", "knn_from_c.c"),
                        "-o", out_path, "-L" + pkg, "-lhgcalml_b200", "-L" + os.path.join(cuda, "lib64"), "-lcudart",
                        "-lm", "-Wl,-rpath," + pkg], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    return out_path


def test_plain_c_user_of_the_abi_compiles_and_links(tmp_path):
    """The header is C (not C++) and the library links into a program that knows nothing of Python or torch."""
    _build_c_user(str(tmp_path / "knn_from_c"))
