"""ctypes binding of libhgcalml_b200.so (the C ABI declared in include/hgcalml_b200.h).

There is no fallback: if the shared library is missing the import of any op fails with a clear
error, and every entry point raises when the library reports a non-zero status.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_int, c_size_t, c_void_p

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libhgcalml_b200.so")

HGC_OK = 0
STATUS_BITS = {1: "bin index out of range", 2: "flat bin index overflow",
               4: "gathered index out of range", 8: "iteration cap reached"}


class HgcError(RuntimeError):
    pass


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build it with `make -C {os.path.join(_HERE, 'csrc')}` "
            "(or __graft_entry__.build()); hgcalml_b200 has no CPU or eager fallback")
    lib = ctypes.CDLL(LIB_PATH)
    P, I, S = c_void_p, c_int, c_size_t
    sig = {
        "hgc_strerror": (ctypes.c_char_p, [I]),
        "hgc_last_cuda_error": (ctypes.c_char_p, []),
        "hgc_version": (I, []),
        "hgc_launch_count": (ctypes.c_ulonglong, []),
        "hgc_workspace_status": (I, [P, P, ctypes.POINTER(ctypes.c_uint)]),
        "hgc_bin_by_coordinates_workspace_bytes": (S, [I, I, I, I]),
        "hgc_bin_by_coordinates": (I, [P, P, P, P, P, P, P, I, I, I, I, I, P, S, P]),
        "hgc_binned_select_knn_workspace_bytes": (S, [I, I, I, I]),
        "hgc_binned_select_knn": (I, [P] * 9 + [I] * 7 + [P, S, P]),
        "hgc_binned_select_knn_static": (I, [P] * 9 + [I] * 7 + [P]),
        "hgc_binned_select_knn_static_status": (I, [P, ctypes.POINTER(ctypes.c_uint)]),
        "hgc_index_replacer": (I, [P, P, P, I, I, P, P]),
        "hgc_accumulate_knn": (I, [P] * 5 + [I] * 6 + [P]),
        "hgc_accumulate_knn_exp": (I, [P] * 5 + [I] * 5 + [ctypes.c_float, P, P]),
        "hgc_gravnet_collect": (I, [P, P, I, I, I, P, P, I, P, I, I, ctypes.c_float, I, P, P]),
        "hgc_binned_select_knn_ragged_workspace_bytes": (S, [I] * 6),
        "hgc_binned_select_knn_ragged": (I, [P] * 6 + [I] * 8 + [P, S, P]),
        "hgc_build_and_assign_condensates_workspace_bytes": (S, [I] * 4),
        "hgc_build_and_assign_condensates": (I, [P] * 11 + [I] * 3 + [ctypes.c_float] * 2 + [I] * 2 + [P, S, P]),
        "hgc_local_distance": (I, [P, P, P, I, I, I, I, P]),
        "hgc_push_knn": (I, [P, P, P, P, I, I, I, P, S, P]),
        "hgc_push_knn_grad": (I, [P] * 6 + [I] * 3 + [P]),
        "hgc_knn_grad_workspace_bytes": (S, [I, I]),
        "hgc_accumulate_knn_grad": (I, [P] * 7 + [I] * 6 + [P, S, P]),
        "hgc_accumulate_knn_grad_ordered": (I, [P] * 7 + [I] * 6 + [P, P, S, P]),
        "hgc_select_knn_grad": (I, [P] * 5 + [I] * 3 + [P, S, P]),
        "hgc_binned_assign_to_condensates_workspace_bytes": (S, [I] * 4),
        "hgc_binned_assign_to_condensates": (I, [I, I] + [P] * 4 + [P] + [P] * 2 + [P] * 4 + [P] * 4 + [P] * 3
                                             + [P, I, I, I, I] + [P, S, P]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()
EXPORTED = [n for n in dir(lib) if n.startswith("hgc_")]


def check(rc: int, what: str) -> None:
    if rc != HGC_OK:
        msg = lib.hgc_strerror(rc).decode()
        if rc == -4:
            msg += ": " + lib.hgc_last_cuda_error().decode()
        raise HgcError(f"{what}: {msg} ({rc})")


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    if t is None:
        return None
    return c_void_p(t.data_ptr())


def stream_of(t: torch.Tensor):
    """The current stream of the tensor's device.  The library launches on the calling thread's
    current device, so that device must be the tensor's."""
    if t.device.index is not None and t.device.index != torch.cuda.current_device():
        raise HgcError(f"tensors live on {t.device} but the current CUDA device is "
                       f"cuda:{torch.cuda.current_device()}: call torch.cuda.set_device (or use "
                       "torch.cuda.device) before calling hgcalml_b200 ops")
    return c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def workspace(nbytes: int, device) -> torch.Tensor:
    return torch.empty((max(int(nbytes), 256),), dtype=torch.uint8, device=device)


def read_status(ws: torch.Tensor, raise_on_flag: bool = True) -> int:
    """Synchronising read of the status word a call left in its workspace."""
    out = ctypes.c_uint(0)
    rc = lib.hgc_workspace_status(ptr(ws), stream_of(ws), ctypes.byref(out))
    if rc not in (0, -5):
        check(rc, "hgc_workspace_status")
    if out.value and raise_on_flag:
        names = [v for k, v in STATUS_BITS.items() if out.value & k]
        raise HgcError("device status: " + ", ".join(names))
    return out.value


def f32(t, device=None):
    t = torch.as_tensor(t, device=device)
    return t.to(torch.float32).contiguous()


def i32(t, device=None):
    t = torch.as_tensor(t, device=device)
    return t.to(torch.int32).contiguous()


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise HgcError("hgcalml_b200 ops take CUDA tensors; there is no CPU path")
