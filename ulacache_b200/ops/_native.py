"""ctypes bindings for the in-tree native libraries.

``cuda()`` returns ``libulc_cuda.so`` (kernels for sm_100a), ``host()`` returns
``libulc_host.so`` (CPU oracles).  Both are built ahead of time by
``ulacache_b200.build`` and live under ``ulacache_b200/_lib``.  There is no
silent fallback: on a machine with a GPU a missing CUDA library is an error.

Every exported function returns 0 on success, a positive ``cudaError_t`` when
the launch failed, or a negative :class:`Status` code when the arguments were
rejected before launching.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_LIB_DIR = Path(__file__).resolve().parent.parent / "_lib"
_cuda = None
_host = None

MAX_RANKS = 8
STATUS_WORDS = 4
NUM_COUNTERS = 32
RING_BUCKETS = 256
PLAN_ROWS = 5

STATUS_NAMES = {
    0: "ok", 1: "index out of bounds", 2: "capacity exhausted", 3: "invariant violated",
    4: "bounded wait timed out", 5: "misaligned pointer or extent", 6: "unsupported shape",
    7: "tensor-core pipeline wait timed out",
}


class NativeError(RuntimeError):
    pass


class OwnerMap(C.Structure):
    _fields_ = [("ranks", C.c_int32), ("stripe_shift", C.c_int32)]


class PoolView(C.Structure):
    _fields_ = [
        ("hbm", C.c_void_p * MAX_RANKS),
        ("host", C.c_void_p),
        ("dir", C.c_void_p * MAX_RANKS),
        ("dir_len", C.c_int32),
        ("hbm_slots", C.c_int32),
        ("host_slots", C.c_int32),
        ("rec_bytes", C.c_int32),
        ("map", OwnerMap),
        ("my_rank", C.c_int32),
        ("pad_", C.c_int32),
    ]


class IndexPoolView(C.Structure):
    _fields_ = [
        ("pages", C.c_void_p * MAX_RANKS),
        ("pages_per_rank", C.c_int32),
        ("ranks", C.c_int32),
        ("my_rank", C.c_int32),
        ("pad_", C.c_int32),
    ]


class ResidencyState(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "directory", "hbm_tags", "host_tags", "stamps", "access_time", "hbm_free", "host_free",
        "counters", "ring", "promote", "plan", "victims")] + [
        ("dir_len", C.c_int32), ("hbm_slots", C.c_int32), ("host_slots", C.c_int32),
        ("plan_capacity", C.c_int32),
        # optional presence-bitmap victim index (null pointers = scan the stamps)
        ("bits", C.c_void_p), ("summary", C.c_void_p), ("vlist", C.c_void_p), ("chunk_count", C.c_void_p),
        ("w0", C.c_int32), ("w1", C.c_int32)]


class PlaneSet(C.Structure):
    _fields_ = [
        ("hbm", C.c_void_p), ("host", C.c_void_p),
        ("hbm_layer_stride", C.c_longlong), ("host_layer_stride", C.c_longlong),
        ("rec_bytes", C.c_int32), ("layer_begin", C.c_int32), ("layer_count", C.c_int32),
        ("pad_", C.c_int32),
    ]


def lib_path(name: str) -> Path:
    return _LIB_DIR / name


def _load(name: str):
    path = lib_path(name)
    if not path.exists():
        # build in tree on first use (nvcc cross-compiles for sm_100a without a GPU)
        try:
            from .. import build

            build.build_host() if name == "libulc_host.so" else build.build_cuda()
        except Exception as exc:
            raise NativeError(
                f"{path} is missing and could not be built ({exc}); run `python -m ulacache_b200.build`") from exc
    return C.CDLL(str(path))


def cuda():
    global _cuda
    if _cuda is None:
        _cuda = _load("libulc_cuda.so")
    return _cuda


def host():
    global _host
    if _host is None:
        _host = _load("libulc_host.so")
    return _host


def available() -> bool:
    return lib_path("libulc_cuda.so").exists()


def ptr(t):
    """Device (or host) address of a tensor, or NULL for None."""
    return C.c_void_p(0 if t is None else t.data_ptr())


def stream():
    import torch

    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


# Kernels launched per successful entry-point call (used to report launch counts).
KERNELS_PER_CALL = {"res_plan": 3, "res_commit": 2, "index_score": 2, "gemm_wt_bf16": 1,
                    "fp8_grouped_gemm_experts": 2}
LAUNCHES = 0


def check(code: int, what: str):
    global LAUNCHES
    if code == 0:
        LAUNCHES += KERNELS_PER_CALL.get(what, 1)
        return
    if code < 0:
        raise NativeError(f"{what}: rejected ({STATUS_NAMES.get(-code, code)})")
    raise NativeError(f"{what}: CUDA error {code}")


def new_status(device):
    import torch

    return torch.zeros(STATUS_WORDS, dtype=torch.int32, device=device)


def raise_on_status(status, what: str):
    """Read a status buffer back (synchronises) and raise if a kernel reported an error."""
    vals = status.tolist()
    if vals[0] != 0:
        status.zero_()
        raise NativeError(
            f"{what}: {STATUS_NAMES.get(vals[0], vals[0])} (detail {vals[1]}, {vals[2]} reports)")
