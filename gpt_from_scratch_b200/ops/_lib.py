"""ctypes binding to the native sm_100a library (``lib/libgfs_b200.so``).

The library is built in-tree by :mod:`gpt_from_scratch_b200.build`. Nothing here
falls back silently: asking for the library on a machine where it has not been
built raises, so a GPU run can never pass on a PyTorch fallback by accident.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_uint32, c_void_p, POINTER
from pathlib import Path

import torch

# GFS_LIB_PATH selects another build of the library (e.g. an experimental variant) explicitly.
_LIB_PATH = Path(os.environ.get("GFS_LIB_PATH") or
                 Path(__file__).resolve().parent.parent / "lib" / "libgfs_b200.so")
_lib = None
_lock = threading.Lock()

# Number of kernels of this library launched since the last reset (host-side count
# of successful launcher calls; used by the benchmark's ``gpu_launches`` field).
_launch_count = 0

STATUS_NAMES = {
    0: "ok",
    1: "timeout: consumer waited for a TMA stage",
    2: "timeout: producer waited for a free stage",
    3: "timeout: epilogue waited for the accumulator",
    4: "timeout: MMA warp waited for a drained accumulator",
    5: "timeout: attention role hand-off",
    6: "timeout: cross-GPU flag never arrived",
    7: "timeout: grid barrier",
    8: "bad argument",
    9: "timeout: test flag (expected by the wait probe)",
}


class NativeLibraryError(RuntimeError):
    pass


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    return _LIB_PATH.exists()


def _declare(lib: ctypes.CDLL) -> None:
    vp, i, sz, f, i64, d = c_void_p, c_int, c_size_t, c_float, c_int64, ctypes.c_double
    lp = POINTER(ctypes.c_longlong)
    ulp = POINTER(ctypes.c_ulonglong)
    uip = POINTER(ctypes.c_uint)
    ip = POINTER(ctypes.c_int)
    cl = ctypes.c_long
    sigs = {
        "gfs_read_status": ([POINTER(c_uint32), i], i),
        "gfs_sm_count": ([], i),
        "gfs_last_cuda_error": ([], c_char_p),
        "gfs_gemm_bf16": ([vp, vp, vp, vp, i, i, i, i, i, i, i, i, i, i, vp, sz, i, vp], i),
        "gfs_gemm_bf16_launches": ([i, i, i, sz], i),
        "gfs_rmsnorm_fwd": ([vp, vp, vp, vp, i, i, f, vp], i),
        "gfs_rmsnorm_bwd_parts": ([i], i),
        "gfs_rmsnorm_bwd": ([vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, vp], i),
        "gfs_rope": ([vp, vp, vp, i, i, i, i, i, cl, i, i, vp], i),
        "gfs_swiglu_fwd": ([vp, vp, i, i, vp], i),
        "gfs_swiglu_bwd": ([vp, vp, vp, i, i, vp], i),
        "gfs_embedding_fwd": ([vp, vp, vp, i, i, i, i, i, i, i, vp], i),
        "gfs_embedding_bwd": ([vp, vp, vp, vp, i, i, i, i, vp], i),
        "gfs_embedding_sort_keys": ([vp, vp, i, i, i, i, vp], i),
        "gfs_embedding_bwd_keys": ([vp, vp, vp, i, i, i, vp], i),
        "gfs_ce_fwd": ([vp, vp, vp, vp, vp, i, i, cl, i, i, vp], i),
        "gfs_ce_combine": ([vp, vp, vp, i, i, vp], i),
        "gfs_ce_bwd": ([vp, vp, vp, vp, i, i, cl, i, vp], i),
        "gfs_sumsq_scratch_bytes": ([], i),
        "gfs_sumsq_bf16": ([vp, i64, vp, vp, vp], i),
        "gfs_adamw_step": ([vp, vp, vp, vp, vp, i64, vp, vp, f, d, d, f, f, f, f, f, f, vp, vp], i),
        "gfs_flag_slots": ([], i),
        "gfs_wait_probe": ([vp, i64, vp], i),
        "gfs_flash_fwd": ([vp, vp, vp, vp, vp, i, i, i, i, lp, f, i, vp], i),
        "gfs_flash_bwd": ([vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, i, lp, f, i, vp, vp, vp], i),
        "gfs_gemm_bf16_comm": ([i, vp, i, vp, i, vp, i, vp, i, i, i, i, i, i, i, ulp, ulp, uip, vp, vp, i, i, i,
                                ctypes.c_longlong, vp], i),
        "gfs_rmsnorm_dw_reduce_multi": ([i, ulp, ulp, ip, ip, i, vp], i),
        "gfs_dropout_residual": ([vp, vp, vp, ctypes.c_longlong, f, ctypes.c_ulonglong, i, vp], i),
        "gfs_gemm2_ce_parts": ([i], i),
        "gfs_gemm2_bf16_ce": ([vp, vp, vp, vp, i, i, i, i, i, i, vp], i),
        "gfs_ce_from_partials": ([vp, vp, vp, vp, vp, vp, i, i, i, cl, i, i, vp], i),
        "gfs_gemm2_wgrad_grouped": ([i, ulp, ulp, ulp, ip, ip, ip, ip, ip, ip, ip, vp], i),
        "gfs_gemm2_bf16_comm": ([i, vp, i, vp, i, vp, i, vp, i, i, i, i, i, i, i, ulp, ulp, uip, vp, vp, i, i, i,
                                 ctypes.c_longlong, vp], i),
        "gfs_gemm2_bf16_allgather_ce": ([vp, i, vp, i, vp, i, vp, i, i, i, i, i, ulp, ulp, uip, ctypes.c_longlong,
                                         vp], i),
        "gfs_gemm2_bf16_comm_swiglu": ([i, vp, i, vp, i, vp, i, vp, i, i, i, i, i, i, ulp, ulp, uip,
                                        ctypes.c_longlong, vp], i),
        "gfs_symm_barrier": ([ulp, i, i, i, uip, ctypes.c_longlong, vp], i),
        "gfs_allgather": ([vp, i, i, i, ulp, ulp, i, i, i, uip, ctypes.c_longlong, vp], i),
        "gfs_embedding_scatter": ([vp, vp, i, i, i, i, i, ulp, ulp, i, i, i, uip, ctypes.c_longlong, vp], i),
        "gfs_ce_exchange": ([vp, vp, vp, i, ulp, ulp, i, i, i, uip, ctypes.c_longlong, vp], i),
        "gfs_dp_reduce_norm_scratch_floats": ([], i),
        "gfs_dp_push_grads": ([vp, ulp, ulp, i, lp, lp, lp, i, i, i, i, uip, vp], i),
        "gfs_dp_sum_norm": ([vp, ulp, ulp, ulp, vp, i, lp, lp, lp, i, i, i, ctypes.c_uint, i, uip, vp,
                             ctypes.c_longlong, vp], i),
        "gfs_dp_adam_gather": ([ulp, ulp, ulp, vp, vp, vp, vp, i, lp, lp, lp, i, i, i, ctypes.c_uint, i, uip, vp, vp,
                                f, d, d, f, f, f, f, f, f, vp, ctypes.c_longlong, vp], i),
        "gfs_gemm_bf16_swiglu": ([i, vp, vp, vp, vp, i, i, i, i, i, i, i, vp], i),
        "gfs_gemm2_bf16_swiglu": ([i, vp, vp, vp, vp, i, i, i, i, i, i, i, vp], i),
        "gfs_gemm2_bf16": ([vp, vp, vp, vp, i, i, i, i, i, i, i, i, i, vp, vp, i, i, i, vp], i),
        "gfs_gemm_bf16_rope": ([vp, vp, vp, vp, i, i, i, i, i, i, i, i, i, i, vp, sz, i, vp, vp, i, i, i, vp], i),
    }
    for name, (argtypes, restype) in sigs.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue
        fn.argtypes = argtypes
        fn.restype = restype


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not _LIB_PATH.exists():
                    raise NativeLibraryError(
                        f"{_LIB_PATH} is missing: build it with `python -m gpt_from_scratch_b200.build`")
                handle = ctypes.CDLL(os.fspath(_LIB_PATH))
                _declare(handle)
                _lib = handle
    return _lib


class _NullRange:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


class _NvtxRange:
    __slots__ = ("name",)

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        torch.cuda.nvtx.range_pop()
        return False


_NVTX = os.environ.get("GFS_NVTX", "0") == "1"
_NULL_RANGE = _NullRange()


def nvtx(name: str):
    """``with nvtx("name"):`` marks a fused operator for timeline tools (chrome traces of
    ``tools/profile_train.py``, ncu's NVTX filters). Enabled with GFS_NVTX=1, free otherwise."""
    return _NvtxRange(name) if _NVTX else _NULL_RANGE


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None) -> int:
    return 0 if t is None else t.data_ptr()


def check(rc: int, what: str) -> None:
    global _launch_count
    if rc != 0:
        raise NativeLibraryError(f"{what} failed with code {rc}")
    _launch_count += 1


def add_launches(n: int) -> None:
    global _launch_count
    _launch_count += n


def launch_count() -> int:
    return _launch_count


def reset_launch_count() -> None:
    global _launch_count
    _launch_count = 0


def read_status(clear: bool = True) -> tuple[int, int]:
    """Synchronise and return the (code, detail) status words of the current device."""
    out = (c_uint32 * 2)()
    lib().gfs_read_status(out, 1 if clear else 0)
    return int(out[0]), int(out[1])


def raise_on_status() -> None:
    code, detail = read_status(clear=True)
    if code != 0:
        raise NativeLibraryError(
            f"device status {code} ({STATUS_NAMES.get(code, 'unknown')}), detail 0x{detail:x}")
