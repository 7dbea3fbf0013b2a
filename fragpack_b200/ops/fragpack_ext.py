"""Loader of the C-ABI kernel library (replaces ``fragpack/ops/fragpack_ext.py:14-32``).

The reference JIT-builds a pybind11 torch extension; here the kernels live in
``libfragpack_b200.so`` (built in-tree by ``fragpack_b200.csrc.build`` for
sm_100a) whose ``extern "C"`` entry points take raw device pointers.  They are
bound with ``ctypes``; tensors are passed as ``data_ptr()`` and the current
CUDA stream as its handle.  There is no fallback: without the library, or
without a CUDA device, the operators raise.
"""

from __future__ import annotations

import ctypes
import functools
import os
from pathlib import Path

import torch

_DIR = Path(__file__).resolve().parent
# FRAGPACK_B200_LIBRARY points at another build of the same C ABI (for example
# one compiled with different flags); by default the in-tree library is used.
LIBRARY = Path(os.environ.get("FRAGPACK_B200_LIBRARY") or _DIR / "libfragpack_b200.so")

c_i32, c_i64, c_f32, c_ptr = ctypes.c_int32, ctypes.c_int64, ctypes.c_float, ctypes.c_void_p


class FpStore(ctypes.Structure):
    """``fp_store`` of ``include/fragpack_b200.h``."""

    _fields_ = [
        ("counters", c_ptr),
        ("wslot", c_ptr),
        ("tags", c_ptr),
        ("free_stack", c_ptr),
        ("ovf_bits", c_ptr),
        ("claim_list", c_ptr),
        ("close_list", c_ptr),
        ("rec_addr", c_ptr),
        ("rec_len", c_ptr),
        ("staging", c_ptr),
        ("scratch", c_ptr),
        ("overflow", c_ptr),
        ("fill", c_ptr),
        ("slot_owner", c_ptr),
        ("seen_list", c_ptr),
        ("overflow_records", c_i64),
        ("L", c_i32),
        ("H", c_i32),
        ("NB", c_i32),
        ("S_p", c_i32),
        ("S_t", c_i32),
        ("ovf_words", c_i32),
        ("cap", c_i32),
    ]


class FpPeers(ctypes.Structure):
    """``fp_peers`` of ``include/fragpack_b200.h``."""

    _fields_ = [
        ("out", c_ptr * 8),
        ("flag", c_ptr * 8),
        ("epoch", c_ptr),
        ("status", c_ptr),
        ("world", c_i32),
        ("rank", c_i32),
    ]


# name -> argument types; every function returns int.
_SIGNATURES = {
    "fp_decode_workspace": [c_i32, c_i32, c_ptr, c_ptr, c_ptr],
    "fp_fused_decode": [c_ptr, c_i64, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_i64, c_ptr, c_ptr, c_i64,
                        c_ptr, c_i64, c_ptr, c_i64, c_ptr, c_i64, c_i32, c_i32, c_i32, c_i32, c_i32,
                        c_f32, c_i32, c_ptr],
    "fp_fused_decode_peers": [c_ptr, c_i64, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_i64, c_ptr, c_ptr,
                              c_i64, c_ptr, c_i64, c_ptr, c_i64, c_ptr, c_i32, c_i64, c_i32, c_i32,
                              c_i32, c_i32, c_i32, c_f32, c_i32, c_ptr],
    "fp_plain_decode": [c_ptr, c_i64, c_ptr, c_ptr, c_ptr, c_i64, c_ptr, c_ptr, c_i64, c_ptr, c_i64,
                        c_ptr, c_i64, c_ptr, c_i64, c_i32, c_i32, c_i32, c_i32, c_i32, c_f32, c_i32,
                        c_ptr],
    "fp_fused_decode_noalloc": [c_ptr, c_i64, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_i64, c_ptr, c_ptr,
                                c_i64, c_i32, c_i32, c_i32, c_i32, c_i32, c_f32, c_i32, c_ptr],
    "fp_prefill_attention": [c_ptr, c_i64, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_i64, c_ptr, c_ptr, c_ptr,
                             c_i64, c_i32, c_i32, c_i32, c_i32, c_f32, c_ptr, c_ptr],
    "fp_hbm_prepare": [c_ptr, c_ptr, c_i64, c_ptr, c_i64, c_i32, c_ptr],
    "fp_hbm_write": [c_ptr, c_ptr, c_i64, c_i64, c_ptr, c_i64, c_i64, c_ptr, c_i64, c_i32, c_ptr],
    "fp_hbm_encode": [c_ptr, c_ptr, c_i32, c_ptr, c_i64, c_i64, c_ptr],
    "fp_hbm_commit": [c_ptr, c_ptr],
    "fp_hbm_gather": [c_ptr, c_i64, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_i64, c_i32, c_ptr],
    "fp_hbm_gather_status": [c_ptr],
    "fp_debug_wait_limit": [c_i64, c_i64],
    "fp_hbm_export": [c_ptr, c_i64, c_ptr, c_ptr, c_ptr, c_i64, c_i64, c_ptr, c_ptr, c_i32, c_i32,
                      c_i32, c_i64, c_ptr],
    "fp_hbm_import": [c_ptr, c_ptr, c_i64, c_ptr, c_ptr, c_i64, c_ptr, c_ptr, c_ptr, c_ptr, c_i64,
                      c_ptr],
    "fp_encode_records": [c_ptr, c_i64, c_ptr, c_ptr, c_ptr, c_ptr, c_i64, c_ptr, c_ptr],
    "fp_decode_records": [c_ptr, c_i64, c_ptr, c_i64, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr],
}
EXPORTED = tuple(_SIGNATURES) + ("fp_last_error", "fp_version")


@functools.cache
def extension() -> ctypes.CDLL:
    """Load the kernel library once per process.

    Returns:
        The ``ctypes`` handle with argument types set.

    Raises:
        RuntimeError: If the library has not been built.
    """
    if not LIBRARY.exists():
        raise RuntimeError(
            f"{LIBRARY} is missing: build it with `python -m fragpack_b200.csrc.build` "
            "(there is no CPU or PyTorch fallback for fragpack_b200.ops)"
        )
    lib = ctypes.CDLL(str(LIBRARY))
    for name, argtypes in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = ctypes.c_int
    lib.fp_last_error.restype = ctypes.c_char_p
    lib.fp_version.restype = ctypes.c_char_p
    return lib


def check(code: int) -> None:
    """Raise ``RuntimeError`` with the library's message for a nonzero status."""
    if code:
        raise RuntimeError(extension().fp_last_error().decode() or f"fragpack_b200 error {code}")


def require_cuda(tensor: torch.Tensor, name: str) -> None:
    """Reject host tensors: the operators have no CPU path."""
    if not tensor.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: fragpack_b200.ops has no CPU fallback")


def stream_ptr() -> int:
    """Handle of the current CUDA stream."""
    return torch.cuda.current_stream().cuda_stream


__all__ = ["EXPORTED", "FpStore", "check", "extension", "require_cuda", "stream_ptr"]
