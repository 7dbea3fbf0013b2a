"""Drop-in for the reference's ``fragpack/ops/fragpack_ext.py``.

The reference loads a pybind11 module ``fragpack_cuda`` whose eight functions
take ``torch.Tensor`` arguments (``fragpack/ops/fragpack_ext.cpp:5-66``) and
calls them only through ``fragpack_ext.extension()``.  A maintainer who wants
to keep the reference's own Python (``fragpack/ops/hbm_kv.py``,
``fragpack/ops/fused_attn_decode.py``) and run it on a B200 replaces that one
file by this one: ``extension()`` returns an object with the same eight
functions, same names, same positional arguments, bound to the C ABI of
``libfragpack_b200.so`` (``include/fragpack_b200.h``) with ``ctypes``.

Two things the reference's store state does not have are kept here, per store
(keyed by the address of its ``counters`` tensor) and created on first use:
the staging-slot owner table and the list of blocks seen opening / closing in
a step, both used by this library's ``prepare``; and the free-slot counter of
the overflow pool in ``counters[13]``, which the reference leaves unused.

Differences a caller of the reference's Python sees: none in results.
``workspace_elems`` of the reference sizes ``plan`` as ``2 + 4 * units`` int32;
this library needs ``2 + 8 * units + 262`` (a spare, a status word, the words
of its item schedule and four words per unit of item descriptors), so
:func:`plan_words` must be used for that allocation.
"""

from __future__ import annotations

import ctypes
import functools
import os
from pathlib import Path

import torch

_LIBRARY = Path(
    os.environ.get("FRAGPACK_B200_LIBRARY")
    or Path(__file__).resolve().parents[1] / "ops" / "libfragpack_b200.so"
)
_OVF_FREE = 13  # FP_CTR_OVF_FREE
_ptr, _i32, _i64, _f32 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_float


class _Store(ctypes.Structure):
    """``fp_store`` of ``include/fragpack_b200.h``."""

    _fields_ = (
        [(name, _ptr) for name in (
            "counters", "wslot", "tags", "free_stack", "ovf_bits", "claim_list", "close_list",
            "rec_addr", "rec_len", "staging", "scratch", "overflow", "fill", "slot_owner",
            "seen_list")]
        + [("overflow_records", _i64)]
        + [(name, _i32) for name in ("L", "H", "NB", "S_p", "S_t", "ovf_words", "cap")]
    )


def plan_words(units: int) -> int:
    """int32 elements of the decode ``plan`` workspace for ``units`` work units."""
    return 2 + 4 * units + 2 + 260 + 4 * units


def _p(t: torch.Tensor | None) -> ctypes.c_void_p:
    return _ptr(None if t is None else t.data_ptr())


class ReferenceExtension:
    """The eight functions of the reference's ``fragpack_cuda`` module over the C ABI.

    All of them enqueue on the current CUDA stream and return ``None``; a
    rejected call raises ``RuntimeError`` with the library's message, as the
    reference's ``TORCH_CHECK`` failures do.
    """

    def __init__(self, library: Path = _LIBRARY) -> None:
        if not library.exists():
            raise RuntimeError(f"{library} is missing: build it with `python -m fragpack_b200.csrc.build`")
        self._lib = ctypes.CDLL(str(library))
        self._lib.fp_last_error.restype = ctypes.c_char_p
        self._side: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}

    # ---- plumbing -------------------------------------------------------
    def _check(self, rc: int) -> None:
        if rc:
            raise RuntimeError(self._lib.fp_last_error().decode() or f"fragpack_b200 error {rc}")

    @staticmethod
    def _stream() -> ctypes.c_void_p:
        return _ptr(torch.cuda.current_stream().cuda_stream)

    def _store(self, counters, wslot, tags, free_stack, ovf_bits, claim_list, close_list, rec_addr,
               rec_len, staging, scratch, overflow, fill) -> _Store:
        L, NB, _, H = rec_addr.shape
        S_p = free_stack.numel()
        S_t = scratch.numel() // (2 * H * 32768)
        cap = claim_list.numel() // 2
        key = counters.data_ptr()
        if key not in self._side:
            i32 = dict(dtype=torch.int32, device=counters.device)
            self._side[key] = (torch.full((S_p + S_t,), -1, **i32), torch.zeros(2 * cap, **i32))
            # Free overflow slots = clear bits of the bitmap (its tail bits are preset).
            used = int(torch.count_nonzero(
                (ovf_bits.view(torch.int32)[:, None] >> torch.arange(32, device=ovf_bits.device)) & 1))
            counters[_OVF_FREE] = ovf_bits.numel() * 32 - used
        slot_owner, seen_list = self._side[key]
        tensors = (counters, wslot, tags, free_stack, ovf_bits, claim_list, close_list, rec_addr,
                   rec_len, staging, scratch, overflow, fill, slot_owner, seen_list)
        return _Store(*(t.data_ptr() for t in tensors), overflow.shape[0], L, H, NB, S_p, S_t,
                      ovf_bits.numel(), cap)

    # ---- fragpack_ext.cpp:5-9 -------------------------------------------
    def fused_decode(self, q, rec_addr, rec_len, plut, slut, block_table, seq_lens, opart, ml, plan,
                     out, units: int, replan: bool, scale: float) -> None:
        kv_heads = rec_addr.shape[2]
        self._check(self._lib.fp_fused_decode(
            _p(q), _i64(q.stride(0)), _p(rec_addr), _p(rec_len), _p(plut), _p(slut), _p(block_table),
            _i64(block_table.stride(0)), _p(seq_lens), _p(opart), _i64(opart.numel()), _p(ml),
            _i64(ml.numel()), _p(plan), _i64(plan.numel()), _p(out), _i64(out.stride(0)),
            _i32(q.shape[0]), _i32(kv_heads), _i32(q.shape[1] // kv_heads), _i32(units),
            _i32(int(bool(replan))), _f32(scale), _i32(0), self._stream()))

    # ---- fragpack_ext.cpp:11-17 -----------------------------------------
    def hbm_prepare(self, *args) -> None:
        state, (slot_mapping, n_tok, live, n_live, step) = args[:13], args[13:]
        store = self._store(*state)
        self._check(self._lib.fp_hbm_prepare(
            ctypes.byref(store), _p(slot_mapping), _i64(n_tok), _p(live), _i64(n_live), _i32(step),
            self._stream()))

    # ---- fragpack_ext.cpp:19-25 -----------------------------------------
    def hbm_write(self, *args) -> None:
        state, (key, value, slot_mapping, layer) = args[:13], args[13:]
        store = self._store(*state)
        self._check(self._lib.fp_hbm_write(
            ctypes.byref(store), _p(key), _i64(key.stride(0)), _i64(key.stride(1)), _p(value),
            _i64(value.stride(0)), _i64(value.stride(1)), _p(slot_mapping), _i64(key.shape[0]),
            _i32(layer), self._stream()))

    # ---- fragpack_ext.cpp:27-33 -----------------------------------------
    def hbm_encode(self, *args) -> None:
        state, (rank_of, layer, arena, arena_stride, max_close) = args[:13], args[13:]
        store = self._store(*state)
        self._check(self._lib.fp_hbm_encode(
            ctypes.byref(store), _p(rank_of), _i32(layer), _ptr(arena), _i64(arena_stride),
            _i64(max_close), self._stream()))

    # ---- fragpack_ext.cpp:35-39 -----------------------------------------
    def hbm_commit(self, *state) -> None:
        store = self._store(*state)
        self._check(self._lib.fp_hbm_commit(ctypes.byref(store), self._stream()))

    # ---- fragpack_ext.cpp:41-43 -----------------------------------------
    def hbm_gather(self, src_blocks, rec_addr, rec_len, plut, slut, wk, wv, kv_heads: int) -> None:
        size = min(wk.numel() * wk.element_size(), wv.numel() * wv.element_size())
        self._check(self._lib.fp_hbm_gather(
            _p(src_blocks), _i64(src_blocks.numel()), _p(rec_addr), _p(rec_len), _p(plut), _p(slut),
            _p(wk), _p(wv), _i64(size), _i32(kv_heads), self._stream()))

    # ---- fragpack_ext.cpp:45-46 -----------------------------------------
    def hbm_export(self, blocks, rec_addr, rec_len, out, stride: int, lengths, digest: int) -> None:
        L, NB, _, H = rec_addr.shape
        scratch = torch.empty((blocks.numel(), L * 2 * H), dtype=torch.int64, device=out.device)
        self._check(self._lib.fp_hbm_export(
            _p(blocks), _i64(blocks.numel()), _p(rec_addr), _p(rec_len), _p(out), _i64(out.numel()),
            _i64(stride), _p(lengths), _p(scratch), _i32(L), _i32(H), _i32(NB), _i64(digest),
            self._stream()))

    # ---- fragpack_ext.cpp:48-55 -----------------------------------------
    def hbm_import(self, *args) -> None:
        state, (src, offsets, blocks, status, arena_base, arena_stride, digest) = args[:13], args[13:]
        store = self._store(*state)
        scratch = torch.empty((2, blocks.numel(), store.L * 2 * store.H), dtype=torch.int64,
                              device=src.device)
        self._check(self._lib.fp_hbm_import(
            ctypes.byref(store), _p(src), _i64(src.numel()), _p(offsets), _p(blocks),
            _i64(blocks.numel()), _p(status), _p(scratch), _p(arena_base), _p(arena_stride),
            _i64(digest), self._stream()))


@functools.cache
def extension() -> ReferenceExtension:
    """The stand-in for the reference's ``fragpack_ext.extension()``."""
    return ReferenceExtension()


__all__ = ["ReferenceExtension", "extension", "plan_words"]
