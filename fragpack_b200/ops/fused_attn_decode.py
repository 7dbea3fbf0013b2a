"""Split-KV decode attention over FragPack KV records (sm_100a).

Same public names and argument meaning as the reference
``fragpack/ops/fused_attn_decode.py`` (``GQA``, ``RecordTables``,
``decode_units``, ``workspace_elems``, ``decode_attention``), so the
reference's tests and callers run unchanged.  Differences, all internal:

* the query group (1, 2, 4 or 8 heads per KV head) is handled natively by the
  kernel, so no padded copies of ``q`` / ``out`` are made;
* a work unit is still a chunk of pages of one sequence, but units x KV heads
  are executed by persistent CTAs that stream every record of their items
  through one bulk-copy ring; :func:`decode_units` therefore reserves more
  split capacity than the reference (finer chunks cost almost nothing);
* the ``plan`` workspace ends with a status word that the kernel sets if a
  bounded device-side wait ever runs out (:func:`decode_status`).

Records are located through ``rec_addr[P, 2, H]`` (absolute device addresses)
and ``rec_len[P, 2, H]`` (record bytes minus ``DENSE_BYTES``; raw records
included).  A launch depends only on ``(B, units, H)`` and is CUDA-graph safe;
the plan is computed on the device when ``replan`` is true and reused by the
other layers of the step.
"""

from __future__ import annotations

from dataclasses import dataclass
import functools

import torch

from fragpack_b200.logging import init_logger
from fragpack_b200.ops.fragpack_ext import check, extension, require_cuda, stream_ptr

logger = init_logger(__name__)

GQA = 8
# Split capacity reserved per KV head, in waves of resident CTAs.
SPLIT_WAVES = 8
# Bits of the status word (include/fragpack_b200.h).
# Words of the dynamic item schedule at the end of the plan (started CTAs, one
# item counter per attention launch since the plan was made).
_PLAN_SCHEDULE_WORDS = 4 + 256
DECODE_WAIT_TIMEOUT = 1
DECODE_NOT_PLAIN = 2


@dataclass(frozen=True)
class RecordTables:
    """One layer's record tables for :func:`decode_attention`.

    Attributes:
        rec_addr: int64 ``[P, 2, H]`` record device addresses.
        rec_len: int32 ``[P, 2, H]`` record bytes minus ``DENSE_BYTES``.
        plut: int32 ``[2, H, 2]`` primary ``prmt`` tables.
        slut: uint8 ``[2, H, 16]`` extended tables.
    """

    rec_addr: torch.Tensor
    rec_len: torch.Tensor
    plut: torch.Tensor
    slut: torch.Tensor


def decode_units(batch: int, kv_heads: int, num_sms: int) -> int:
    """Return the work-unit capacity per KV head of a decode launch.

    One unit per sequence plus ``SPLIT_WAVES`` waves (two CTAs per SM) of split
    capacity minus one.  It depends only on the (padded) batch size, so the
    launch shape stays fixed under CUDA graphs (reference:
    ``fused_attn_decode.py:58-85``, which reserves a single wave).

    Args:
        batch: Number of sequences.
        kv_heads: KV heads per sequence.
        num_sms: Streaming multiprocessor count.

    Returns:
        Unit count, at least ``batch``.
    """
    wave = max(1, (2 * num_sms) // max(1, kv_heads))
    return batch + SPLIT_WAVES * wave - 1


def workspace_elems(kv_heads: int, units: int) -> tuple[int, int, int]:
    """Return the element counts of the ``(opart, ml, plan)`` workspace.

    Reference: ``fused_attn_decode.py:88-102``.  The plan holds more than the
    reference's: a spare and the status word, the words of the dynamic item
    schedule, and four words per unit of item descriptors in schedule order.

    Args:
        kv_heads: KV heads per sequence.
        units: Work-unit capacity per KV head.

    Returns:
        Float elements of ``opart`` and ``ml``, int32 elements of ``plan``.
    """
    rows = kv_heads * units * GQA
    return rows * 128, rows * 2, 2 + 4 * units + 2 + _PLAN_SCHEDULE_WORDS + 4 * units


@functools.cache
def _sm_count(index: int) -> int:
    return torch.cuda.get_device_properties(index).multi_processor_count


def _check_decode_args(q, tables, block_table, seq_lens, out, workspace):
    """Shape / dtype checks shared by the decode entry points; returns (kv_heads, group, workspace)."""
    kv_heads = tables.rec_addr.shape[2]
    group = q.shape[1] // kv_heads
    if group == 0 or group * kv_heads != q.shape[1] or GQA % group:
        raise ValueError(f"query heads {q.shape[1]} need a group dividing {GQA}")
    require_cuda(q, "q")
    if q.dim() != 3 or q.shape[2] != 128 or q.stride(2) != 1 or q.stride(1) != 128:
        raise RuntimeError("q must be [B, H, 128] with contiguous heads")
    if out.dim() != 3 or out.stride(2) != 1 or out.stride(1) != 128 or out.shape != q.shape:
        raise RuntimeError("out must be [B, H, 128] with contiguous heads")
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise RuntimeError("q and out must be bfloat16")
    if block_table.stride(1) != 1 or block_table.dtype != torch.int32:
        raise RuntimeError("block_table must be int32 with contiguous rows")
    if seq_lens.dtype != torch.int32 or not seq_lens.is_contiguous():
        raise RuntimeError("seq_lens must be contiguous int32")
    opart, ml, plan = workspace
    if plan.dtype != torch.int32 or opart.dtype != torch.float32 or ml.dtype != torch.float32:
        raise RuntimeError("decode workspace must be (float32, float32, int32)")
    return kv_heads, group, (opart, ml, plan)


def decode_attention(
    q: torch.Tensor,
    tables: RecordTables,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    scale: float,
    units: int,
    out: torch.Tensor,
    workspace: tuple[torch.Tensor, torch.Tensor, torch.Tensor],
    replan: bool,
) -> None:
    """Run split-KV decode attention for one query token per sequence.

    Args:
        q: BF16 ``[B, H * G, 128]`` queries (rows may be strided).
        tables: Record tables of this layer.
        block_table: int32 ``[B, max_pages]`` page ids (rows may be strided).
        seq_lens: int32 ``[B]`` context lengths; 0 yields a zero output row.
        scale: Softmax scale.
        units: Work-unit capacity per KV head, at least ``B``.
        out: BF16 ``[B, H * G, 128]`` output (rows may be strided).
        workspace: ``(opart, ml, plan)`` float, float, int32 tensors sized by
            :func:`workspace_elems`.
        replan: Recompute the work plan from ``seq_lens`` and ``units``; later
            calls with the same batch (the other layers of a step) may pass
            False to reuse it.

    Raises:
        ValueError: If the query group does not divide ``GQA``.
        RuntimeError: For rejected arguments or a failed launch.

    Async/thread-safety:
        Enqueues on the current CUDA stream; not synchronized; allocates nothing.
    """
    kv_heads, group, (opart, ml, plan) = _check_decode_args(q, tables, block_table, seq_lens, out, workspace)
    check(
        extension().fp_fused_decode(
            q.data_ptr(), q.stride(0), tables.rec_addr.data_ptr(), tables.rec_len.data_ptr(),
            tables.plut.data_ptr(), tables.slut.data_ptr(), block_table.data_ptr(),
            block_table.stride(0), seq_lens.data_ptr(), opart.data_ptr(), opart.numel(),
            ml.data_ptr(), ml.numel(), plan.data_ptr(), plan.numel(), out.data_ptr(),
            out.stride(0), q.shape[0], kv_heads, group, units, int(bool(replan)), float(scale),
            _sm_count(q.device.index if q.device.index is not None else torch.cuda.current_device()),
            stream_ptr(),
        )
    )


def plain_decode_attention(
    q: torch.Tensor,
    tables: RecordTables,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    scale: float,
    units: int,
    out: torch.Tensor,
    workspace: tuple[torch.Tensor, torch.Tensor, torch.Tensor],
    replan: bool,
) -> None:
    """Comparison arm: :func:`decode_attention` over plain BF16 records only.

    Every record the batch references must be raw (32,768 bytes in fragment
    order, ``rec_len > 2048``: open, overflow or never-coded blocks); the decode
    tables of ``tables`` are not read.  Same planner, pipeline, softmax and
    merge as the fused kernel without the decode step, so its time is the cost
    of a plain BF16 paged read of the same logical KV.  A coded record
    contributes zeros and sets ``DECODE_NOT_PLAIN`` in the status word.  The
    reference has no counterpart.

    Args, raises and stream behaviour: as :func:`decode_attention`.
    """
    kv_heads, group, (opart, ml, plan) = _check_decode_args(q, tables, block_table, seq_lens, out, workspace)
    check(
        extension().fp_plain_decode(
            q.data_ptr(), q.stride(0), tables.rec_addr.data_ptr(), tables.rec_len.data_ptr(),
            block_table.data_ptr(), block_table.stride(0), seq_lens.data_ptr(), opart.data_ptr(),
            opart.numel(), ml.data_ptr(), ml.numel(), plan.data_ptr(), plan.numel(), out.data_ptr(),
            out.stride(0), q.shape[0], kv_heads, group, units, int(bool(replan)), float(scale),
            _sm_count(q.device.index if q.device.index is not None else torch.cuda.current_device()),
            stream_ptr(),
        )
    )


def decode_status(workspace: tuple[torch.Tensor, torch.Tensor, torch.Tensor], units: int) -> int:
    """Read the status word of a decode workspace (synchronises the stream).

    Returns:
        0, or a combination of ``DECODE_*`` bits: the kernel gave up a bounded
        wait and the outputs of that step are invalid.
    """
    return int(workspace[2][2 + 4 * units + 1].item())


__all__ = [
    "GQA",
    "RecordTables",
    "DECODE_NOT_PLAIN",
    "DECODE_WAIT_TIMEOUT",
    "decode_attention",
    "decode_status",
    "decode_units",
    "plain_decode_attention",
    "workspace_elems",
]
