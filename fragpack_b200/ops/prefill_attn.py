"""Causal prefill attention directly over FragPack KV records (sm_100a, tcgen05).

The reference's prefill path decompresses a request's blocks into a BF16
workspace (``HbmKvStore.gather``) and runs FlashAttention over it
(``fragpack/integrations/vllm/backend.py:560-575``).
:func:`prefill_attention` does both in one kernel: records are decoded into
shared-memory operand tiles and multiplied on the tensor cores, and the
decompressed KV never goes to HBM.  The new tokens of the step must already be
in the store (``HbmKvStore.write`` runs before attention, as in the reference).
"""

from __future__ import annotations

import torch

from fragpack_b200.ops.fragpack_ext import check, extension, require_cuda, stream_ptr
from fragpack_b200.ops.fused_attn_decode import GQA, RecordTables

PREFILL_WAIT_TIMEOUT = 1
_STATUS: dict[int, torch.Tensor] = {}


def _status_word(device: torch.device) -> torch.Tensor:
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _STATUS:
        _STATUS[index] = torch.zeros(1, dtype=torch.int32, device=device)
    return _STATUS[index]


def prefill_attention(
    q: torch.Tensor,
    tables: RecordTables,
    block_table: torch.Tensor,
    q_start: torch.Tensor,
    ctx_lens: torch.Tensor,
    scale: float,
    out: torch.Tensor,
    max_query_tokens: int,
) -> None:
    """Attend every request's new tokens over its whole context, causally.

    Request ``r`` owns the query rows ``q_start[r] .. q_start[r + 1]``; they are
    the last tokens of its context of ``ctx_lens[r]`` tokens, whose pages are
    ``block_table[r]``.  Query ``i`` of the request sits at position
    ``ctx_lens[r] - n_r + i`` and sees the keys up to and including itself.

    Args:
        q: BF16 ``[T, H * G, 128]`` queries (rows may be strided by a 16-byte multiple).
        tables: Record tables of this layer.
        block_table: int32 ``[R, max_pages]`` page ids.
        q_start: int32 ``[R + 1]`` first query row of each request.
        ctx_lens: int32 ``[R]`` context lengths, new tokens included.
        scale: Softmax scale.
        out: BF16 ``[T, H * G, 128]`` output.
        max_query_tokens: The most query tokens any request has (sizes the grid).

    Raises:
        ValueError: If the query group does not divide ``GQA``.
        RuntimeError: For rejected arguments or a failed launch.

    Async/thread-safety:
        Enqueues on the current CUDA stream; not synchronized.  The first call
        on a device allocates a 4-byte status word (see :func:`prefill_status`).
    """
    kv_heads = tables.rec_addr.shape[2]
    group = q.shape[1] // kv_heads
    if group == 0 or group * kv_heads != q.shape[1] or GQA % group:
        raise ValueError(f"query heads {q.shape[1]} need a group dividing {GQA}")
    require_cuda(q, "q")
    if q.dim() != 3 or q.shape[2] != 128 or q.stride(2) != 1 or q.stride(1) != 128:
        raise RuntimeError("q must be [T, H, 128] with contiguous heads")
    if out.shape != q.shape or out.stride(2) != 1 or out.stride(1) != 128:
        raise RuntimeError("out must be [T, H, 128] with contiguous heads")
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise RuntimeError("q and out must be bfloat16")
    if block_table.dtype != torch.int32 or block_table.stride(1) != 1:
        raise RuntimeError("block_table must be int32 with contiguous rows")
    if q_start.dtype != torch.int32 or ctx_lens.dtype != torch.int32:
        raise RuntimeError("q_start and ctx_lens must be int32")
    if q_start.numel() != ctx_lens.numel() + 1:
        raise RuntimeError("q_start needs one more entry than ctx_lens")
    check(
        extension().fp_prefill_attention(
            q.data_ptr(), q.stride(0), tables.rec_addr.data_ptr(), tables.rec_len.data_ptr(),
            tables.plut.data_ptr(), tables.slut.data_ptr(), block_table.data_ptr(),
            block_table.stride(0), q_start.data_ptr(), ctx_lens.data_ptr(), out.data_ptr(),
            out.stride(0), ctx_lens.numel(), int(max_query_tokens), kv_heads, group, float(scale),
            _status_word(q.device).data_ptr(), stream_ptr(),
        )
    )


def prefill_status(device: torch.device | None = None) -> int:
    """Status word of the prefill kernel on ``device`` (synchronises) and clear it.

    Returns:
        0, or ``PREFILL_WAIT_TIMEOUT`` if a bounded device-side wait ran out
        since the last read (the outputs of those calls are invalid).
    """
    device = device or torch.device("cuda", torch.cuda.current_device())
    word = _status_word(device)
    value = int(word.item())
    word.zero_()
    return value


__all__ = ["PREFILL_WAIT_TIMEOUT", "prefill_attention", "prefill_status"]
