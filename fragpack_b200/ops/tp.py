"""Tensor-parallel helpers: KV-head sharding and the per-layer output gather.

Every (sequence, KV head) pair of decode attention is independent, so the path
shards by KV head with no exchange inside the kernels.  Rank ``r`` of ``tp``
holds the contiguous KV heads ``[r * H / tp, (r + 1) * H / tp)`` and the query
heads of those groups - the layout the reference declares for its tables
(``fragpack/integrations/vllm/backend.py:223-226``,
``fragpack/compression/attn_tables.py:70-93``).  The one exchange is an
all-gather of the attention output into the ``o_proj`` input layout
``[B, Hq, 128]`` after each layer.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def head_shard(rank: int, world: int, kv_heads: int) -> slice:
    """KV heads held by ``rank``.

    Raises:
        ValueError: If ``world`` does not divide ``kv_heads``.
    """
    if world <= 0 or kv_heads % world:
        raise ValueError(f"tensor-parallel size {world} must divide the {kv_heads} KV heads")
    per = kv_heads // world
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    return slice(rank * per, (rank + 1) * per)


class HeadGather:
    """All-gathers per-rank outputs ``[B, Hq / tp, 128]`` into ``[B, Hq, 128]``.

    NCCL (and gloo) gather rank-major, so the gathered buffer is
    ``[tp, B, Hq / tp, 128]``; one strided copy puts the heads of every rank
    side by side per sequence.  Buffers are allocated once.

    Args:
        batch: Sequences ``B``.
        local_q_heads: Query heads per rank.
        dtype, device: Of the outputs.
        group: Process group (default: the world).
    """

    def __init__(self, batch: int, local_q_heads: int, dtype: torch.dtype, device: torch.device,
                 group: dist.ProcessGroup | None = None) -> None:
        self.group = group
        self.world = dist.get_world_size(group)
        # Rank-major rows: rank r's [B, Hq / tp, 128] block is rows [r * B, (r + 1) * B).
        self.staged = torch.empty(self.world * batch, local_q_heads, 128, dtype=dtype, device=device)
        self.full = torch.empty(batch, self.world * local_q_heads, 128, dtype=dtype, device=device)

    def __call__(self, local_out: torch.Tensor) -> torch.Tensor:
        """Gather ``local_out`` (contiguous) from every rank; returns ``[B, Hq, 128]``."""
        dist.all_gather_into_tensor(self.staged, local_out, group=self.group)
        batch, heads = local_out.shape[0], local_out.shape[1]
        self.full.view(batch, self.world, heads, 128).copy_(
            self.staged.view(self.world, batch, heads, 128).transpose(0, 1)
        )
        return self.full


__all__ = ["HeadGather", "head_shard"]
