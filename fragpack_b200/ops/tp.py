"""Tensor-parallel helpers: KV-head sharding and the per-layer output gather.

Every (sequence, KV head) pair of decode attention is independent, so the path
shards by KV head with no exchange inside the kernels.  Rank ``r`` of ``tp``
holds the contiguous KV heads ``[r * H / tp, (r + 1) * H / tp)`` and the query
heads of those groups - the layout the reference declares for its tables
(``fragpack/integrations/vllm/backend.py:223-226``,
``fragpack/compression/attn_tables.py:70-93``).  The one exchange is the
gather of the attention output into the ``o_proj`` input layout
``[B, Hq, 128]`` after each layer, done either by the merge kernel itself
through peer pointers (:class:`PeerGather`, NVLink stores into every rank's
buffer) or by an NCCL all-gather after it (:class:`HeadGather`).
"""

from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from fragpack_b200.ops.fragpack_ext import FpPeers, check, extension, stream_ptr


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


PEER_WAIT_TIMEOUT = 1
MAX_PEERS = 8


class PeerGather:
    """Decode attention whose merge kernel writes every rank's ``o_proj`` input.

    Each rank owns one symmetric allocation holding two alternating gathered
    copies ``[2, B, Hq, 128]`` and its arrival words; every rank maps all of
    them (``torch.distributed._symmetric_memory``: plain peer mappings, the
    multicast binding is switched off).  :meth:`decode` runs fused decode
    attention for this rank's KV heads; the merge kernel stores this rank's
    heads of every row into every rank's copy over NVLink, signals its arrival
    and enqueues a bounded wait for the other ranks, so work enqueued afterwards
    on the same stream sees the complete ``[B, Hq, 128]``.

    Every rank must make the same sequence of calls.  Calls alternate between
    the two copies: a rank that is one call ahead writes the copy the slower
    ranks are not reading.  (Inside a CUDA graph the copy of each call is fixed
    at capture; capture an even number of calls per replay.)

    Args:
        batch: Sequences ``B``.
        local_q_heads: Query heads of this rank (KV heads x group).
        device: This rank's CUDA device.
        group: Process group (default: the world); ``None`` without an
            initialised process group means a group of one.
    """

    def __init__(self, batch: int, local_q_heads: int, device: torch.device,
                 group: dist.ProcessGroup | None = None) -> None:
        ready = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if ready else 1
        self.rank = dist.get_rank(group) if ready else 0
        if self.world > MAX_PEERS:
            raise ValueError(f"at most {MAX_PEERS} ranks, got {self.world}")
        self.batch, self.heads = batch, self.world * local_q_heads
        self.local_q_heads = local_q_heads
        out_bytes = 2 * batch * self.heads * 128 * 2
        flag_at = (out_bytes + 255) // 256 * 256
        total = flag_at + 256
        if self.world > 1:
            # No multicast object is ever bound to this memory: the kernels use
            # plain peer stores and loads only.
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm_mem

            self._buffer = symm_mem.empty(total, dtype=torch.uint8, device=device)
            self._buffer.zero_()
            handle = symm_mem.rendezvous(self._buffer, group if group is not None else dist.group.WORLD)
            bases = [int(p) for p in handle.buffer_ptrs]
            self._handle = handle
            torch.cuda.synchronize(device)
            dist.barrier(group)  # every rank's words are zero before anyone signals
        else:
            self._buffer = torch.zeros(total, dtype=torch.uint8, device=device)
            bases = [self._buffer.data_ptr()]
        if bases[self.rank] != self._buffer.data_ptr():
            raise RuntimeError("symmetric memory handle does not describe this rank's buffer")
        self.gathered = self._buffer[:out_bytes].view(torch.bfloat16).view(2, batch, self.heads, 128)
        self._epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self._status = torch.zeros(1, dtype=torch.int32, device=device)
        peers = FpPeers()
        for r, base in enumerate(bases):
            peers.out[r] = base
            peers.flag[r] = base + flag_at
        peers.epoch = self._epoch.data_ptr()
        peers.status = self._status.data_ptr()
        peers.world, peers.rank = self.world, self.rank
        self._peers = peers
        self._calls = 0

    def decode(self, q: torch.Tensor, tables, block_table: torch.Tensor, seq_lens: torch.Tensor,
               scale: float, units: int, workspace, replan: bool) -> torch.Tensor:
        """Fused decode attention + gather; returns this call's ``[B, Hq, 128]`` copy.

        Arguments as ``fused_attn_decode.decode_attention`` without ``out``.
        """
        from fragpack_b200.ops import fused_attn_decode as fad

        out = self.gathered[self._calls & 1]
        local_view = out[:, self.rank * self.local_q_heads : (self.rank + 1) * self.local_q_heads]
        kv_heads, group, (opart, ml, plan) = fad._check_decode_args(
            q, tables, block_table, seq_lens, local_view, workspace)
        check(
            extension().fp_fused_decode_peers(
                q.data_ptr(), q.stride(0), tables.rec_addr.data_ptr(), tables.rec_len.data_ptr(),
                tables.plut.data_ptr(), tables.slut.data_ptr(), block_table.data_ptr(),
                block_table.stride(0), seq_lens.data_ptr(), opart.data_ptr(), opart.numel(),
                ml.data_ptr(), ml.numel(), plan.data_ptr(), plan.numel(), ctypes.byref(self._peers),
                self._calls & 1, out.stride(0), q.shape[0], kv_heads, group, units,
                int(bool(replan)), float(scale),
                fad._sm_count(q.device.index if q.device.index is not None else torch.cuda.current_device()),
                stream_ptr(),
            )
        )
        self._calls += 1
        return out

    def status(self) -> int:
        """Status word (synchronises): ``PEER_WAIT_TIMEOUT`` if a peer did not arrive in time."""
        return int(self._status.item())


__all__ = ["HeadGather", "PEER_WAIT_TIMEOUT", "PeerGather", "head_shard"]
