"""The multi-rank path on CPU: KV-head sharding and the output gather (gloo, world size 2)."""

from __future__ import annotations

import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fragpack_b200.ops.tp import HeadGather, head_shard


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, result) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        batch, kv_heads, group = 3, 4, 8
        full = torch.arange(batch * kv_heads * group * 128, dtype=torch.float32).reshape(
            batch, kv_heads * group, 128
        )
        heads = head_shard(rank, world, kv_heads)
        local = full[:, heads.start * group : heads.stop * group].contiguous()
        gather = HeadGather(batch, local.shape[1], local.dtype, local.device)
        for _ in range(2):  # buffers are reused across layers
            got = gather(local)
            assert torch.equal(got, full)
        # Max-over-ranks timing reduction used by the benchmark.
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert t.item() == world
        result.put((rank, True))
    finally:
        dist.destroy_process_group()


def test_head_shard_and_gather_world_size_2() -> None:
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, result)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert sorted(result.get(timeout=5)[0] for _ in range(2)) == [0, 1]


def test_head_shard_partitions_heads() -> None:
    for world in (1, 2, 4, 8):
        seen = np.concatenate([np.arange(8)[head_shard(r, world, 8)] for r in range(world)])
        assert np.array_equal(seen, np.arange(8))
