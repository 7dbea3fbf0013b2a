"""Output gather by the merge kernel through peer pointers.

* A group of one (no process group) must reproduce ``decode_attention`` bit for
  bit in both alternating copies and report no timeout.
* The bounded wait: a two-rank group whose second rank never signals (both
  "ranks" are buffers on this GPU; nothing ever writes the second arrival word)
  must return with ``PEER_WAIT_TIMEOUT`` set and leave the context usable.
* With two GPUs, two processes must each end up with the same ``[B, Hq, 128]``
  an NCCL all-gather of the per-rank outputs gives.
"""

from __future__ import annotations

import ctypes
import os

import numpy as np
import pytest
import torch

from benchmarks import workloads
from fragpack_b200.ops.fragpack_ext import FpPeers, check, extension, stream_ptr
from fragpack_b200.ops.fused_attn_decode import (
    RecordTables,
    decode_attention,
    decode_units,
    workspace_elems,
)
from fragpack_b200.ops.tp import PEER_WAIT_TIMEOUT, HeadGather, PeerGather

pytestmark = pytest.mark.gpu
SCALE = 128**-0.5


def _setup(device, head_slice=slice(None), seed=3):
    cfg = workloads.CONFIGS["c1"]
    work = workloads.build_decode_workload(cfg, device, seed=seed, head_slice=head_slice)
    B, H, G = work.cfg.batch, work.cfg.kv_heads, work.cfg.group
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    units = decode_units(B, H, sms)
    sizes = workspace_elems(H, units)
    ws = (torch.empty(sizes[0], device=device), torch.empty(sizes[1], device=device),
          torch.empty(sizes[2], dtype=torch.int32, device=device))
    gen = torch.Generator(device=device).manual_seed(17)
    q = torch.randn(B, H * G, 128, generator=gen, device=device).to(torch.bfloat16)
    tabs = RecordTables(*work.store.layer_tables(0))
    return work, tabs, q, units, ws


def test_group_of_one_matches_decode_attention() -> None:
    device = torch.device("cuda", torch.cuda.current_device())
    work, tabs, q, units, ws = _setup(device)
    want = torch.empty_like(q)
    decode_attention(q, tabs, work.block_table, work.seq_lens, SCALE, units, want, ws, replan=True)
    gather = PeerGather(q.shape[0], q.shape[1], device)
    gather.gathered.fill_(float("nan"))
    first = gather.decode(q, tabs, work.block_table, work.seq_lens, SCALE, units, ws, replan=True)
    second = gather.decode(q, tabs, work.block_table, work.seq_lens, SCALE, units, ws, replan=False)
    assert first.data_ptr() != second.data_ptr()
    for got in (first, second):
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    assert gather.status() == 0


def test_wait_for_a_silent_peer_times_out_cleanly() -> None:
    device = torch.device("cuda", torch.cuda.current_device())
    work, tabs, q, units, ws = _setup(device)
    B, heads = q.shape[0], q.shape[1]
    # Two ranks' buffers, both on this GPU; "rank 1" never runs.
    outs = [torch.zeros(2, B, 2 * heads, 128, dtype=torch.bfloat16, device=device) for _ in range(2)]
    flags = [torch.zeros(8, dtype=torch.int32, device=device) for _ in range(2)]
    epoch = torch.zeros(1, dtype=torch.int32, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    peers = FpPeers()
    for r in range(2):
        peers.out[r] = outs[r].data_ptr()
        peers.flag[r] = flags[r].data_ptr()
    peers.epoch, peers.status = epoch.data_ptr(), status.data_ptr()
    peers.world, peers.rank = 2, 0
    opart, ml, plan = ws
    H = tabs.rec_addr.shape[2]
    check(extension().fp_fused_decode_peers(
        q.data_ptr(), q.stride(0), tabs.rec_addr.data_ptr(), tabs.rec_len.data_ptr(),
        tabs.plut.data_ptr(), tabs.slut.data_ptr(), work.block_table.data_ptr(),
        work.block_table.stride(0), work.seq_lens.data_ptr(), opart.data_ptr(), opart.numel(),
        ml.data_ptr(), ml.numel(), plan.data_ptr(), plan.numel(), ctypes.byref(peers), 0,
        outs[0].stride(1), B, H, heads // H, units, 1, SCALE, 0, stream_ptr()))
    torch.cuda.synchronize()  # returns: the wait gave up after its limit
    assert int(status.item()) == PEER_WAIT_TIMEOUT
    assert flags[0][0].item() == 1 and flags[1][0].item() == 1  # rank 0 told both ranks
    assert flags[0][1].item() == 0  # nobody spoke for rank 1
    # Rank 0's heads reached both buffers; the context still works.
    want = torch.empty_like(q)
    decode_attention(q, tabs, work.block_table, work.seq_lens, SCALE, units, want, ws, replan=True)
    for r in range(2):
        assert torch.equal(outs[r][0][:, :heads].view(torch.int16), want.view(torch.int16))


def _two_rank_worker(rank: int, world: int, port: int, result) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        per = workloads.CONFIGS["c1"].kv_heads // world
        work, tabs, q, units, ws = _setup(device, slice(rank * per, (rank + 1) * per))
        local = torch.empty_like(q)
        decode_attention(q, tabs, work.block_table, work.seq_lens, SCALE, units, local, ws, replan=True)
        want = HeadGather(q.shape[0], q.shape[1], torch.bfloat16, device)(local).clone()
        gather = PeerGather(q.shape[0], q.shape[1], device)
        ok = True
        for call in range(4):
            got = gather.decode(q, tabs, work.block_table, work.seq_lens, SCALE, units, ws, replan=call == 0)
            torch.cuda.synchronize()
            ok &= bool(torch.equal(got.view(torch.int16), want.view(torch.int16)))
        ok &= gather.status() == 0
        result[rank] = int(ok)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_gather_equals_all_gather() -> None:
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    result = ctx.Array("i", [0, 0])
    procs = [ctx.Process(target=_two_rank_worker, args=(r, 2, 29533, result)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    assert all(p.exitcode == 0 for p in procs)
    assert list(result) == [1, 1]
