"""Every device-side wait is bounded: make one run out, safely, and look at the result.

The decode attention kernel and the prefill decompressor stream records
through a ring of shared-memory slots; their consumer warps wait for a slot to
fill, their producer warp waits for a slot to drain.  The prefill attention
kernel's decoder, softmax and product-issuing warps hand tiles to one another
through mbarriers.  Each wait gives up after
a cycle budget, raises a status bit and lets the kernel finish its control
flow, so that a lost copy can never hang the GPU.  ``fp_debug_wait_limit``
shortens the budget to a millisecond and makes the producer leave one record
out (the prefill decoders: not report one page's K tile), which is exactly the
situation the bound exists for.  The tests check that
the call returns, that the status word says so, and that the next ordinary
call is bit-identical to the one before.
"""

from __future__ import annotations

import pytest
import torch

from benchmarks import workloads
from fragpack_b200.ops.fragpack_ext import check, extension
from fragpack_b200.ops.prefill_attn import PREFILL_WAIT_TIMEOUT, prefill_attention, prefill_status
from fragpack_b200.ops.fused_attn_decode import (
    DECODE_WAIT_TIMEOUT,
    RecordTables,
    decode_attention,
    decode_status,
    decode_units,
    workspace_elems,
)

pytestmark = pytest.mark.gpu
SCALE = 128**-0.5
SHORT_WAIT_CYCLES = 2_000_000  # about a millisecond


@pytest.fixture()
def short_waits():
    """Arms the hook for the test body and always restores the defaults."""

    def arm(skip_record: int) -> None:
        check(extension().fp_debug_wait_limit(SHORT_WAIT_CYCLES, skip_record))

    try:
        yield arm
    finally:
        check(extension().fp_debug_wait_limit(0, -1))
        torch.cuda.synchronize()


def _workload():
    device = torch.device("cuda", torch.cuda.current_device())
    cfg = workloads.CONFIGS["c1"]
    return cfg, workloads.build_decode_workload(cfg, device, seed=4)


def test_decode_wait_runs_out_and_the_next_call_is_clean(short_waits) -> None:
    cfg, work = _workload()
    device = work.block_table.device
    B, H, G = cfg.batch, cfg.kv_heads, cfg.group
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    units = decode_units(B, H, sms)
    sizes = workspace_elems(H, units)
    ws = (
        torch.empty(sizes[0], device=device),
        torch.empty(sizes[1], device=device),
        torch.empty(sizes[2], dtype=torch.int32, device=device),
    )
    tabs = RecordTables(*work.store.layer_tables(0))
    q = torch.randn(B, H * G, 128, device=device).to(torch.bfloat16)

    def run() -> torch.Tensor:
        out = torch.full_like(q, float("nan"))
        decode_attention(q, tabs, work.block_table, work.seq_lens, SCALE, units, out, ws, True)
        torch.cuda.synchronize()
        return out

    before = run()
    assert decode_status(ws, units) == 0
    # The second record of every CTA (the V record of its first page) never arrives.
    short_waits(1)
    run()
    assert decode_status(ws, units) & DECODE_WAIT_TIMEOUT
    check(extension().fp_debug_wait_limit(0, -1))
    after = run()
    assert decode_status(ws, units) == 0
    assert torch.equal(after, before)


def test_decompressor_wait_runs_out_and_the_next_call_is_clean(short_waits) -> None:
    cfg, work = _workload()
    device = work.block_table.device
    H = cfg.kv_heads
    blocks = work.block_table[0, :4].contiguous()

    def run():
        wk = torch.zeros(4, 128, H, 128, dtype=torch.bfloat16, device=device)
        wv = torch.zeros_like(wk)
        work.store.gather(0, blocks, wk, wv)
        torch.cuda.synchronize()
        return wk, wv

    before = run()
    assert work.store.gather_status() == 0
    short_waits(0)
    run()
    assert work.store.gather_status() & 1
    check(extension().fp_debug_wait_limit(0, -1))
    after = run()
    assert work.store.gather_status() == 0  # reading the status word also cleared it
    assert torch.equal(after[0], before[0]) and torch.equal(after[1], before[1])


def test_prefill_attention_wait_runs_out_and_the_next_call_is_clean(short_waits) -> None:
    cfg, work = _workload()
    device = work.block_table.device
    H, G = cfg.kv_heads, cfg.group
    tabs = RecordTables(*work.store.layer_tables(0))
    # Two requests re-attend the last 200 tokens of their cached contexts.
    ctx = work.seq_lens[:2].to(torch.int32).contiguous()
    n_new = 200
    assert int(ctx.min()) >= n_new
    q_start = torch.tensor([0, n_new, 2 * n_new], dtype=torch.int32, device=device)
    q = torch.randn(2 * n_new, H * G, 128, device=device).to(torch.bfloat16)
    block_table = work.block_table[:2].contiguous()

    def run() -> torch.Tensor:
        out = torch.full_like(q, float("nan"))
        prefill_attention(q, tabs, block_table, q_start, ctx, SCALE, out, n_new)
        torch.cuda.synchronize()
        return out

    before = run()
    assert prefill_status() == 0
    assert not torch.isnan(before.float()).any()
    # Page 1's K tile is never reported: the thread that issues the products gives up.
    short_waits(1)
    run()
    assert prefill_status() & PREFILL_WAIT_TIMEOUT
    check(extension().fp_debug_wait_limit(0, -1))
    after = run()
    assert prefill_status() == 0
    assert torch.equal(after, before)
