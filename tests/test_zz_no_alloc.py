"""The allocation-free decode entry point against the regular one.

``fp_fused_decode_noalloc`` serves hosts that cannot allocate device memory
for this library (an engine that owns every byte of the device, a plugin under
a foreign memory planner, a worker with a frozen allocator): it keeps the
split-KV workspace in a fixed array inside the library instead of taking it
from the caller.  This file is collected last on purpose, so that a run that
stops at the first failure has already run every other test; it passes alone
in a fresh process as well as after the others.

The check: two calls in a row through the C ABI (the second one reusing the
plan left in the shared array by the first, then a third with new lengths)
must give exactly what ``fp_fused_decode`` gives with a caller-owned workspace
- the same kernels run with the same plan, and the merge order is fixed by the
plan, so the outputs are equal bit for bit - and, like every decode test, must
match fp32 attention over the written KV (the oracle) within 1e-2 max-abs and
2e-3 mean-abs (relative to the magnitude for outputs above 1).
"""

from __future__ import annotations

import pytest
import torch

import oracle
from benchmarks import workloads
from tests._util import assert_attention_close
from fragpack_b200.ops.fragpack_ext import check, extension, stream_ptr
from fragpack_b200.ops.fused_attn_decode import (
    RecordTables,
    decode_attention,
    decode_units,
    workspace_elems,
)

pytestmark = pytest.mark.gpu
SCALE = 128**-0.5


def _noalloc(q, tabs, block_table, seq_lens, out, kv_heads, group, units, replan) -> int:
    sms = torch.cuda.get_device_properties(q.device).multi_processor_count
    return extension().fp_fused_decode_noalloc(
        q.data_ptr(), q.stride(0), tabs.rec_addr.data_ptr(), tabs.rec_len.data_ptr(),
        tabs.plut.data_ptr(), tabs.slut.data_ptr(), block_table.data_ptr(), block_table.stride(0),
        seq_lens.data_ptr(), out.data_ptr(), out.stride(0), q.shape[0], kv_heads, group, units,
        int(replan), SCALE, sms, stream_ptr(),
    )


def test_noalloc_matches_workspace_entry_point_twice_in_a_row() -> None:
    device = torch.device("cuda", torch.cuda.current_device())
    cfg = workloads.CONFIGS["c1"]
    work = workloads.build_decode_workload(cfg, device, seed=11, keep_layers=(0,), keep_seqs=cfg.batch)
    H, G, B = cfg.kv_heads, cfg.group, cfg.batch
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    units = decode_units(B, H, sms)
    assert H * units <= 4096
    sizes = workspace_elems(H, units)
    ws = (
        torch.empty(sizes[0], device=device),
        torch.empty(sizes[1], device=device),
        torch.empty(sizes[2], dtype=torch.int32, device=device),
    )
    tabs = RecordTables(*work.store.layer_tables(0))
    gen = torch.Generator(device=device).manual_seed(5)
    lens_a = work.seq_lens.clone()
    lens_b = torch.tensor([300, 77], dtype=torch.int32, device=device)
    # (lengths, replan): the second call reuses the first call's plan.
    for lens, replan in ((lens_a, True), (lens_a, False), (lens_b, True)):
        q = torch.randn(B, H * G, 128, generator=gen, device=device).to(torch.bfloat16)
        want = torch.full_like(q, float("nan"))
        decode_attention(q, tabs, work.block_table, lens, SCALE, units, want, ws, replan)
        got = torch.full_like(q, float("nan"))
        check(_noalloc(q, tabs, work.block_table, lens, got, H, G, units, replan))
        torch.cuda.synchronize()
        assert not torch.isnan(got).any()
        assert torch.equal(got, want)
        # Against the oracle: fp32 attention over the first `lens` written tokens.
        for b in range(B):
            kv = work.sample[(0, b)].float().cpu()
            n = int(lens[b].item())
            for h in range(H):
                ref = oracle.attention_fp32(
                    q[b, h * G : (h + 1) * G].float().cpu(), kv[0][:n, h], kv[1][:n, h], SCALE
                )
                assert_attention_close(got[b, h * G : (h + 1) * G], ref, (n, b, h))


def test_noalloc_rejects_sizes_beyond_its_scratch() -> None:
    device = torch.device("cuda", torch.cuda.current_device())
    dummy = torch.zeros(64, dtype=torch.int64, device=device)
    q = torch.zeros(1, 8, 128, dtype=torch.bfloat16, device=device)
    tabs = RecordTables(dummy, dummy, dummy, dummy)
    rc = _noalloc(q, tabs, dummy, dummy, q, kv_heads=1, group=8, units=4097, replan=True)
    assert rc != 0
    message = extension().fp_last_error().decode()
    assert "4096" in message and "units" in message
    rc = _noalloc(q, tabs, dummy, dummy, q, kv_heads=8, group=8, units=1024, replan=True)
    assert rc != 0
