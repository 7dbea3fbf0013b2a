"""Parity on the benchmark configurations' own geometries, through the C ABI.

Reduced copies of the four GPU configurations keep what makes each one
different - KV heads, query group, ragged raw tails, heavy tails, junk, pages
per sequence - and cut layers, batch or context so that a case holds well
under a gigabyte.  For each:

* a sample of the store's records equals the oracle encoder's bytes
  (``attn_page.encode_record``; raw tails equal the staging layout);
* the prefill decompressor returns the written bits;
* decode attention matches fp32 attention over the written KV within the
  stated 1e-2 max-abs / 2e-3 mean-abs on BF16 outputs; outputs of magnitude
  above 1 (the x64 heavy tails of configuration 3 reach ~100, where BF16 is
  spaced 0.5 apart) are bounded relative to their magnitude (see
  ``tests/_util.assert_attention_close``); both forms are asserted.
"""

from __future__ import annotations

from dataclasses import replace

import numpy as np
import pytest
import torch

import oracle
from benchmarks import workloads
from fragpack_b200.compression import attn_page as ap
from fragpack_b200.ops.fused_attn_decode import (
    RecordTables,
    decode_attention,
    decode_status,
    decode_units,
    workspace_elems,
)
from tests._util import assert_attention_close, bits_of, record_bytes

pytestmark = pytest.mark.gpu
SCALE = 128**-0.5

CASES = {
    # Qwen3-30B-A3B-like: 4 KV heads, GQA 8, context 8192 (64 blocks per sequence).
    "c2": dict(base="c2", layers=2, batch=2),
    # Llama-3-8B-like: 8 KV heads, GQA 4, ragged contexts with raw tails, 0.5 % x64;
    # enough (sequence, head) pairs for the first-come-first-served item schedule.
    "c3": dict(base="c3", layers=1, batch=40, ctx_min=1000, ctx_max=1500),
    # Prefill stress: MHA, 32 KV heads, 0.9 % junk (most records still code).
    "c4": dict(base="c4", layers=1, batch=2, ctx_min=1024, ctx_max=1024, junk=0.009),
    # The same at the nominal 2 % junk: every record falls back to raw.
    "c4-junk2": dict(base="c4", layers=1, batch=1, ctx_min=512, ctx_max=512, junk=0.02),
    # The MHA geometry without junk, for attention (group 1, 32 KV heads).
    "c4-clean": dict(base="c4", layers=1, batch=2, ctx_min=1024, ctx_max=1024, junk=0.0),
    # Llama-3-70B-like: 8 KV heads, GQA 8, 256 blocks per sequence.
    "c5": dict(base="c5", layers=1, batch=2),
}


def _build(name: str):
    spec = dict(CASES[name])
    cfg = workloads.CONFIGS[spec.pop("base")]
    layers = spec.pop("layers")
    cfg = replace(cfg, **spec)
    device = torch.device("cuda", torch.cuda.current_device())
    work = workloads.build_decode_workload(
        cfg, device, seed=21, layers=layers, keep_layers=tuple(range(layers)), keep_seqs=2,
        overflow_records=8192,
    )
    return cfg, work


@pytest.fixture(scope="module", params=list(CASES))
def case(request):
    cfg, work = _build(request.param)
    yield request.param, cfg, work
    del work
    torch.cuda.empty_cache()


def test_records_equal_oracle_bytes(case) -> None:
    name, cfg, work = case
    rng = np.random.default_rng(5)
    bt = work.block_table.cpu().numpy()
    layers = work.cfg.layers
    checked = raw_seen = spilled = 0
    for b in range(min(2, cfg.batch)):
        tokens = int(work.lens_host[b])
        pages = (tokens + 127) // 128
        # Every head of a few pages: always the first and the last (the open
        # tail where the context is ragged), the others picked at random.
        picks = sorted({0, pages - 1, *rng.integers(0, pages, size=6).tolist()})
        for layer in range(layers):
            src = bits_of(work.sample[(layer, b)])  # [2, tokens, H, 128]
            for page in picks:
                full = (page + 1) * 128 <= tokens
                for kv in range(2):
                    for h in range(work.cfg.kv_heads):
                        rec = np.zeros((128, 128), np.uint16)
                        rows = src[kv, page * 128 : (page + 1) * 128, h]
                        rec[: rows.shape[0]] = rows
                        got = record_bytes(work, layer, int(bt[b, page]), kv, h)
                        if full:
                            want = oracle.encode_record(rec, work.table[layer, kv, h], kv)
                            if len(want) == ap.RAW_RECORD_BYTES:
                                raw_seen += 1
                            elif len(got) == ap.RAW_RECORD_BYTES:
                                # A record that codes but found its block's page full
                                # is kept raw in the overflow pool (a spill); only the
                                # junk-laden MHA pages are that tight.
                                assert name.startswith("c4"), (name, layer, b, page, kv, h)
                                base = work.store.overflow.data_ptr()
                                addr = int(work.store.rec_addr[layer, int(bt[b, page]), kv, h].item())
                                assert base <= addr < base + work.store.overflow.numel()
                                want = oracle.raw_record(rec, kv)
                                spilled += 1
                        else:
                            # An open block is its staging record; positions past the
                            # last token were never written (staging starts zeroed).
                            want = oracle.raw_record(rec, kv)
                        assert len(got) == len(want), (name, layer, b, page, kv, h)
                        assert got == want, (name, layer, b, page, kv, h)
                        checked += 1
    assert checked > 0
    if name == "c4-junk2":
        assert raw_seen == checked  # 2 % junk: nothing codes
    if name in ("c2", "c5", "c4-clean"):
        assert raw_seen == 0
    if not name.startswith("c4"):
        assert spilled == 0


def test_decompressor_returns_written_bits(case) -> None:
    name, cfg, work = case
    H = work.cfg.kv_heads
    bt = work.block_table.cpu().numpy()
    for b in range(min(2, cfg.batch)):
        tokens = int(work.lens_host[b])
        pages = (tokens + 127) // 128
        blocks = torch.from_numpy(bt[b, :pages].copy()).to(work.block_table.device)
        wk = torch.empty(pages, 128, H, 128, dtype=torch.bfloat16, device=blocks.device)
        wv = torch.empty_like(wk)
        for layer in range(work.cfg.layers):
            work.store.gather(layer, blocks, wk, wv)
            src = work.sample[(layer, b)]
            assert torch.equal(wk.view(-1, H, 128)[:tokens], src[0]), (name, layer, b)
            assert torch.equal(wv.view(-1, H, 128)[:tokens], src[1]), (name, layer, b)
    assert work.store.gather_status() == 0


def test_decode_attention_within_the_stated_tolerance(case) -> None:
    name, cfg, work = case
    if cfg.junk:
        # Junk scalars are arbitrary finite bit patterns, up to 3e38: their scores
        # overflow fp32 in any attention, the fp32 reference included.  Configuration
        # 4 measures the prefill side; its geometry is attended in the junk-free case.
        pytest.skip("random-bit-pattern KV overflows fp32 attention")
    device = work.block_table.device
    B, H, G = work.cfg.batch, work.cfg.kv_heads, work.cfg.group
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    if name == "c3":
        # More (sequence, head) pairs than resident CTAs: the kernel instantiation
        # with the first-come-first-served item schedule is the one launched.
        assert B * H > 2 * sms
    units = decode_units(B, H, sms)
    sizes = workspace_elems(H, units)
    ws = (
        torch.empty(sizes[0], device=device),
        torch.empty(sizes[1], device=device),
        torch.empty(sizes[2], dtype=torch.int32, device=device),
    )
    gen = torch.Generator(device=device).manual_seed(9)
    for layer in range(work.cfg.layers):
        q = torch.randn(B, H * G, 128, generator=gen, device=device).to(torch.bfloat16)
        out = torch.full_like(q, float("nan"))
        tabs = RecordTables(*work.store.layer_tables(layer))
        decode_attention(q, tabs, work.block_table, work.seq_lens, SCALE, units, out, ws, layer == 0)
        torch.cuda.synchronize()
        assert decode_status(ws, units) == 0
        assert not torch.isnan(out).any()
        for b in range(min(2, B)):
            kv = work.sample[(layer, b)].float().cpu()
            for h in range(H):
                ref = oracle.attention_fp32(
                    q[b, h * G : (h + 1) * G].float().cpu(), kv[0][:, h], kv[1][:, h], SCALE
                )
                assert_attention_close(out[b, h * G : (h + 1) * G], ref, (name, layer, b, h))


def test_back_to_back_launches_on_one_plan_keep_their_item_counters_apart(case) -> None:
    """Many launches of the first-come-first-served schedule in flight on one plan.

    Each attention launch since the plan was made draws its items from its own
    counter, found from the order in which its CTAs arrive; consecutive
    launches overlap (programmatic dependent launch), so a launch that drew
    from a neighbour's counter would skip or repeat items.  Forty-eight
    launches are queued without a synchronisation in between, each with its
    own queries and output, and every output must equal, bit for bit, what the
    same call returns when it runs alone on a fresh plan.
    """
    name, cfg, work = case
    if name != "c3":
        pytest.skip("the first-come-first-served schedule needs more (sequence, head) pairs than CTAs")
    device = work.block_table.device
    B, H, G = work.cfg.batch, work.cfg.kv_heads, work.cfg.group
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    assert B * H > 2 * sms
    units = decode_units(B, H, sms)
    sizes = workspace_elems(H, units)
    ws = (
        torch.empty(sizes[0], device=device),
        torch.empty(sizes[1], device=device),
        torch.empty(sizes[2], dtype=torch.int32, device=device),
    )
    tabs = RecordTables(*work.store.layer_tables(0))
    gen = torch.Generator(device=device).manual_seed(77)
    launches = 48
    qs = [torch.randn(B, H * G, 128, generator=gen, device=device).to(torch.bfloat16) for _ in range(launches)]
    alone = []
    for q in qs:
        out = torch.full_like(q, float("nan"))
        decode_attention(q, tabs, work.block_table, work.seq_lens, SCALE, units, out, ws, True)
        torch.cuda.synchronize()
        assert decode_status(ws, units) == 0
        alone.append(out)
    queued = [torch.full_like(q, float("nan")) for q in qs]
    for i, (q, out) in enumerate(zip(qs, queued)):
        decode_attention(q, tabs, work.block_table, work.seq_lens, SCALE, units, out, ws, i == 0)
    torch.cuda.synchronize()
    assert decode_status(ws, units) == 0
    for i, (a, b) in enumerate(zip(alone, queued)):
        assert torch.equal(a, b), f"launch {i} differs from the same call run alone"
