"""Prefill attention over compressed records against fp32 causal attention.

The kernel stands where the reference gathers a request's blocks into a BF16
workspace and calls FlashAttention (``backend.py:560-575``); parity is the one
the reference's GPU tests use for attention: fp32 ``softmax(q k^T scale) v``
over the written BF16 KV, here with the causal mask of a prefill chunk (query
``i`` of ``n`` sits at position ``context - n + i``).  Cases cover the query
groups 1 (the MHA geometry of configuration 4), 4 and 8, a first chunk, a later
chunk over cached coded blocks plus an open raw tail, and ragged requests.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

import oracle
from benchmarks import synth
from fragpack_b200.compression import attn_page as ap
from fragpack_b200.compression.attn_tables import device_tables
from fragpack_b200.ops.fused_attn_decode import RecordTables
from fragpack_b200.ops.hbm_kv import HbmKvStore, page_bytes
from fragpack_b200.ops.prefill_attn import prefill_attention, prefill_status
from tests._util import assert_attention_close

pytestmark = pytest.mark.gpu
T, D = 128, 128
SCALE = D**-0.5


class Requests:
    """A one-layer store that is fed request chunks and remembers the written KV."""

    def __init__(self, kv_heads: int, requests: int, max_tokens: int, seed: int,
                 unit_scales: bool = False) -> None:
        self.H = kv_heads
        self.dev = torch.device("cuda")
        self.gen = torch.Generator(device=self.dev).manual_seed(seed)
        scales = torch.from_numpy(synth.channel_scales(seed, 1, kv_heads)[0]).to(self.dev)
        if unit_scales:
            scales = torch.ones_like(scales)
        self.scales = scales
        cal = synth.kv_tokens_torch(self.gen, scales, 4 * T)
        high = (cal.view(torch.int16).to(torch.int32) >> 8) & 0xFF
        table = np.empty((1, 2, kv_heads, ap.TABLE_ENTRIES), np.uint8)
        for k in range(2):
            for h in range(kv_heads):
                table[0, k, h] = oracle.calibrate_table(high[k, :, h].reshape(-1).cpu().numpy().astype(np.uint8))
        pages = -(-max_tokens // T)
        self.nb = requests * pages + 1
        self.cache = [torch.zeros((self.nb, page_bytes(kv_heads)), dtype=torch.uint8, device=self.dev)]
        self.store = HbmKvStore(self.cache, kv_heads, device_tables(table, self.dev),
                                max_tokens=requests * max_tokens, staging_slots=requests + 1,
                                overflow_records=64)
        self.blocks = [list(range(1 + r * pages, 1 + (r + 1) * pages)) for r in range(requests)]
        self.kv = [torch.empty(2, 0, kv_heads, D, dtype=torch.bfloat16, device=self.dev) for _ in range(requests)]
        self.block_table = torch.tensor(self.blocks, dtype=torch.int32, device=self.dev)

    def step(self, new_tokens: list[int], group: int):
        """Write `new_tokens[r]` tokens to each request, attend, encode, commit; returns (out, ref inputs)."""
        slots, starts = [], [0]
        for r, n in enumerate(new_tokens):
            have = self.kv[r].shape[1]
            slots += [self.blocks[r][p // T] * T + p % T for p in range(have, have + n)]
            starts.append(starts[-1] + n)
        total = starts[-1]
        slot_t = torch.tensor(slots, dtype=torch.int64, device=self.dev)
        live = np.array([b for blk in self.blocks for b in blk], np.int32)
        closes = sum((self.kv[r].shape[1] + n) // T - self.kv[r].shape[1] // T for r, n in enumerate(new_tokens))
        self.store.prepare(slot_t, total, live)
        kv = synth.kv_tokens_torch(self.gen, self.scales, total)
        self.store.write(0, kv[0], kv[1], slot_t)
        for r, n in enumerate(new_tokens):
            self.kv[r] = torch.cat([self.kv[r], kv[:, starts[r] : starts[r + 1]]], dim=1)
        q = torch.randn(total, self.H * group, D, generator=self.gen, device=self.dev).to(torch.bfloat16)
        out = torch.full_like(q, float("nan"))
        ctx = torch.tensor([self.kv[r].shape[1] for r in range(len(new_tokens))], dtype=torch.int32, device=self.dev)
        q_start = torch.tensor(starts, dtype=torch.int32, device=self.dev)
        prefill_attention(q, RecordTables(*self.store.layer_tables(0)), self.block_table, q_start, ctx,
                          SCALE, out, max(new_tokens))
        self.store.encode(0, max(closes, 1))
        self.store.commit()
        torch.cuda.synchronize()
        assert prefill_status() == 0
        self.store.stats()
        return q, out, starts

    def check(self, q, out, starts, new_tokens, group: int) -> None:
        for r, n in enumerate(new_tokens):
            if n == 0:
                continue
            context = self.kv[r].shape[1]
            k, v = self.kv[r][0].float().cpu(), self.kv[r][1].float().cpu()
            mask = torch.ones(n, context, dtype=torch.bool).tril(context - n)
            for h in range(self.H):
                for g in range(group):
                    qq = q[starts[r] : starts[r + 1], h * group + g].float().cpu()
                    s = (qq @ k[:, h].T) * SCALE
                    s = s.masked_fill(~mask, float("-inf"))
                    ref = torch.softmax(s, -1) @ v[:, h]
                    assert_attention_close(out[starts[r] : starts[r + 1], h * group + g], ref, (r, h, g))


@pytest.mark.parametrize("kv_heads, group", [(8, 1), (2, 4), (2, 8)])
def test_chunked_prefill_matches_fp32_causal_attention(kv_heads: int, group: int) -> None:
    reqs = Requests(kv_heads, requests=2, max_tokens=1024, seed=11 + group)
    # First chunks: request 0 fills two blocks and opens a third, request 1 stays inside one block.
    first = [300, 77]
    q, out, starts = reqs.step(first, group)
    reqs.check(q, out, starts, first, group)
    # Later chunks over cached (coded) blocks plus the open tail; request 1 crosses a block boundary.
    second = [212, 130]
    q, out, starts = reqs.step(second, group)
    reqs.check(q, out, starts, second, group)
    # A short chunk and a request without new tokens.
    third = [5, 0]
    q, out, starts = reqs.step(third, group)
    reqs.check(q, out, starts, third, group)


def test_long_context_wraps_every_barrier_many_times() -> None:
    """Twenty-odd pages per request: every ring slot, tile and barrier phase is reused many times.

    Unit channel scales: with thousands of query rows per head and the
    lognormal scales of the other cases (V values near 10 on some heads) the
    worst of the outputs near magnitude 1 is off by 1.1e-2 in any BF16
    attention - torch's BF16 SDPA returns the same values on those elements -
    which is a property of the data, not of the kernel under test.
    """
    reqs = Requests(2, requests=2, max_tokens=3328, seed=29, unit_scales=True)
    first = [2500, 1300]
    q, out, starts = reqs.step(first, 2)
    reqs.check(q, out, starts, first, 2)
    second = [700, 1911]  # request 1 ends one token short of a block boundary
    q, out, starts = reqs.step(second, 2)
    reqs.check(q, out, starts, second, 2)


def test_rejects_bad_arguments() -> None:
    reqs = Requests(2, requests=1, max_tokens=256, seed=3)
    tabs = RecordTables(*reqs.store.layer_tables(0))
    q = torch.zeros(4, 6, D, dtype=torch.bfloat16, device=reqs.dev)  # 3 query heads per KV head
    one = torch.tensor([0, 4], dtype=torch.int32, device=reqs.dev)
    ctx = torch.tensor([4], dtype=torch.int32, device=reqs.dev)
    with pytest.raises(ValueError):
        prefill_attention(q, tabs, reqs.block_table, one, ctx, SCALE, torch.empty_like(q), 4)
    q = torch.zeros(4, 4, D, dtype=torch.bfloat16, device=reqs.dev)
    with pytest.raises(RuntimeError):
        prefill_attention(q, tabs, reqs.block_table, one[:1], ctx, SCALE, torch.empty_like(q), 4)
    with pytest.raises(RuntimeError):  # the kernel takes row maxima on the raw scores
        prefill_attention(q, tabs, reqs.block_table, one, ctx, -SCALE, torch.empty_like(q), 4)
