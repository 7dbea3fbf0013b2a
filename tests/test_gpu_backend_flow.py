"""A miniature engine loop through the backend's per-layer flow.

Two requests go through chunked prefill and several decode steps with the
metadata the vLLM builder would produce (``backend.py:274-323``) and
``run_layer`` for every layer (``backend.py:536-579``): write, decode rows
through the fused kernel, prefill rows over the decompressed workspace, encode
of the blocks closed in the step, commit.  Every output row must match fp32
causal attention over that request's whole history, and the store must not
have dropped anything.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from fragpack_b200.compression.attn_tables import calibrate, device_tables
from fragpack_b200.integrations.vllm.backend import (
    FragPackMetadata,
    count_closes,
    plan_prefill_groups,
    run_layer,
)
from fragpack_b200.ops.fused_attn_decode import RecordTables, decode_units, workspace_elems
from fragpack_b200.ops.hbm_kv import HbmKvStore, page_bytes

pytestmark = pytest.mark.gpu

L, H, G, D, T, NB = 2, 2, 4, 128, 128, 16
HQ = H * G
SCALE = D**-0.5
MAX_TOKENS, WORKSPACE_PAGES = 512, 6


class Request:
    def __init__(self, blocks):
        self.blocks = blocks
        self.computed = 0
        # history[layer] = (K, V) float32 [tokens, H, D]
        self.history = [(torch.zeros(0, H, D), torch.zeros(0, H, D)) for _ in range(L)]


def _reference(q, k, v, n_new):
    """fp32 causal attention of the last n_new positions; q [n_new, HQ, D], k/v [ctx, H, D]."""
    ctx = k.shape[0]
    out = torch.empty(n_new, HQ, D)
    for h in range(H):
        qh = q[:, h * G : (h + 1) * G].float()                      # [n, G, D]
        logits = torch.einsum("ngd,td->ngt", qh, k[:, h]) * SCALE
        pos = torch.arange(ctx - n_new, ctx)[:, None, None]
        logits = logits.masked_fill(torch.arange(ctx)[None, None, :] > pos, float("-inf"))
        out[:, h * G : (h + 1) * G] = torch.einsum("ngt,td->ngd", logits.softmax(-1), v[:, h])
    return out


@pytest.mark.parametrize("fused_prefill", [True, False])
def test_chunked_prefill_then_decode_matches_fp32_attention(fused_prefill: bool) -> None:
    """Prefill rows over the compressed records (one kernel) or over the decompressed workspace."""
    device = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator().manual_seed(41)
    sample = (torch.randn(8, L, 2, T, H, D, generator=gen) * 0.5).to(torch.bfloat16)
    table = calibrate(sample.view(torch.int16).numpy().view(np.uint16))
    caches = [torch.empty(NB, page_bytes(H), dtype=torch.uint8, device=device) for _ in range(L)]
    store = HbmKvStore(caches, H, device_tables(table, device), MAX_TOKENS, staging_slots=2,
                       overflow_records=64)
    layer_tables = [RecordTables(*store.layer_tables(i)) for i in range(L)]
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    sizes = workspace_elems(H, decode_units(2, H, sms))
    workspace = (torch.empty(sizes[0], device=device), torch.empty(sizes[1], device=device),
                 torch.empty(sizes[2], dtype=torch.int32, device=device))
    wk = torch.empty(WORKSPACE_PAGES, T, H, D, dtype=torch.bfloat16, device=device)
    wv = torch.empty_like(wk)

    a, b = Request([3, 7, 1, 9]), Request([5, 2, 8, 4])
    # (request, new tokens) per step; decode rows (one token, context already there) come first.
    steps = [
        [(a, 200), (b, 150)],      # two prefill chunks
        [(a, 1), (b, 100)],        # a decodes (closes nothing), b continues its prefill past a block end
        [(a, 1), (b, 1)],
        [(b, 1), (a, 55)],         # a chunk on a running request: a's 2nd block closes at 256
        [(a, 1), (b, 5)],
    ]
    for rows in steps:
        decodes = [(r, n) for r, n in rows if n == 1 and r.computed > 0]
        prefills = [(r, n) for r, n in rows if not (n == 1 and r.computed > 0)]
        ordered = decodes + prefills
        nd, num_reqs = len(decodes), len(ordered)
        qlen = np.array([n for _, n in ordered], np.int64)
        seq = np.array([r.computed + n for r, n in ordered], np.int64)
        qsl = np.concatenate(([0], np.cumsum(qlen)))
        total = int(qsl[-1])
        slots = np.concatenate([
            np.array([r.blocks[p // T] * T + p % T for p in range(r.computed, r.computed + n)], np.int64)
            for r, n in ordered
        ])
        slot_t = torch.from_numpy(slots).to(device)
        block_table = torch.tensor([r.blocks for r, _ in ordered], dtype=torch.int32, device=device)
        # Blocks partially written before this step keep their staging slot.
        live = np.array([r.blocks[r.computed // T] for r, _ in ordered if r.computed % T], np.int32)
        store.prepare(slot_t, total, live)
        md = FragPackMetadata(
            store=store, layer_tables=layer_tables, layer_index={}, last_layer=L - 1,
            slot_mapping=slot_t, num_tokens=total, num_decodes=nd,
            decode_block_table=block_table[:nd],
            decode_seq_lens=torch.from_numpy(seq[:nd].astype(np.int32)).to(device),
            units=decode_units(max(nd, 1), H, sms), decode_workspace=workspace,
            max_close=min(max(count_closes(seq, qlen), nd), MAX_TOKENS),
            prefills=plan_prefill_groups(block_table, nd, num_reqs, qsl, seq, WORKSPACE_PAGES, device)
            if len(prefills) else [],
            wk=wk, wv=wv,
        )
        for layer in range(L):
            q = (torch.randn(total, HQ, D, generator=gen)).to(torch.bfloat16)
            k = (torch.randn(total, H, D, generator=gen) * 0.5).to(torch.bfloat16)
            v = (torch.randn(total, H, D, generator=gen) * 0.5).to(torch.bfloat16)
            out = torch.full((total, HQ, D), float("nan"), dtype=torch.bfloat16, device=device)
            run_layer(md, layer, q.to(device), k.to(device), v.to(device), out, SCALE,
                      fused_prefill=fused_prefill)
            got = out.float().cpu()
            for i, (r, n) in enumerate(ordered):
                t0, t1 = int(qsl[i]), int(qsl[i + 1])
                hk, hv = r.history[layer]
                hk = torch.cat([hk, k[t0:t1].float()])
                hv = torch.cat([hv, v[t0:t1].float()])
                r.history[layer] = (hk, hv)
                want = _reference(q[t0:t1], hk, hv, n)
                err = (got[t0:t1] - want).abs()
                # The decode parity bar: 1e-2 max-abs, 2e-3 mean-abs on BF16 outputs.
                assert float(err.max()) <= 1e-2 and float(err.mean()) <= 2e-3, (layer, i, n)
        for r, n in ordered:
            r.computed += n
    stats = store.stats()
    assert stats.err_staging == 0 and stats.err_overflow == 0
    # Both requests passed 256 tokens: two closed blocks each, K and V records of every head and layer.
    assert stats.encoded == 4 * L * 2 * H
