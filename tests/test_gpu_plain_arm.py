"""The plain-BF16 comparison kernel: same attention, records never coded.

A store whose tables match no value of the data sends every closed block to
the overflow pool as a raw record; the plain kernel must then agree with fp32
attention over the source KV and, bit for bit, with the fused kernel (which
reads raw records through its in-place path and does the same arithmetic).
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from fragpack_b200.compression import attn_page as ap
from fragpack_b200.compression.attn_tables import calibrate, device_tables
from fragpack_b200.ops.fused_attn_decode import (
    DECODE_NOT_PLAIN,
    GQA,
    RecordTables,
    decode_attention,
    decode_status,
    decode_units,
    plain_decode_attention,
    workspace_elems,
)
from fragpack_b200.ops.hbm_kv import HbmKvStore, page_bytes

pytestmark = pytest.mark.gpu

HEADS, BLOCKS, TOKENS, DIM = 2, 12, ap.PAGE_TOKENS, ap.HEAD_DIM
SCALE = DIM**-0.5


def _store(table: np.ndarray, source: torch.Tensor, tokens: int):
    device = source.device
    arena = [torch.empty(BLOCKS, page_bytes(HEADS), dtype=torch.uint8, device=device)]
    store = HbmKvStore(arena, HEADS, device_tables(table, device), max_tokens=BLOCKS * TOKENS,
                       staging_slots=2, overflow_records=BLOCKS * 2 * HEADS)
    slots = torch.arange(tokens, dtype=torch.int64, device=device)
    open_blocks = np.array([tokens // TOKENS], np.int32) if tokens % TOKENS else np.zeros(0, np.int32)
    store.prepare(slots, tokens, open_blocks)
    store.write(0, source[0, :tokens], source[1, :tokens], slots)
    store.encode(0, tokens // TOKENS)
    store.commit()
    return store, arena


def _reference(q, source, lengths):
    out = torch.zeros_like(q, dtype=torch.float32)
    for b, n in enumerate(lengths):
        for h in range(HEADS):
            k, v = source[0, :n, h].float(), source[1, :n, h].float()
            qh = q[b, h * GQA : (h + 1) * GQA].float()
            out[b, h * GQA : (h + 1) * GQA] = torch.softmax(qh @ k.T * SCALE, -1) @ v
    return out


@pytest.mark.parametrize("tokens", [BLOCKS * TOKENS, BLOCKS * TOKENS - 77])
def test_plain_kernel_matches_reference_and_fused_kernel(tokens: int) -> None:
    device = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator().manual_seed(5)
    source = torch.randn(2, BLOCKS * TOKENS, HEADS, DIM, generator=gen).to(torch.bfloat16).to(device)
    never = np.broadcast_to(np.arange(0x60, 0x60 + 22, dtype=np.uint8), (1, 2, HEADS, 22)).copy()
    store, _arena = _store(never, source, tokens)
    stats = store.stats()
    assert stats.fallbacks == stats.encoded == (tokens // TOKENS) * 2 * HEADS
    tabs = RecordTables(*store.layer_tables(0))
    assert int((tabs.rec_len[: (tokens + TOKENS - 1) // TOKENS] <= ap.VAR_CAP).sum()) == 0

    lengths = np.array([tokens, tokens - 130, 1, 0, 5 * TOKENS], np.int32)
    batch = len(lengths)
    table = torch.arange(BLOCKS, dtype=torch.int32, device=device).repeat(batch, 1)
    lens = torch.from_numpy(lengths).to(device)
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    units = decode_units(batch, HEADS, sms)
    sizes = workspace_elems(HEADS, units)
    q = torch.randn(batch, HEADS * GQA, DIM, generator=torch.Generator().manual_seed(6)).to(torch.bfloat16).to(device)
    outs = []
    for fn in (plain_decode_attention, decode_attention):
        ws = (torch.empty(sizes[0], device=device), torch.empty(sizes[1], device=device),
              torch.empty(sizes[2], dtype=torch.int32, device=device))
        out = torch.full_like(q, float("nan"))
        fn(q, tabs, table, lens, SCALE, units, out, ws, replan=True)
        assert decode_status(ws, units) == 0
        outs.append(out)
    ref = _reference(q, source, lengths)
    # Tolerance of the decode parity bar: 1e-2 max-abs, 2e-3 mean-abs.
    err = (outs[0].float() - ref).abs()
    assert float(err.max()) <= 1e-2 and float(err.mean()) <= 2e-3
    assert torch.count_nonzero(outs[0][3]).item() == 0
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))


def test_plain_kernel_flags_coded_records() -> None:
    device = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator().manual_seed(8)
    source = torch.randn(2, BLOCKS * TOKENS, HEADS, DIM, generator=gen).to(torch.bfloat16).to(device)
    bits = source.view(torch.int16).cpu().numpy().view(np.uint16)
    table = calibrate(bits.reshape(2, BLOCKS, TOKENS, HEADS, DIM).transpose(1, 0, 2, 3, 4)[:, None])
    store, _arena = _store(table, source, BLOCKS * TOKENS)
    tabs = RecordTables(*store.layer_tables(0))
    lens = torch.tensor([BLOCKS * TOKENS], dtype=torch.int32, device=device)
    block_table = torch.arange(BLOCKS, dtype=torch.int32, device=device)[None]
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    units = decode_units(1, HEADS, sms)
    sizes = workspace_elems(HEADS, units)
    ws = (torch.empty(sizes[0], device=device), torch.empty(sizes[1], device=device),
          torch.empty(sizes[2], dtype=torch.int32, device=device))
    q = torch.randn(1, HEADS * GQA, DIM, generator=gen).to(torch.bfloat16).to(device)
    out = torch.empty_like(q)
    plain_decode_attention(q, tabs, block_table, lens, SCALE, units, out, ws, replan=True)
    assert decode_status(ws, units) & DECODE_NOT_PLAIN
    assert torch.isfinite(out.float()).all()
