"""The stand-in for the reference's ``fragpack/ops/fragpack_ext.py``, driven as the reference drives it.

``fragpack_b200.integrations.reference_ext.extension()`` offers the eight
functions of the reference's pybind11 module with the same positional
``torch.Tensor`` arguments (``fragpack/ops/fragpack_ext.cpp:5-66``).  This test
makes the calls the reference's ``HbmKvStore`` and ``decode_attention`` make
(``hbm_kv.py:372-557``, ``fused_attn_decode.py:174-219``) - thirteen state
tensors first, then the call's own arguments - and checks the results against
the oracle: record bytes, decompressed bits, attention, a blob round trip.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

import oracle
from fragpack_b200.compression import attn_page as ap
from fragpack_b200.compression.attn_tables import device_tables
from fragpack_b200.integrations.reference_ext import extension, plan_words
from fragpack_b200.ops.hbm_kv import HbmKvStore, page_bytes
from tests._util import assert_attention_close, bf16_tensor, to_bits

pytestmark = pytest.mark.gpu
L, H, NB, T, D = 2, 4, 8, 128, 128
SCALE = D**-0.5


def test_reference_call_sequence_through_the_stand_in() -> None:
    ext = extension()
    rng = np.random.default_rng(3)
    dev = torch.device("cuda")
    cal = to_bits(rng.standard_normal((L, 2, H, 4 * T, D)) * 0.5)
    table = np.empty((L, 2, H, ap.TABLE_ENTRIES), np.uint8)
    for idx in np.ndindex(L, 2, H):
        table[idx] = oracle.calibrate_table((cal[idx] >> 8).astype(np.uint8))
    tables = device_tables(table, dev)
    caches = [torch.zeros((NB, page_bytes(H)), dtype=torch.uint8, device=dev) for _ in range(L)]
    # The tensors the reference's HbmKvStore allocates (same shapes and initial
    # values); only the stand-in's functions are called below.
    st = HbmKvStore(caches, H, tables, max_tokens=512, staging_slots=2, overflow_records=8)
    state = (st.counters, st.wslot, st.tags, st.free_stack, st.ovf_bits, st.claim_list, st.close_list,
             st.rec_addr, st.rec_len, st.staging, st.scratch, st.overflow, st.fill)

    # One prefill step: blocks 1 and 2 close, block 3 stays open with 40 tokens.
    blocks, tokens = [1, 2, 3], 2 * T + 40
    slots = torch.tensor([blocks[p // T] * T + p % T for p in range(tokens)], dtype=torch.int64, device=dev)
    live = torch.tensor(blocks, dtype=torch.int32, device=dev)
    ext.hbm_prepare(*state, slots, tokens, live, len(blocks), 1)
    kv = to_bits(rng.standard_normal((L, 2, tokens, H, D)) * 0.5)
    for layer in range(L):
        ext.hbm_write(*state, bf16_tensor(kv[layer, 0]), bf16_tensor(kv[layer, 1]), slots, layer)
        ext.hbm_encode(*state, tables.rank_of, layer, caches[layer].data_ptr(),
                       caches[layer].stride(0), 2)
    ext.hbm_commit(*state)
    torch.cuda.synchronize()

    # Closed blocks: record bytes equal the oracle encoder's.
    addr, length = st.rec_addr.cpu().numpy(), st.rec_len.cpu().numpy()
    for layer in range(L):
        arena = caches[layer].cpu().numpy().reshape(-1)
        for i, b in enumerate(blocks[:2]):
            for k in range(2):
                for h in range(H):
                    want = oracle.encode_record(kv[layer, k, i * T : (i + 1) * T, h], table[layer, k, h], k)
                    off = int(addr[layer, b, k, h]) - caches[layer].data_ptr()
                    assert ap.DENSE_BYTES + int(length[layer, b, k, h]) == len(want)
                    assert arena[off : off + len(want)].tobytes() == want

    # Decompressor: written bits come back (the open block up to its 40 tokens).
    src = torch.tensor(blocks, dtype=torch.int32, device=dev)
    wk = torch.empty(3, T, H, D, dtype=torch.bfloat16, device=dev)
    wv = torch.empty_like(wk)
    for layer in range(L):
        ext.hbm_gather(src, st.rec_addr[layer], st.rec_len[layer], tables.plut[layer], tables.slut[layer],
                       wk, wv, H)
        got_k = wk.view(torch.int16).cpu().numpy().view(np.uint16).reshape(-1, H, D)[:tokens]
        got_v = wv.view(torch.int16).cpu().numpy().view(np.uint16).reshape(-1, H, D)[:tokens]
        assert np.array_equal(got_k, kv[layer, 0]) and np.array_equal(got_v, kv[layer, 1])

    # Decode attention, as fused_attn_decode._launch calls it (group 8).
    units = 1 + 16
    opart = torch.empty(H * units * 8 * 128, device=dev)
    ml = torch.empty(H * units * 8 * 2, device=dev)
    plan = torch.empty(plan_words(units), dtype=torch.int32, device=dev)
    block_table = torch.tensor([blocks], dtype=torch.int32, device=dev)
    seq_lens = torch.tensor([tokens], dtype=torch.int32, device=dev)
    for layer in range(L):
        q = torch.randn(1, H * 8, D, device=dev).to(torch.bfloat16)
        out = torch.full_like(q, float("nan"))
        ext.fused_decode(q, st.rec_addr[layer], st.rec_len[layer], tables.plut[layer], tables.slut[layer],
                         block_table, seq_lens, opart, ml, plan, out, units, layer == 0, SCALE)
        kvf = bf16_tensor(kv[layer]).float().cpu()
        for h in range(H):
            ref = oracle.attention_fp32(q[0, 8 * h : 8 * h + 8].float().cpu(), kvf[0, :, h], kvf[1, :, h], SCALE)
            assert_attention_close(out[0, 8 * h : 8 * h + 8], ref, (layer, h))

    # Blob round trip: export the closed blocks, import them as blocks 5 and 6.
    stride = st.blob_stride
    blob = torch.zeros(2 * stride, dtype=torch.uint8, device=dev)
    ids = torch.tensor(blocks[:2], dtype=torch.int32, device=dev)
    lengths = torch.empty(2, dtype=torch.int64, device=dev)
    ext.hbm_export(ids, st.rec_addr, st.rec_len, blob, stride, lengths, st.table_digest)
    status = torch.zeros(2, dtype=torch.int32, device=dev)
    ext.hbm_import(*state, blob, torch.tensor([0, stride], dtype=torch.int64, device=dev),
                   torch.tensor([5, 6], dtype=torch.int32, device=dev), status, st.arena_base_dev,
                   st.arena_stride_dev, st.table_digest)
    torch.cuda.synchronize()
    assert status.cpu().tolist() == [0, 0]
    assert (lengths.cpu() % ap.BLOB_ALIGN == 0).all()
    src = torch.tensor([5, 6], dtype=torch.int32, device=dev)
    ext.hbm_gather(src, st.rec_addr[0], st.rec_len[0], tables.plut[0], tables.slut[0], wk, wv, H)
    got_k = wk.view(torch.int16).cpu().numpy().view(np.uint16).reshape(-1, H, D)[: 2 * T]
    assert np.array_equal(got_k, kv[0, 0, : 2 * T])
    with pytest.raises(RuntimeError):
        ext.fused_decode(q, st.rec_addr[0], st.rec_len[0], tables.plut[0], tables.slut[0], block_table,
                         seq_lens, opart, ml, plan[:8], out, units, True, SCALE)
