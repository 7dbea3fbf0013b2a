"""Token writer: the staged records must hold exactly the written tokens.

The writer has a coalesced path for groups of sixteen tokens that are complete
and contiguous in the input and a scattered path for everything else; both
must produce the reference's staging layout (``hbm_kv.cu:221-255``: raw
records in kernel order).  Each case writes tokens through ``HbmKvStore.write``
and compares every written scalar of every staged record with the oracle's
kernel order of the same tokens; scalars that were not written must keep the
0xA5 fill the test puts there first.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

import oracle
from fragpack_b200.compression import attn_page as ap
from fragpack_b200.compression.attn_tables import device_tables
from fragpack_b200.ops.hbm_kv import HbmKvStore, page_bytes
from tests._util import bf16_tensor, to_bits

pytestmark = pytest.mark.gpu

L, H, D, T, NB = 2, 5, ap.HEAD_DIM, ap.PAGE_TOKENS, 10
FILL = 0xA5A5


def _layouts():
    """name -> steps; a step is a list of rows (block list, first position, token count)."""
    return {
        # Whole blocks, aligned in the input: every token on the coalesced path.
        "aligned_prefill": [[([1, 2, 3], 0, 3 * T)]],
        # A sequence that starts 5 tokens into the input and ends mid-group.
        "shifted": [[([4], 0, 5), ([5, 6], 0, T + 37)]],
        # A second chunk that continues an open block from offset 21.
        "continuing": [[([7, 8], 0, 21)], [([7, 8], 21, 200)]],
        # Single decode tokens appended to open blocks of several sequences.
        "decode": [[([1], 0, 17), ([2], 0, 126), ([3], 0, 64)], [([1], 17, 1), ([2], 126, 1), ([3], 64, 1)]],
    }


def _run(steps, *, pad: int = 0, shuffle: bool = False, misalign: bool = False) -> None:
    rng = np.random.default_rng(11)
    device = torch.device("cuda", torch.cuda.current_device())
    table = np.broadcast_to(np.arange(22, dtype=np.uint8), (L, 2, H, 22)).copy()
    arenas = [torch.empty(NB, page_bytes(H), dtype=torch.uint8, device=device) for _ in range(L)]
    store = HbmKvStore(arenas, H, device_tables(table, device), max_tokens=1024,
                       staging_slots=NB, overflow_records=4)
    fill16 = int(np.uint16(FILL).view(np.int16))
    # Blocks that stay open keep a persistent staging slot; blocks that fill up
    # within one step use the transient pool, which holds one layer at a time.
    store.staging.view(torch.int16).fill_(fill16)
    pools = [(t.data_ptr(), t.numel(), t.view(-1)) for t in (store.staging, store.scratch)]
    pos = np.arange(ap.RAW_RECORD_BYTES // 2)
    word, within = pos // 8, pos % 8
    # Raw record: owner t's word st at 16 (256 st + t) holds kernel positions 64 t + 8 st + (0..7).
    kernel_pos = 64 * (word % 256) + 8 * (word // 256) + within
    want = np.full((L, 2, NB, T, H, D), FILL, np.uint16)
    for rows in steps:
        slots = [blocks[p // T] * T + p % T for blocks, start, n in rows for p in range(start, start + n)]
        if shuffle:
            # Same tokens, input order broken inside one group: that group is not contiguous.
            slots[16:32] = slots[16:32][::-1]
        slots = slots + [-1] * pad
        n = len(slots)
        slot_t = torch.tensor(slots, dtype=torch.int64, device=device)
        live = sorted({s // T for s in slots if s >= 0})
        store.prepare(slot_t, n, np.array(live, np.int32))
        addr = store.rec_addr.cpu().numpy()
        for layer in range(L):
            kv = to_bits(rng.standard_normal((2, n, H, D)))
            for i, s in enumerate(slots):
                if s >= 0:
                    want[layer, :, s // T, s % T] = kv[:, i]
            if misalign:
                # Rows that start 4 bytes off a 16-byte boundary: only the scattered path applies.
                buf = torch.empty(2, n * H * D + 2, dtype=torch.bfloat16, device=device)
                key = buf[0, 2:].view(n, H, D)
                value = buf[1, 2:].view(n, H, D)
                key.copy_(bf16_tensor(kv[0]))
                value.copy_(bf16_tensor(kv[1]))
            else:
                key, value = bf16_tensor(kv[0]), bf16_tensor(kv[1])
            store.scratch.view(torch.int16).fill_(fill16)
            store.write(layer, key, value, slot_t)
            torch.cuda.synchronize()
            for b in live:
                for kv_i in range(2):
                    order = oracle.kernel_order(kv_i)  # kernel position -> token-major index
                    for h in range(H):
                        a = int(addr[layer, b, kv_i, h])
                        hit = [(flat, a - base) for base, size, flat in pools if base <= a < base + size]
                        assert hit, "a written block's record must sit in a staging pool"
                        flat, at = hit[0]
                        got = flat[at : at + ap.RAW_RECORD_BYTES].cpu().numpy().view(np.uint16)
                        expect = want[layer, kv_i, b, :, h].reshape(-1)[order[kernel_pos]]
                        assert np.array_equal(got, expect), (layer, b, kv_i, h)
        store.commit()


@pytest.mark.parametrize("name", list(_layouts()))
def test_writer_layouts(name: str) -> None:
    _run(_layouts()[name])


def test_writer_padding_and_broken_contiguity() -> None:
    _run(_layouts()["aligned_prefill"], pad=7, shuffle=True)


def test_writer_unaligned_rows_take_the_scattered_path() -> None:
    _run(_layouts()["shifted"], misalign=True)
