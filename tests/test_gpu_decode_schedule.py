"""Decode scheduling contracts for ragged and CUDA-graph-padded batches.

Follows the reference's ``tests/gpu/test_fragpack_decode_schedule.py``: three
physical pages are repeated through 1024-entry block tables to reach long
contexts without a large KV allocation (a correctness device only - repeated
pages would fake bandwidth, so no timing is taken here).  The fp32 reference
folds identical token copies into multiplicities; it never looks at the planner
or the split-KV workspace.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from fragpack_b200.compression import attn_page as ap
from fragpack_b200.compression.attn_tables import calibrate, device_tables
from fragpack_b200.ops.fused_attn_decode import (
    GQA,
    RecordTables,
    decode_attention,
    decode_status,
    decode_units,
    workspace_elems,
)
from fragpack_b200.ops.hbm_kv import HbmKvStore, page_bytes

pytestmark = pytest.mark.gpu

LAYERS, HEADS, BLOCKS = 2, 4, 3
TOKENS, DIM = ap.PAGE_TOKENS, ap.HEAD_DIM
MAX_PAGES = 1024
SCALE = DIM**-0.5


@pytest.fixture(scope="module")
def encoded_store():
    """Two layers of encoded KV; returns (store, arena owners, BF16 source KV)."""
    generator = torch.Generator().manual_seed(231)
    source = torch.randn(LAYERS, 2, BLOCKS, TOKENS, HEADS, DIM, generator=generator).mul_(0.5)
    # Distinct page means make omitted or misassigned pages visible even when
    # attention is nearly uniform over many repeated tokens.
    source[:, 1] += torch.arange(BLOCKS)[None, :, None, None, None] - 1
    source = source.to(torch.bfloat16)
    bits = source.view(torch.int16).numpy().view(np.uint16)
    table = calibrate(bits.transpose(2, 0, 1, 3, 4, 5))
    device = torch.device("cuda", torch.cuda.current_device())
    arenas = [
        torch.empty(BLOCKS, page_bytes(HEADS), dtype=torch.uint8, device=device)
        for _ in range(LAYERS)
    ]
    store = HbmKvStore(
        arenas,
        HEADS,
        device_tables(table, device),
        max_tokens=BLOCKS * TOKENS,
        staging_slots=1,
        overflow_records=LAYERS * BLOCKS * 2 * HEADS,
    )
    source = source.to(device)
    slots = torch.arange(BLOCKS * TOKENS, dtype=torch.int64, device=device)
    store.prepare(slots, slots.numel(), np.arange(BLOCKS, dtype=np.int32))
    for layer in range(LAYERS):
        key, value = source[layer].reshape(2, BLOCKS * TOKENS, HEADS, DIM)
        store.write(layer, key, value, slots)
        store.encode(layer, BLOCKS)
    store.commit()
    stats = store.stats()
    assert stats.err_staging == 0 and stats.err_overflow == 0
    assert stats.encoded > stats.fallbacks
    return store, arenas, source


def _block_table(batch: int) -> np.ndarray:
    return ((np.arange(batch)[:, None] + np.arange(MAX_PAGES)[None, :]) % BLOCKS).astype(np.int32)


def _ragged_lengths(batch: int) -> np.ndarray:
    lengths = np.resize(
        np.array([1, TOKENS - 1, TOKENS, TOKENS + 1, 8 * TOKENS + 13], np.int32), batch
    )
    lengths[1::7] = 0
    lengths[0] = 63 * TOKENS + 1
    lengths[-1] = MAX_PAGES * TOKENS - 1
    return lengths


def _workspace(units: int, device):
    opart, ml, plan = workspace_elems(HEADS, units)
    return (
        torch.empty(opart, dtype=torch.float32, device=device),
        torch.empty(ml, dtype=torch.float32, device=device),
        torch.empty(plan, dtype=torch.int32, device=device),
    )


def _reference(q, source, block_table, lengths):
    """fp32 attention with repeated pages folded into log-multiplicities."""
    counts = np.zeros((len(lengths), BLOCKS, TOKENS), dtype=np.float32)
    for row, length in enumerate(lengths):
        full_pages, tail = divmod(int(length), TOKENS)
        counts[row] = np.bincount(block_table[row, :full_pages], minlength=BLOCKS)[:, None]
        if tail:
            counts[row, block_table[row, full_pages], :tail] += 1
    multiplicity = torch.from_numpy(counts.reshape(len(lengths), -1)).to(q.device)
    key, value = source.permute(0, 3, 1, 2, 4).reshape(2, HEADS, BLOCKS * TOKENS, DIM).float()
    group = q.shape[1] // HEADS
    query = q.reshape(len(lengths), HEADS, group, DIM).float()
    logits = torch.einsum("bhgd,htd->bhgt", query, key) * SCALE
    logits += multiplicity.log()[:, None, None, :]
    padding = torch.from_numpy(lengths == 0).to(q.device)
    logits[padding] = 0
    reference = torch.einsum("bhgt,htd->bhgd", logits.softmax(-1), value)
    reference[padding] = 0
    return reference.reshape_as(q)


def _decode_layers(store, queries, outputs, block_table, lengths, units, workspace) -> None:
    for layer in range(LAYERS):
        decode_attention(
            queries[layer],
            RecordTables(*store.layer_tables(layer)),
            block_table,
            lengths,
            SCALE,
            units,
            outputs[layer],
            workspace,
            replan=layer == 0,
        )


def _check_outputs(queries, outputs, source, block_table, lengths) -> None:
    padding = torch.from_numpy(lengths == 0).to(source.device)
    for layer in range(LAYERS):
        reference = _reference(queries[layer], source[layer], block_table, lengths)
        torch.testing.assert_close(outputs[layer].float(), reference, atol=2e-3, rtol=1e-2)
        # Zero-length rows must be explicitly overwritten with zeros.
        assert torch.count_nonzero(outputs[layer][padding]).item() == 0


@pytest.mark.parametrize("batch_case", ["below_wave", "at_wave", "above_wave", "tiled"])
def test_ragged_batches_match_fp32_attention(encoded_store, batch_case: str) -> None:
    store, _arenas, source = encoded_store
    sms = torch.cuda.get_device_properties(source.device).multi_processor_count
    wave = max(1, 2 * sms // HEADS)
    batch = {
        "below_wave": max(1, wave - 1),
        "at_wave": wave,
        "above_wave": wave + 1,
        "tiled": max(269, wave + 1),
    }[batch_case]
    table = _block_table(batch)
    lengths = _ragged_lengths(batch)
    units = decode_units(batch, HEADS, sms)
    generator = torch.Generator(device=source.device).manual_seed(325 + batch)
    queries = [
        torch.randn(batch, HEADS * GQA, DIM, dtype=torch.bfloat16, device=source.device,
                    generator=generator)
        for _ in range(LAYERS)
    ]
    outputs = [torch.full_like(q, float("nan")) for q in queries]
    workspace = _workspace(units, source.device)
    _decode_layers(
        store, queries, outputs, torch.from_numpy(table).to(source.device),
        torch.from_numpy(lengths).to(source.device), units, workspace,
    )
    _check_outputs(queries, outputs, source, table, lengths)
    assert decode_status(workspace, units) == 0


@pytest.mark.parametrize("units_policy", ["auto", "minimum"])
@pytest.mark.parametrize("group", [1, 2, 4, GQA])
def test_graph_replans_padding_and_reuses_plan_across_layers(
    encoded_store, units_policy: str, group: int
) -> None:
    """Replay every query group with changing lengths and empty rows."""
    store, _arenas, source = encoded_store
    batch = 269
    table = _block_table(batch)
    initial = _ragged_lengths(batch)
    changed = np.roll(initial, 17)
    changed[0] = changed[256] = 0
    changed[257] = MAX_PAGES * TOKENS - 11
    empty = np.zeros(batch, dtype=np.int32)
    sparse = empty.copy()
    sparse[[0, 256, batch - 1]] = [1, TOKENS + 1, MAX_PAGES * TOKENS - 17]
    device_table = torch.from_numpy(table).to(source.device)
    device_lengths = torch.from_numpy(initial).to(source.device)
    sms = torch.cuda.get_device_properties(source.device).multi_processor_count
    units = decode_units(batch, HEADS, sms) if units_policy == "auto" else batch
    workspace = _workspace(units, source.device)
    generator = torch.Generator(device=source.device).manual_seed(401)
    queries = [
        torch.randn(batch, HEADS * group, DIM, dtype=torch.bfloat16, device=source.device,
                    generator=generator)
        for _ in range(LAYERS)
    ]
    outputs = [torch.full_like(q, float("nan")) for q in queries]
    args = store, queries, outputs, device_table, device_lengths, units, workspace
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(3):
            _decode_layers(*args)
    torch.cuda.current_stream().wait_stream(stream)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        _decode_layers(*args)
    for lengths in (initial, changed, empty, sparse):
        device_lengths.copy_(torch.from_numpy(lengths))
        for output in outputs:
            output.fill_(float("nan"))
        graph.replay()
        _check_outputs(queries, outputs, source, table, lengths)
    assert decode_status(workspace, units) == 0


@pytest.mark.parametrize("units_policy", ["auto", "minimum"])
def test_repeated_launches_are_bitwise_identical(encoded_store, units_policy: str) -> None:
    """The same launch twenty times: any difference would be a race between warps."""
    store, _arenas, source = encoded_store
    batch = 269
    sms = torch.cuda.get_device_properties(source.device).multi_processor_count
    units = decode_units(batch, HEADS, sms) if units_policy == "auto" else batch
    workspace = _workspace(units, source.device)
    table = torch.from_numpy(_block_table(batch)).to(source.device)
    lengths = torch.from_numpy(_ragged_lengths(batch)).to(source.device)
    generator = torch.Generator(device=source.device).manual_seed(77)
    q = torch.randn(batch, HEADS * GQA, DIM, dtype=torch.bfloat16, device=source.device,
                    generator=generator)
    tabs = RecordTables(*store.layer_tables(0))
    first = None
    for _ in range(20):
        out = torch.full_like(q, float("nan"))
        decode_attention(q, tabs, table, lengths, SCALE, units, out, workspace, replan=True)
        if first is None:
            first = out
        else:
            assert torch.equal(out.view(torch.int16), first.view(torch.int16))


def _equal_lengths(batch: int, pages: int) -> np.ndarray:
    lengths = np.full(batch, pages * TOKENS, np.int32)
    lengths[3::5] = 0  # padding rows
    return lengths


@pytest.mark.parametrize(
    "lengths_case",
    ["ragged-17", "ragged-130", "ragged-700", "equal-6x256", "equal-40x37", "equal-200x3", "equal-600x5",
     "one-long", "all-empty"],
)
def test_plan_cuts_every_sequence_once_and_lists_units_longest_first(encoded_store, lengths_case: str) -> None:
    """The planner's words, read back: a partition of every sequence, and the item descriptors.

    Every sequence's pages are covered once by consecutive units in page order;
    no unit is empty; padding rows have no unit; unused units are marked; and
    the item descriptors both schedules walk are a permutation of the units in
    use with non-increasing lengths, each repeating its unit's entry and its
    sequence's length.
    """
    store, _, _ = encoded_store
    device = store.rec_addr.device
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    if lengths_case.startswith("ragged"):
        lengths = _ragged_lengths(int(lengths_case.split("-")[1]))
    elif lengths_case.startswith("equal"):
        batch, pages = map(int, lengths_case.split("-")[1].split("x"))
        lengths = _equal_lengths(batch, pages)
    elif lengths_case == "one-long":
        lengths = np.array([MAX_PAGES * TOKENS], np.int32)
    else:
        lengths = np.zeros(9, np.int32)
    batch = len(lengths)
    units = decode_units(batch, HEADS, sms)
    workspace = _workspace(units, device)
    q = torch.zeros(batch, HEADS * GQA, DIM, dtype=torch.bfloat16, device=device)
    out = torch.empty_like(q)
    decode_attention(q, RecordTables(*store.layer_tables(0)), torch.from_numpy(_block_table(batch)).to(device),
                     torch.from_numpy(lengths).to(device), SCALE, units, out, workspace, replan=True)
    torch.cuda.synchronize()
    assert decode_status(workspace, units) == 0
    plan = workspace[2].cpu().numpy()
    pages_of = (lengths.astype(np.int64) + TOKENS - 1) // TOKENS
    used = int(plan[1])
    assert 0 <= used <= units - batch + int((pages_of > 0).sum()) or used == 0
    unit_seq = plan[2 : 2 + 2 * units : 2]
    unit_where = plan[3 : 3 + 2 * units : 2]
    assert (unit_seq[used:] == -1).all()
    seq_plan = plan[2 + 2 * units : 2 + 2 * units + 2 * batch].reshape(batch, 2)
    longest = 0
    for b in range(batch):
        first, chunks = map(int, seq_plan[b])
        assert (chunks == 0) == (pages_of[b] == 0)
        page = 0
        for u in range(first, first + chunks):
            assert unit_seq[u] == b
            assert (int(unit_where[u]) & 0xFFFF) == page
            count = int(unit_where[u]) >> 16
            assert count > 0
            longest = max(longest, count)
            page += count
        assert page == pages_of[b]
    assert int(seq_plan[:, 1].sum()) == used
    assert int(plan[0]) == longest
    # The item descriptors, in the order the schedules hand the units out.
    first_desc = 2 + 4 * units + 2 + 4 + 256
    desc = plan[first_desc : first_desc + 4 * units].reshape(units, 4)
    assert sorted(desc[:used, 3].tolist()) == list(range(used))
    assert (desc[used:, 0] == -1).all()
    assert (np.diff(desc[:used, 1] >> 16) <= 0).all()
    for place in range(used):
        seq, where, length, unit = map(int, desc[place])
        assert seq == unit_seq[unit] and where == unit_where[unit] and length == lengths[seq]
