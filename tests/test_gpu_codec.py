"""Block encoder / decompressor kernels vs the oracle, through the C ABI.

Bit-exact bar: the compressed stream and the reconstructed KV must equal the
oracle's (itself pinned to the reference codec by the golden vectors).
"""

from __future__ import annotations

from pathlib import Path

import numpy as np
import pytest

import oracle
from benchmarks import synth
from fragpack_b200.compression import attn_page as ap
from tests._util import gpu_decode, gpu_encode

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def _same_records(out, lens, want_out, want_lens) -> None:
    assert np.array_equal(lens, want_lens)
    for i in range(len(lens)):
        assert np.array_equal(out[i, : lens[i]], want_out[i, : lens[i]]), i


def test_golden_records_encode_and_decode_bit_exact() -> None:
    g = np.load(GOLDEN / "codec_golden.npz")
    out, lens = gpu_encode(g["records"], g["tables"], g["kv"])
    _same_records(out, lens, g["encoded"], g["lens"])
    # Bytes past the record are left untouched.
    for i in range(len(lens)):
        assert (out[i, lens[i] :] == 0xA5).all()
    assert np.array_equal(gpu_decode(g["encoded"], g["lens"], g["tables"], g["kv"]), g["records"])


@pytest.mark.parametrize(
    "heavy, junk",
    [(0.0, 0.0), (0.005, 0.0), (0.0, 0.009), (0.0, 0.0125), (0.0, 0.02), (0.05, 0.004)],
)
def test_seeded_records_match_oracle(heavy: float, junk: float) -> None:
    rng = np.random.default_rng(int(1000 * heavy + 100000 * junk) + 5)
    scales = synth.channel_scales(11, 1, 4)[0]
    cal = synth.kv_tokens_numpy(rng, scales, 512, heavy, junk)
    kvt = synth.kv_tokens_numpy(rng, scales, 6 * 128, heavy, junk)
    records, tables, kvs = [], [], []
    for k in range(2):
        for h in range(4):
            table = ap.calibrate_table((cal[k, :, h] >> 8).astype(np.uint8))
            for b in range(6):
                records.append(kvt[k, b * 128 : (b + 1) * 128, h])
                tables.append(table)
                kvs.append(k)
    records, tables, kvs = np.stack(records), np.stack(tables), np.array(kvs, np.int32)
    want_out, want_lens = oracle.encode_records(records, tables, kvs)
    out, lens = gpu_encode(records, tables, kvs)
    _same_records(out, lens, want_out, want_lens)
    assert np.array_equal(gpu_decode(want_out, want_lens, tables, kvs), records)


def test_dense_escape_runs_and_raw_limits() -> None:
    """Escape runs longer than 16 per owner, and the 32-raw-per-warp boundary."""
    rng = np.random.default_rng(3)
    base = synth.bf16_rne(rng.standard_normal((128, 128)).astype(np.float32))
    table = ap.calibrate_table((base >> 8).astype(np.uint8))
    absent = [b for b in range(256) if b not in set(table.tolist())]
    rare = int(table[21])
    records, kvs = [], []
    for kv in (0, 1):
        order = oracle.kernel_order(kv)
        # (a) one owner's 64 scalars all extended-table escapes.
        rec = base.copy().reshape(-1)
        rec[order[64 * 37 : 64 * 38]] = (rare << 8) | 0x11
        records.append(rec.reshape(128, 128)); kvs.append(kv)
        # (b) exactly 32 raw scalars in warp 3 (codes), (c) 33 (falls back raw).
        for count in (32, 33):
            rec = base.copy().reshape(-1)
            pos = order[2048 * 3 + 61 * np.arange(count)]
            rec[pos] = (absent[0] << 8) | 0x22
            records.append(rec.reshape(128, 128)); kvs.append(kv)
        # (d) raw scalars at the first and last position of the record.
        rec = base.copy().reshape(-1)
        rec[order[0]] = (absent[1] << 8) | 1
        rec[order[-1]] = (absent[2] << 8) | 2
        records.append(rec.reshape(128, 128)); kvs.append(kv)
    records, kvs = np.stack(records), np.array(kvs, np.int32)
    tables = np.tile(table, (len(kvs), 1))
    want_out, want_lens = oracle.encode_records(records, tables, kvs)
    assert want_lens[2] == ap.RAW_RECORD_BYTES and want_lens[1] < ap.RAW_RECORD_BYTES
    out, lens = gpu_encode(records, tables, kvs)
    _same_records(out, lens, want_out, want_lens)
    assert np.array_equal(gpu_decode(want_out, want_lens, tables, kvs), records)


def test_compression_api_single_record() -> None:
    """fragpack.compression-style calls (attn_page.encode_record / decode_record)."""
    g = np.load(GOLDEN / "codec_golden.npz")
    for i in (0, 5, 6):
        rec = ap.encode_record(g["records"][i], g["tables"][i], int(g["kv"][i]))
        assert rec == g["encoded"][i, : g["lens"][i]].tobytes()
        assert np.array_equal(ap.decode_record(rec, g["tables"][i], int(g["kv"][i])), g["records"][i])
    with pytest.raises(ValueError):
        ap.decode_record(b"\x00" * 100, g["tables"][0], 0)
