"""The numpy codec of ``fragpack_b200.compression`` against the golden vectors and the oracle.

Without a CUDA device ``attn_page.encode_record`` / ``decode_record`` run
:mod:`fragpack_b200.compression.host_codec`; its bytes must be the reference
codec's (the golden file was written by importing the reference).
"""

from __future__ import annotations

from pathlib import Path

import numpy as np
import pytest

import oracle
from benchmarks import synth
from fragpack_b200.compression import attn_page as ap
from fragpack_b200.compression import host_codec

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_golden_records_byte_for_byte() -> None:
    g = np.load(GOLDEN / "codec_golden.npz")
    for i in range(len(g["lens"])):
        table, kv = g["tables"][i], int(g["kv"][i])
        want = g["encoded"][i, : g["lens"][i]].tobytes()
        assert host_codec.encode(g["records"][i], ap.rank_table(table), kv) == want, g["names"][i]
        assert np.array_equal(host_codec.decode(want, table, kv), g["records"][i]), g["names"][i]


@pytest.mark.parametrize("heavy, junk", [(0.0, 0.0), (0.005, 0.0), (0.0, 0.009), (0.0, 0.0125), (0.0, 0.02)])
def test_seeded_records_match_the_oracle(heavy: float, junk: float) -> None:
    rng = np.random.default_rng(int(1e5 * junk + 1e3 * heavy) + 1)
    scales = synth.channel_scales(17, 1, 2)[0]
    kvt = synth.kv_tokens_numpy(rng, scales, 3 * 128, heavy, junk)
    for kv in range(2):
        for h in range(2):
            table = ap.calibrate_table((kvt[kv, :, h] >> 8).astype(np.uint8))
            for b in range(3):
                rec = kvt[kv, b * 128 : (b + 1) * 128, h]
                want = oracle.encode_record(rec, table, kv)
                assert host_codec.encode(rec, ap.rank_table(table), kv) == want
                assert np.array_equal(host_codec.decode(want, table, kv), rec)


def test_public_functions_work_without_a_gpu() -> None:
    import torch

    if torch.cuda.is_available():
        pytest.skip("with a CUDA device the public functions call the kernels")
    rng = np.random.default_rng(0)
    rec = synth.bf16_rne(rng.standard_normal((128, 128)).astype(np.float32))
    table = ap.calibrate_table((rec >> 8).astype(np.uint8))
    out = ap.encode_record(rec, table, 1)
    assert len(out) < 0.75 * ap.RAW_RECORD_BYTES
    assert np.array_equal(ap.decode_record(out, table, 1), rec)
    with pytest.raises(ValueError):
        ap.encode_record(rec[:64], table, 0)
    with pytest.raises(ValueError):
        ap.decode_record(out[:-1], table, 1)


def test_malformed_record_is_rejected() -> None:
    rng = np.random.default_rng(1)
    rec = synth.bf16_rne(rng.standard_normal((128, 128)).astype(np.float32))
    table = ap.calibrate_table((rec >> 8).astype(np.uint8))
    out = bytearray(host_codec.encode(rec, ap.rank_table(table), 0))
    out[ap.DENSE_BYTES] ^= 0xFF  # escape count no longer matches the codes
    with pytest.raises(ValueError):
        host_codec.decode(bytes(out), table, 0)
