"""The CPU oracle against the golden vectors produced by the reference codec.

``tests/golden/codec_golden.npz`` and ``codec_hashes.json`` were written by
``tests/golden/make_golden.py`` from the reference's
``fragpack.compression.attn_page`` / ``attn_tables``; these tests pin the C
restatement in ``oracle/`` (and the product's host-side table builders) to
them.  The cases follow the reference's own unit tests
(``tests/unit/test_attn_page.py``).
"""

from __future__ import annotations

import hashlib
import os
import json
from pathlib import Path
import sys

import numpy as np
import pytest

import oracle
from fragpack_b200.compression import attn_page as ap
from fragpack_b200.compression import attn_tables as at

GOLDEN = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLDEN))
import make_golden  # noqa: E402


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN / "codec_golden.npz")


def test_kernel_order_matches_reference(golden) -> None:
    assert np.array_equal(oracle.kernel_order(0), golden["order_k"])
    assert np.array_equal(oracle.kernel_order(1), golden["order_v"])
    for kv in (0, 1):
        assert np.array_equal(np.sort(oracle.kernel_order(kv)), np.arange(128 * 128))


def test_encode_matches_reference_bytes(golden) -> None:
    for i, name in enumerate(golden["names"]):
        want = golden["encoded"][i, : golden["lens"][i]].tobytes()
        got = oracle.encode_record(golden["records"][i], golden["tables"][i], int(golden["kv"][i]))
        assert got == want, name


def test_decode_round_trips(golden) -> None:
    for i, name in enumerate(golden["names"]):
        rec = golden["encoded"][i, : golden["lens"][i]].tobytes()
        out = oracle.decode_record(rec, golden["tables"][i], int(golden["kv"][i]))
        assert np.array_equal(out, golden["records"][i]), name


def test_reference_unit_test_cases(golden) -> None:
    """Sizes the reference's unit tests assert (tests/unit/test_attn_page.py:16-47)."""
    names = list(golden["names"])
    esc = names.index("unit_escapes")
    assert golden["lens"][esc] % 16 == 0
    assert golden["lens"][esc] <= oracle.DENSE_BYTES + oracle.VAR_CAP
    raw = names.index("unit_incompressible")
    assert golden["lens"][raw] == oracle.RAW_RECORD_BYTES
    gauss = names.index("gauss_k")
    assert golden["lens"][gauss] < 0.75 * oracle.RAW_RECORD_BYTES
    junk = names.index("junk2_k")
    assert golden["lens"][junk] == oracle.RAW_RECORD_BYTES


def test_rejects_wrong_record_size() -> None:
    with pytest.raises(ValueError):
        oracle.encode_record(np.zeros(10, np.uint16), np.arange(22, dtype=np.uint8), 0)
    with pytest.raises(ValueError):
        ap.encode_record(np.zeros(10, np.uint16), np.arange(22, dtype=np.uint8), 0)


def test_tables_and_luts_match_reference(golden) -> None:
    for i in range(len(golden["names"])):
        table = golden["tables"][i]
        plut, slut = oracle.luts(table)
        assert np.array_equal(plut, golden["plut"][i])
        assert np.array_equal(slut, golden["slut"][i])
        # The product's host-side builders give the same words.
        assert ap.primary_lut(table) == tuple(int(v) for v in golden["plut"][i])
        assert ap.secondary_lut(table) == golden["slut"][i].tobytes()
    first = golden["records"][0]
    assert np.array_equal(
        oracle.calibrate_table((first >> 8).astype(np.uint8)), golden["tables"][0]
    )
    assert np.array_equal(ap.calibrate_table((first >> 8).astype(np.uint8)), golden["tables"][0])


def test_calibrate_ties_go_to_smaller_byte() -> None:
    high = np.array([9, 9, 3, 3, 200, 200, 7], np.uint8)
    for fn in (oracle.calibrate_table, ap.calibrate_table):
        table = fn(high)
        assert list(table[:4]) == [3, 9, 200, 7]
        assert list(table[4:8]) == [0, 1, 2, 4]


def test_small_configuration_hashes() -> None:
    """Config 1 (1 layer, 4 KV heads, 2 x 4 full blocks): 64 records by hash."""
    want = json.loads((GOLDEN / "codec_hashes.json").read_text())
    dump, kv = make_golden.cfg1_inputs()
    assert hashlib.sha256(kv.tobytes()).hexdigest() == want["input_sha256"]
    assert hashlib.sha256(dump.tobytes()).hexdigest() == want["dump_sha256"]
    table = oracle.calibrate(dump)
    assert table.tolist() == want["table"]
    assert at.calibrate(dump).tolist() == want["table"]
    blocks = make_golden.CFG1["seqs"] * make_golden.CFG1["blocks"]
    per_block = kv.reshape(2, blocks, 128, make_golden.CFG1["kv_heads"], 128)
    total = 0
    for key, (length, digest) in want["records"].items():
        b, k, h = (int(x) for x in key.split("."))
        rec = oracle.encode_record(per_block[k, b, :, h], table[0, k, h], k)
        assert len(rec) == length and hashlib.sha256(rec).hexdigest() == digest, key
        assert np.array_equal(oracle.decode_record(rec, table[0, k, h], k), per_block[k, b, :, h])
        total += len(rec)
    assert total / len(want["records"]) == pytest.approx(want["mean_record_bytes"])


def test_batch_forms_agree_with_single_records(golden) -> None:
    recs, tables, kv = golden["records"], golden["tables"], golden["kv"]
    out, lens = oracle.encode_records(recs, tables, kv)
    assert np.array_equal(lens, golden["lens"])
    for i in range(len(lens)):
        assert np.array_equal(out[i, : lens[i]], golden["encoded"][i, : lens[i]])
    assert np.array_equal(oracle.decode_records(out, lens, tables, kv), recs)


def test_raw_record_is_the_staging_layout(golden) -> None:
    i = list(golden["names"]).index("unit_incompressible")
    raw = oracle.raw_record(golden["records"][i], int(golden["kv"][i]))
    assert raw == golden["encoded"][i].tobytes()


# The reference checkout: $FRAGPACK_REFERENCE, else `reference` beside this repository.
REFERENCE = Path(os.environ.get("FRAGPACK_REFERENCE") or Path(__file__).resolve().parents[2] / "reference")


@pytest.mark.skipif(not (REFERENCE / "fragpack").exists(), reason="reference checkout absent")
def test_live_cross_check_against_reference() -> None:
    """Where the reference checkout is present, compare on fresh seeded records."""
    import importlib

    sys.path.insert(0, str(REFERENCE))
    try:
        ref = importlib.import_module("fragpack.compression.attn_page")
    finally:
        sys.path.remove(str(REFERENCE))
    from benchmarks import synth

    rng = np.random.default_rng(99)
    scales = synth.channel_scales(5, 1, 2)[0]
    for junk in (0.0, 0.008, 0.011, 0.02):
        kv = synth.kv_tokens_numpy(rng, scales, 128, heavy=0.005, junk=junk)
        for k in (0, 1):
            for h in range(2):
                rec = kv[k, :, h]
                table = ref.calibrate_table((rec >> 8).astype(np.uint8))
                assert ref.encode_record(rec, table, k) == oracle.encode_record(rec, table, k)
