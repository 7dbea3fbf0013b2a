"""Generate the golden codec vectors by importing the reference codec.

Run where the reference checkout is available (it is not needed afterwards)::

    python tests/golden/make_golden.py /path/to/reference

Writes next to this script:

* ``codec_golden.npz`` - a handful of input records with the bytes the
  reference ``fragpack.compression.attn_page.encode_record`` produced for them,
  their tables (``calibrate_table``), LUT words and the kernel-order
  permutations;
* ``codec_hashes.json`` - SHA-256 of the reference encoder's output for every
  record of the small CPU configuration (1 layer, 4 KV heads, 2 sequences of
  4 full blocks, tables calibrated on 64 seeded sample pages), whose inputs the
  tests regenerate from the same seeds.
"""

from __future__ import annotations

import hashlib
import json
import os
from pathlib import Path
import sys

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))

from benchmarks import synth  # noqa: E402

CFG1 = dict(seed=1001, layers=1, kv_heads=4, seqs=2, blocks=4, samples=64)


def cfg1_inputs() -> tuple[np.ndarray, np.ndarray]:
    """Return ``(dump [S,1,2,128,4,128], kv [2, seqs*blocks*128, 4, 128])`` of config 1."""
    scales = synth.channel_scales(CFG1["seed"], CFG1["layers"], CFG1["kv_heads"])
    dump = synth.calibration_dump(CFG1["seed"] + 1, scales, CFG1["samples"])
    rng = np.random.default_rng(CFG1["seed"] + 2)
    kv = synth.kv_tokens_numpy(rng, scales[0], CFG1["seqs"] * CFG1["blocks"] * 128)
    return dump, kv


def _trunc_bf16(rng: np.random.Generator, scale: float) -> np.ndarray:
    """BF16 by truncation, as the reference unit tests draw it (tests/unit/test_attn_page.py:9-13)."""
    values = (rng.standard_normal((128, 128)) * scale).astype(np.float32)
    return (values.view(np.uint32) >> 16).astype(np.uint16)


def small_cases() -> list[tuple[str, np.ndarray, np.ndarray | None, int]]:
    """(name, record, table-or-None, kv); a None table is calibrated on the record's draw."""
    cases = []
    scales = synth.channel_scales(7, 1, 1)[0]
    rng = np.random.default_rng(8)
    for name, heavy, junk in (
        ("gauss", 0.0, 0.0),
        ("heavy", 0.005, 0.0),
        ("junk09", 0.0, 0.009),
        ("junk2", 0.0, 0.02),
    ):
        kv = synth.kv_tokens_numpy(rng, scales, 128, heavy, junk)
        cases.append((f"{name}_k", kv[0, :, 0], None, 0))
        if name in ("gauss", "junk09"):
            cases.append((f"{name}_v", kv[1, :, 0], None, 1))
    # The reference's own unit-test inputs (tests/unit/test_attn_page.py:16-47).
    rng0 = np.random.default_rng(0)
    cal = _trunc_bf16(rng0, 0.5)
    rec = _trunc_bf16(rng0, 0.5)
    rec[3, 5] = 0x7F00 | (rec[3, 5] & 0xFF)
    rec[100, 127] = 0x0100
    cases.append(("unit_escapes", rec, ("cal", cal), 1))
    rng2 = np.random.default_rng(2)
    cases.append(
        (
            "unit_incompressible",
            rng2.integers(0, 1 << 16, size=(128, 128), dtype=np.uint16),
            ("table", np.arange(22, dtype=np.uint8)),
            0,
        )
    )
    return cases


def main() -> None:
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get(
        "FRAGPACK_REFERENCE", str(Path(__file__).resolve().parents[3] / "reference"))
    sys.path.insert(0, ref_root)
    from fragpack.compression import attn_page as ap
    from fragpack.compression import attn_tables as at

    names, records, tables, kvs, encoded, lens = [], [], [], [], [], []
    for name, rec, tab, kv in small_cases():
        if tab is None:
            table = ap.calibrate_table((rec >> 8).astype(np.uint8))
        elif tab[0] == "cal":
            table = ap.calibrate_table((tab[1] >> 8).astype(np.uint8))
        else:
            table = tab[1]
        out = ap.encode_record(rec, table, kv)
        assert np.array_equal(ap.decode_record(out, table, kv), rec)
        buf = np.zeros(ap.RAW_RECORD_BYTES, np.uint8)
        buf[: len(out)] = np.frombuffer(out, np.uint8)
        names.append(name)
        records.append(rec)
        tables.append(table)
        kvs.append(kv)
        encoded.append(buf)
        lens.append(len(out))
    tables_arr = np.stack(tables)
    plut = np.array([ap.primary_lut(t) for t in tables_arr], np.uint32)
    slut = np.stack([np.frombuffer(ap.secondary_lut(t), np.uint8) for t in tables_arr])
    np.savez_compressed(
        HERE / "codec_golden.npz",
        names=np.array(names),
        records=np.stack(records),
        tables=tables_arr,
        kv=np.array(kvs, np.int32),
        encoded=np.stack(encoded),
        lens=np.array(lens, np.int32),
        plut=plut,
        slut=slut,
        order_k=ap._ORDER[0].astype(np.int32),
        order_v=ap._ORDER[1].astype(np.int32),
    )

    dump, kv = cfg1_inputs()
    table = at.calibrate(dump)
    blocks = CFG1["seqs"] * CFG1["blocks"]
    per_block = kv.reshape(2, blocks, 128, CFG1["kv_heads"], 128)
    hashes = {}
    total = 0
    for b in range(blocks):
        for k in range(2):
            for h in range(CFG1["kv_heads"]):
                out = ap.encode_record(per_block[k, b, :, h], table[0, k, h], k)
                hashes[f"{b}.{k}.{h}"] = [len(out), hashlib.sha256(out).hexdigest()]
                total += len(out)
    payload = {
        "config": CFG1,
        "input_sha256": hashlib.sha256(kv.tobytes()).hexdigest(),
        "dump_sha256": hashlib.sha256(dump.tobytes()).hexdigest(),
        "table": table.tolist(),
        "mean_record_bytes": total / len(hashes),
        "records": hashes,
    }
    (HERE / "codec_hashes.json").write_text(json.dumps(payload, indent=1) + "\n")
    print("wrote", len(names), "records and", len(hashes), "hashes; mean bytes", payload["mean_record_bytes"], "lens", lens)


if __name__ == "__main__":
    main()
