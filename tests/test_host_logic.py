"""Host-side logic and the C-ABI surface (no GPU needed).

Covers: the library loads and exports every symbol ``include/fragpack_b200.h``
declares; the operators refuse host tensors loudly (no CPU fallback); sizes
and layout arithmetic the reference documents (page bytes, workspace sizes,
blob sizes, ``memory_usage`` as in ``tests/unit/test_hbm_capacity.py``); table
building and head slicing.
"""

from __future__ import annotations

from pathlib import Path
import re

import numpy as np
import pytest
import torch

import oracle
from benchmarks import synth, workloads
from fragpack_b200.compression import attn_page as ap
from fragpack_b200.compression import attn_tables as at
from fragpack_b200.ops import fused_attn_decode as fad
from fragpack_b200.ops import hbm_kv
from fragpack_b200.ops.fragpack_ext import EXPORTED, extension
from fragpack_b200.ops.tp import head_shard

ROOT = Path(__file__).resolve().parents[1]


def test_library_exports_every_declared_symbol() -> None:
    header = (ROOT / "include" / "fragpack_b200.h").read_text()
    declared = set(re.findall(r"\b(fp_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations parsed"
    lib = extension()
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared but not exported"
    assert declared == set(EXPORTED)
    assert b"sm_100a" in lib.fp_version()


def test_argument_errors_need_no_gpu() -> None:
    lib = extension()
    rc = lib.fp_decode_workspace(0, 4, None, None, None)
    assert rc != 0 and b"workspace" in lib.fp_last_error()
    import ctypes

    sizes = [ctypes.c_int64() for _ in range(3)]
    assert lib.fp_decode_workspace(4, 77, *(ctypes.byref(s) for s in sizes)) == 0
    assert tuple(s.value for s in sizes) == fad.workspace_elems(4, 77)


def test_decode_entry_points_reject_bad_geometry_before_any_launch() -> None:
    """Rejected arguments return FP_ERR_ARGUMENT with a message; nothing is enqueued (no GPU here)."""
    import ctypes

    from fragpack_b200.ops.fragpack_ext import FpPeers

    lib = extension()
    fake = 0x1000  # never dereferenced: the checks below fail first
    common = dict(batch=2, kv_heads=2, units=4)

    def fused(group=8, units=4, plan_elems=10**6, opart_elems=10**9):
        return lib.fp_fused_decode(fake, 2048, fake, fake, fake, fake, fake, 8, fake, fake, opart_elems,
                                   fake, 10**9, fake, plan_elems, fake, 2048, common["batch"],
                                   common["kv_heads"], group, units, 1, 0.088, 148, None)

    assert fused(group=3) == -1 and b"query group" in lib.fp_last_error()
    assert fused(units=1) == -1 and b"unit" in lib.fp_last_error()
    assert fused(plan_elems=4) == -1 and b"plan" in lib.fp_last_error()
    assert fused(opart_elems=16) == -1 and b"workspace" in lib.fp_last_error()

    peers = FpPeers()
    peers.world, peers.rank = 9, 0
    peers.epoch = peers.status = fake
    rc = lib.fp_fused_decode_peers(fake, 2048, fake, fake, fake, fake, fake, 8, fake, fake, 10**9, fake,
                                   10**9, fake, 10**6, ctypes.byref(peers), 0, 2048 * 9, 2, 2, 8, 4, 1,
                                   0.088, 148, None)
    assert rc == -1 and b"peer group" in lib.fp_last_error()
    peers.world = 2
    rc = lib.fp_fused_decode_peers(fake, 2048, fake, fake, fake, fake, fake, 8, fake, fake, 10**9, fake,
                                   10**9, fake, 10**6, ctypes.byref(peers), 2, 4096, 2, 2, 8, 4, 1,
                                   0.088, 148, None)
    assert rc == -1 and b"buffer 2" in lib.fp_last_error()
    rc = lib.fp_fused_decode_noalloc(fake, 2048, fake, fake, fake, fake, fake, 8, fake, fake, 2048, 2, 64,
                                     8, 5000, 1, 0.088, 148, None)
    assert rc == -1 and b"built-in decode scratch" in lib.fp_last_error()


def test_operators_have_no_cpu_fallback() -> None:
    q = torch.zeros(1, 8, 128, dtype=torch.bfloat16)
    dummy = torch.zeros(1, 2, 1, dtype=torch.int64)
    tabs = fad.RecordTables(dummy, dummy.int(), torch.zeros(2, 1, 2, dtype=torch.int32),
                            torch.zeros(2, 1, 16, dtype=torch.uint8))
    ws = (torch.zeros(8), torch.zeros(8), torch.zeros(8, dtype=torch.int32))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        fad.decode_attention(q, tabs, torch.zeros(1, 1, dtype=torch.int32),
                             torch.zeros(1, dtype=torch.int32), 1.0, 1, q.clone(), ws, True)
    with pytest.raises(ValueError):
        fad.decode_attention(torch.zeros(1, 3, 128, dtype=torch.bfloat16), tabs,
                             torch.zeros(1, 1, dtype=torch.int32),
                             torch.zeros(1, dtype=torch.int32), 1.0, 1, q, ws, True)
    # Only the offline compression package has a host form (tests/test_host_codec.py);
    # the store, like the decode operator, refuses host tensors.
    store = object.__new__(hbm_kv.HbmKvStore)
    store.counters = torch.zeros(16, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        store._require_device()


def test_layout_arithmetic() -> None:
    assert ap.DENSE_BYTES == 22528 and ap.RAW_RECORD_BYTES == 32768 and ap.VAR_CAP == 2048
    assert hbm_kv.page_bytes(4) == 190464  # reference docs/architecture.md:15-18
    assert hbm_kv.RAW_VAR_LEN == 10240
    assert fad.decode_units(4, 4, 148) == 4 + fad.SPLIT_WAVES * 74 - 1
    assert fad.decode_units(3, 0, 148) >= 3
    opart, ml, plan = fad.workspace_elems(4, 77)
    # plan: header, unit and sequence tables, spare + status words, the dynamic schedule words,
    # then four words per unit of item descriptors
    assert (opart, ml, plan) == (4 * 77 * 8 * 128, 4 * 77 * 8 * 2, 2 + 4 * 77 + 2 + 4 + 256 + 4 * 77)
    assert ap.blob_head_bytes(2, 2) == 4096
    assert ap.blob_slot_bytes(2, 2) == 4096 + 2 * 2 * 2 * 32768
    assert ap.blob_head_bytes(80, 8) == -(-(64 + 8 * 80 * 8) // 4096) * 4096
    assert hbm_kv.blob_failures(5) == "bad header, overflow full"


def _tables(layers: int, heads: int) -> np.ndarray:
    rng = np.random.default_rng(0)
    table = np.empty((layers, 2, heads, 22), np.uint8)
    for idx in np.ndindex(layers, 2, heads):
        table[idx] = rng.permutation(256)[:22]
    return table


def test_device_tables_match_oracle_luts() -> None:
    table = _tables(2, 3)
    dev = at.device_tables(table, torch.device("cpu"))
    assert dev.rank_of.shape == (2, 2, 3, 256) and dev.plut.shape == (2, 2, 3, 2)
    assert dev.slut.shape == (2, 2, 3, 16)
    for idx in np.ndindex(2, 2, 3):
        plut, slut = oracle.luts(table[idx])
        assert np.array_equal(dev.plut[idx].numpy().view(np.uint32), plut)
        assert np.array_equal(dev.slut[idx].numpy(), slut)
        rank = dev.rank_of[idx].numpy()
        assert np.array_equal(rank[table[idx]], np.arange(22))
        assert (rank == 255).sum() == 256 - 22
    with pytest.raises(ValueError):
        at.device_tables(table[..., :21], torch.device("cpu"))


def test_load_tables_head_slice(tmp_path) -> None:
    table = _tables(2, 4)
    path = tmp_path / "tables.npz"
    np.savez(path, table=table)
    full = at.load_tables(str(path), torch.device("cpu"))
    for rank in range(2):
        part = at.load_tables(str(path), torch.device("cpu"), heads=head_shard(rank, 2, 4))
        assert torch.equal(part.plut, full.plut[:, :, 2 * rank : 2 * rank + 2])
        assert torch.equal(part.rank_of, full.rank_of[:, :, 2 * rank : 2 * rank + 2])
    with pytest.raises(ValueError):
        at.load_tables(str(path), torch.device("cpu"), heads=slice(4, 8))
    with pytest.raises(ValueError):
        head_shard(0, 3, 8)


def test_memory_usage_counts_real_strides() -> None:
    """As the reference's tests/unit/test_hbm_capacity.py: arena rows by their strides."""
    layers, heads, blocks = 3, 2, 5
    table = _tables(layers, heads)
    caches = [torch.zeros(blocks, hbm_kv.page_bytes(heads) + 32, dtype=torch.uint8)[:, :-32]
              for _ in range(layers)]
    store = hbm_kv.HbmKvStore(caches, heads, at.device_tables(table, torch.device("cpu")),
                              max_tokens=256, staging_slots=2, overflow_records=3)
    usage = store.memory_usage()
    assert usage["arena"] == blocks * layers * (hbm_kv.page_bytes(heads) + 32)
    assert usage["staging"] == 2 * layers * 2 * heads * 32768
    assert usage["scratch"] == (256 // 128 + 2 + 2) * 2 * heads * 32768
    assert usage["overflow"] == 3 * 32768
    assert usage["codebooks"] == layers * 2 * heads * (256 + 8 + 16)
    assert usage["metadata"] > 0
    # Overflow bitmap: bits past the pool are preset so they are never handed out.
    assert store.ovf_bits.numpy().view(np.uint32)[0] == 0xFFFFFFF8
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        store.commit()
    with pytest.raises(ValueError):
        hbm_kv.HbmKvStore(caches, heads + 1, at.device_tables(table, torch.device("cpu")), 256, 2, 3)


def test_store_registry() -> None:
    hbm_kv._ACTIVE = None
    with pytest.raises(RuntimeError):
        hbm_kv.active_store()
    marker = object()
    hbm_kv.register_store(marker)  # type: ignore[arg-type]
    assert hbm_kv.active_store() is marker
    hbm_kv._ACTIVE = None


def test_synthetic_workloads_are_seeded() -> None:
    scales = synth.channel_scales(3, 2, 2)
    assert scales.shape == (2, 2, 2, 128)
    ratio = scales[0, 0, 0, list(synth.K_OUTLIER_CHANNELS)].mean() / np.delete(
        scales[0, 0, 0], list(synth.K_OUTLIER_CHANNELS)).mean()
    assert ratio > 4
    a = synth.kv_tokens_numpy(np.random.default_rng(1), scales[0], 64, heavy=0.01, junk=0.02)
    b = synth.kv_tokens_numpy(np.random.default_rng(1), scales[0], 64, heavy=0.01, junk=0.02)
    assert np.array_equal(a, b) and a.shape == (2, 64, 2, 128)
    assert ((a & 0x7F80) != 0x7F80).all()  # finite
    assert np.array_equal(synth.bf16_rne(np.array([1.0, 1.00390625], np.float32)),
                          np.array([0x3F80, 0x3F80], np.uint16))
    lens = workloads.context_lengths(workloads.CONFIGS["c3"], 5)
    assert lens.shape == (64,) and (lens % 128 != 0).all() and lens.min() >= 1000 and lens.max() <= 4096
    assert (workloads.context_lengths(workloads.CONFIGS["c2"], 5) == 8192).all()
