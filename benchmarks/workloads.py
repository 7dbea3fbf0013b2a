"""The benchmark configurations as seeded synthetic workloads.

Each configuration names a KV geometry and a batch; :func:`build_decode_workload`
fills an :class:`~fragpack_b200.ops.hbm_kv.HbmKvStore` for it on the current
CUDA device by driving the store exactly as a serving engine would (prepare,
write, encode per layer, commit), in chunks of sequences so that staging stays
small.  Physical blocks are assigned by a random permutation and never
repeated, so every timed read comes from HBM.

The KV values follow :mod:`benchmarks.synth`; tables are calibrated per
layer from 64 seeded sample pages drawn from the same distribution.
"""

from __future__ import annotations

from dataclasses import dataclass, replace

import numpy as np
import torch

from benchmarks import synth
from fragpack_b200.compression import attn_page as ap
from fragpack_b200.compression.attn_tables import DeviceTables, device_tables
from fragpack_b200.ops.hbm_kv import HbmKvStore, page_bytes

BLOCK = 128


@dataclass(frozen=True)
class Config:
    """One benchmark configuration.

    Attributes:
        name: Short name used in reports.
        layers: Model layers.
        kv_heads: KV heads (before any head sharding).
        q_heads: Query heads.
        batch: Decode batch (sequences).
        ctx_min, ctx_max: Context lengths are uniform in ``[ctx_min, ctx_max]``;
            equal values give a fixed context.
        ragged: Re-draw lengths that are multiples of 128, so every sequence
            ends in an open (raw, writable) tail block.
        heavy, junk: Contamination fractions (see :mod:`benchmarks.synth`).
    """

    name: str
    layers: int
    kv_heads: int
    q_heads: int
    batch: int
    ctx_min: int
    ctx_max: int
    ragged: bool = False
    heavy: float = 0.0
    junk: float = 0.0

    @property
    def group(self) -> int:
        return self.q_heads // self.kv_heads


CONFIGS = {
    # CPU-runnable reference case: 1 layer, GQA 4, 2 x 512 tokens.
    "c1": Config("c1-cpu-reference", 1, 4, 16, 2, 512, 512),
    # Qwen3-30B-A3B-like: 48 layers, 4 KV heads, GQA 8, batch 4 at 8192.
    "c2": Config("c2-qwen3-30b-a3b-like", 48, 4, 32, 4, 8192, 8192),
    # Llama-3-8B-like: 32 layers, 8 KV heads, GQA 4, batch 64, ragged 1000..4096, 0.5% x64.
    "c3": Config("c3-llama3-8b-like-ragged", 32, 8, 32, 64, 1000, 4096, ragged=True, heavy=0.005),
    # Prefill + encode stress: MHA, 32 layers, 32 KV heads, 16 x 8192, 2% junk.
    "c4": Config("c4-prefill-encode-mha", 32, 32, 32, 16, 8192, 8192, junk=0.02),
    # Llama-3-70B-like: 80 layers, 8 KV heads, GQA 8, batch 128 at 32768.
    "c5": Config("c5-llama3-70b-like", 80, 8, 64, 128, 32768, 32768),
}


def context_lengths(cfg: Config, seed: int) -> np.ndarray:
    """Seeded context lengths of the batch (int32 ``[B]``)."""
    rng = np.random.default_rng(seed)
    lens = rng.integers(cfg.ctx_min, cfg.ctx_max + 1, size=cfg.batch)
    if cfg.ragged:
        while True:
            again = lens % BLOCK == 0
            if not again.any():
                break
            lens[again] = rng.integers(cfg.ctx_min, cfg.ctx_max + 1, size=int(again.sum()))
    return lens.astype(np.int32)


def calibrate_on_device(
    gen: torch.Generator, scales: torch.Tensor, heavy: float, junk: float, samples: int = 64
) -> np.ndarray:
    """Tables ``uint8 [2, H, 22]`` of one layer from ``samples`` seeded pages.

    Same rule as ``attn_tables.calibrate`` (count the high bytes, keep the 22
    most frequent, ties to the smaller byte) with the histogram taken on the
    device the samples are drawn on.
    """
    kv = synth.kv_tokens_torch(gen, scales, samples * BLOCK, heavy, junk)  # [2, T, H, 128]
    high = (kv.view(torch.int16).to(torch.int32) >> 8) & 0xFF
    heads = scales.shape[1]
    out = np.empty((2, heads, ap.TABLE_ENTRIES), np.uint8)
    for k in range(2):
        for h in range(heads):
            counts = torch.bincount(high[k, :, h].reshape(-1), minlength=256).cpu().numpy()
            out[k, h] = np.lexsort((np.arange(256), -counts))[: ap.TABLE_ENTRIES]
    return out


@dataclass
class DecodeWorkload:
    """A filled store plus the batch that reads it.

    Attributes:
        cfg: Geometry actually built (KV heads after sharding, resident layers).
        store: The filled store.
        arenas: Arena tensors (kept alive here).
        block_table: int32 ``[B, pages]`` on the device.
        seq_lens: int32 ``[B]`` on the device.
        lens_host: The same lengths on the host.
        table: uint8 ``[L, 2, H, 22]`` calibrated tables.
        compressed_bytes: Per layer, bytes of every K and V record the batch reads.
        logical_bytes: Per layer, ``sum(ctx) * 2 * H * 128 * 2``.
        sample: Optional ``(layer, KV [2, tokens, H, 128] bf16)`` kept for validation.
    """

    cfg: Config
    store: HbmKvStore
    arenas: list[torch.Tensor]
    block_table: torch.Tensor
    seq_lens: torch.Tensor
    lens_host: np.ndarray
    table: np.ndarray
    compressed_bytes: list[int]
    logical_bytes: int
    sample: dict


def build_decode_workload(
    cfg: Config,
    device: torch.device,
    seed: int = 0,
    layers: int | None = None,
    head_slice: slice = slice(None),
    chunk_tokens: int = 1 << 18,
    keep_layers: tuple[int, ...] = (0,),
    keep_seqs: int = 2,
    overflow_records: int = 8192,
    plain: bool = False,
) -> DecodeWorkload:
    """Fill a store with the configuration's KV on ``device``.

    Args:
        cfg: Configuration.
        device: CUDA device.
        seed: Seed of every random draw.
        layers: Resident layers (default: all of ``cfg.layers``).
        head_slice: KV heads this rank holds (tensor-parallel shard).
        chunk_tokens: Tokens written per store step.
        keep_layers: Layers whose source KV of the first ``keep_seqs``
            sequences is kept (as BF16) for validation.
        keep_seqs: Sequences kept per kept layer.
        overflow_records: Capacity of the overflow pool (``FRAGPACK_OVERFLOW``).
        plain: Build the plain-BF16 comparison workload: tables that match no
            value of the data, so the encoder sends every closed block to the
            overflow pool as a raw 32 KiB record; the pool is sized to hold them
            all (``overflow_records`` is ignored).

    Returns:
        The workload.
    """
    n_layers = layers if layers is not None else cfg.layers
    all_scales = synth.channel_scales(seed + 1, n_layers, cfg.kv_heads)[:, :, head_slice]
    heads = all_scales.shape[2]
    cfg = replace(cfg, layers=n_layers, kv_heads=heads, q_heads=heads * cfg.group)
    lens = context_lengths(cfg, seed + 2)
    pages = (lens + BLOCK - 1) // BLOCK
    n_blocks = int(pages.sum()) + 1  # + a never-written null block (id 0)
    rng = np.random.default_rng(seed + 3)
    ids = rng.permutation(np.arange(1, n_blocks)).astype(np.int32)
    width = int(pages.max())
    bt = np.zeros((cfg.batch, width), np.int32)
    at = 0
    for b in range(cfg.batch):
        bt[b, : pages[b]] = ids[at : at + pages[b]]
        at += pages[b]

    gen = torch.Generator(device=device)
    gen.manual_seed(seed + 4)
    scales_dev = torch.from_numpy(all_scales).to(device)
    if plain:
        # High bytes 0x60..0x75 are magnitudes of 2^65 and more: absent from the
        # data, so every scalar would be a raw entry and no record codes.
        table = np.broadcast_to(
            np.arange(0x60, 0x60 + ap.TABLE_ENTRIES, dtype=np.uint8), (n_layers, 2, heads, ap.TABLE_ENTRIES)
        ).copy()
        overflow_records = n_layers * n_blocks * 2 * heads + 64
    else:
        table = np.stack(
            [calibrate_on_device(gen, scales_dev[layer], cfg.heavy, cfg.junk)
             for layer in range(n_layers)]
        )
    tables: DeviceTables = device_tables(table, device)
    page = page_bytes(heads)
    arenas = [torch.empty((n_blocks, page), dtype=torch.uint8, device=device) for _ in range(n_layers)]
    # Every sequence may keep one open tail.
    chunk_tokens = max(chunk_tokens, int(lens.max()))
    store = HbmKvStore(
        arenas, heads, tables, max_tokens=chunk_tokens, staging_slots=cfg.batch + 1,
        overflow_records=overflow_records,
    )

    sample: dict = {}
    # Sequences are written whole, several per step, as a prefill would.
    order = list(range(cfg.batch))
    start = 0
    open_tails: list[int] = []
    while start < len(order):
        group, tokens = [], 0
        while start < len(order) and (not group or tokens + lens[order[start]] <= chunk_tokens):
            group.append(order[start])
            tokens += int(lens[order[start]])
            start += 1
        slots = np.concatenate(
            [bt[b, np.arange(lens[b]) // BLOCK].astype(np.int64) * BLOCK + np.arange(lens[b]) % BLOCK
             for b in group]
        )
        slot_t = torch.from_numpy(slots).to(device)
        closes = int(sum(lens[b] // BLOCK for b in group))
        open_tails += [int(bt[b, pages[b] - 1]) for b in group if lens[b] % BLOCK]
        store.prepare(slot_t, int(slots.size), np.array(open_tails, np.int32))
        for layer in range(n_layers):
            kv = synth.kv_tokens_torch(gen, scales_dev[layer], int(slots.size), cfg.heavy, cfg.junk)
            if layer in keep_layers:
                off = 0
                for b in group:
                    if b < keep_seqs:
                        sample[(layer, b)] = kv[:, off : off + int(lens[b])].clone()
                    off += int(lens[b])
            store.write(layer, kv[0], kv[1], slot_t)
            store.encode(layer, closes)
        store.commit()
    torch.cuda.synchronize(device)
    store.stats()  # raises StoreError if anything was dropped

    rec_len = store.rec_len  # [L, NB, 2, H]
    bt_dev = torch.from_numpy(bt).to(device)
    used = torch.from_numpy(np.concatenate([bt[b, : pages[b]] for b in range(cfg.batch)])).to(device)
    compressed = [
        int((rec_len[layer, used.long()].to(torch.int64) + ap.DENSE_BYTES).sum().item())
        for layer in range(n_layers)
    ]
    logical = int(lens.astype(np.int64).sum()) * 2 * heads * 128 * 2
    return DecodeWorkload(
        cfg=cfg,
        store=store,
        arenas=arenas,
        block_table=bt_dev,
        seq_lens=torch.from_numpy(lens).to(device),
        lens_host=lens,
        table=table,
        compressed_bytes=compressed,
        logical_bytes=logical,
        sample=sample,
    )


__all__ = [
    "CONFIGS",
    "Config",
    "DecodeWorkload",
    "build_decode_workload",
    "calibrate_on_device",
    "context_lengths",
]
