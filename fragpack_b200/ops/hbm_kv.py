"""HBM-resident FragPack KV store over a paged KV cache (sm_100a kernels).

Same public API and state layout as the reference ``fragpack/ops/hbm_kv.py``
(``HbmKvStore``, ``page_bytes``, ``StoreStats``, ``StoreError``,
``register_store`` / ``active_store``, ``blob_failures``), so callers and the
reference's tests switch by import path only.

The engine's paged KV cache is the arena: row ``b`` of layer ``l`` is one page
shared by the block's ``2 H`` records, packed back to back in encode order.
``rec_addr[L, NB, 2, H]`` / ``rec_len[L, NB, 2, H]`` locate every record, so a
record can live in its block's page, in staging while its block is still
filling (raw, in fragment order), or raw in the overflow pool when it does not
code or its page is full.  Staging comes in persistent slots ``[S_p, L, 2, H,
32768]`` for blocks open across steps and transient scratch ``[S_t, 2, H,
32768]`` for blocks that open and close within a step (reference
``hbm_kv.py:16-38``).

Per step: :meth:`HbmKvStore.prepare` (once), then per layer :meth:`write`,
attention, :meth:`encode`, and :meth:`commit` after the last layer.  The
per-layer calls have launch shapes fixed by host values and are CUDA-graph
safe.  The kernels are reached through the C ABI (``fp_hbm_*``); the thirteen
state tensors the reference passes positionally travel as one ``fp_store``
struct built once.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
import hashlib

import numpy as np
import torch

from fragpack_b200.compression import attn_page as ap
from fragpack_b200.compression.attn_tables import DeviceTables
from fragpack_b200.logging import init_logger
from fragpack_b200.ops.fragpack_ext import FpStore, check, extension, stream_ptr

logger = init_logger(__name__)

BLOCK_TOKENS = 128
HEAD_DIM = 128
# Page budget per record past the dense part (reference hbm_kv.py:66-69).
VAR_SHARE = 1280
RAW_RECORD = 32768
RAW_VAR_LEN = RAW_RECORD - ap.DENSE_BYTES  # rec_len of a raw record

# Counter slots (include/fragpack_b200.h, FP_CTR_*).
_ERR_STAGING = 4
_ERR_OVERFLOW = 5
_FALLBACKS = 6
_ENCODED = 7
_SPILLS = 8
_OVF_FREE = 13
_N_COUNTERS = 16
_N_TAGS = 4
_BLOB_FAILURES = {1: "bad header", 2: "bad lengths", 4: "overflow full"}

_ACTIVE: "HbmKvStore | None" = None


def page_bytes(kv_heads: int) -> int:
    """Arena page bytes per block-layer: ``2 H * (DENSE_BYTES + VAR_SHARE)``."""
    return 2 * kv_heads * (ap.DENSE_BYTES + VAR_SHARE)


@dataclass(frozen=True)
class StoreStats:
    """Cumulative store counters (reference ``hbm_kv.py:102-119``).

    Attributes:
        encoded: Records encoded (all layers).
        fallbacks: Records stored raw in the overflow pool (includes spills).
        spills: Coded records stored raw because their block-layer page was full.
        err_staging: Claims dropped because staging was exhausted.
        err_overflow: Raw records dropped because the overflow pool was full.
    """

    encoded: int
    fallbacks: int
    spills: int
    err_staging: int
    err_overflow: int


class StoreError(RuntimeError):
    """Raised when the store dropped KV data (staging or overflow exhausted)."""


def register_store(store: "HbmKvStore") -> None:
    """Publish the process's store to the KV connector (``hbm_kv.py:126-139``)."""
    global _ACTIVE
    _ACTIVE = store


def active_store() -> "HbmKvStore":
    """Return the store published by :func:`register_store`.

    Raises:
        RuntimeError: If attention has not created one yet.
    """
    if _ACTIVE is None:
        raise RuntimeError("no FragPack KV store: the FragPack attention backend is not active")
    return _ACTIVE


def blob_failures(status: int) -> str:
    """Describe an import status word as comma-separated failure names."""
    return ", ".join(name for bit, name in _BLOB_FAILURES.items() if status & bit)


class HbmKvStore:
    """FragPack KV store whose arena is the engine's paged KV cache.

    Args:
        kv_caches: One uint8-viewable tensor per layer, in layer order; the
            page of block ``b`` at layer ``l`` is row ``b`` (stride a 16-byte
            multiple, normally :func:`page_bytes`).
        kv_heads: KV heads ``H``.
        tables: Calibrated lookup tables for every layer.
        max_tokens: Most tokens in one step.
        staging_slots: Persistent staging slots ``S_p`` (at least one per
            running request).
        overflow_records: Raw records the overflow pool can hold.

    Async/thread-safety:
        All methods enqueue on the current CUDA stream and must be called from
        the thread that drives the forward pass.
    """

    def __init__(
        self,
        kv_caches: list[torch.Tensor],
        kv_heads: int,
        tables: DeviceTables,
        max_tokens: int,
        staging_slots: int,
        overflow_records: int,
    ) -> None:
        dev = kv_caches[0].device
        self.num_layers = len(kv_caches)
        self.kv_heads = kv_heads
        self.num_blocks = kv_caches[0].shape[0]
        self.tables = tables
        if tuple(tables.rank_of.shape[:3]) != (self.num_layers, 2, kv_heads):
            raise ValueError(
                f"tables {tuple(tables.rank_of.shape)} do not match "
                f"L={self.num_layers}, H={kv_heads}"
            )
        # Identifies the codec tables, so blobs coded with others are rejected.
        self.table_digest = int.from_bytes(
            hashlib.blake2b(tables.rank_of.cpu().numpy().tobytes(), digest_size=8).digest(),
            "little",
            signed=True,
        )
        self.arena_base: list[int] = []
        self.arena_stride: list[int] = []
        for cache in kv_caches:
            stride = cache.stride(0) * cache.element_size()
            if cache.shape[0] != self.num_blocks or stride % 16:
                raise ValueError(
                    f"cache {tuple(cache.shape)} stride {stride} is not a 16-byte multiple"
                )
            self.arena_base.append(cache.data_ptr())
            self.arena_stride.append(stride)

        L, NB, H = self.num_layers, self.num_blocks, kv_heads
        i32 = dict(dtype=torch.int32, device=dev)
        # Blocks opening and closing in the step, plus one heir per persistent slot.
        transient = max_tokens // BLOCK_TOKENS + 2 + staging_slots
        self.max_tokens = max_tokens
        self.overflow_records = overflow_records
        self.counters = torch.zeros(_N_COUNTERS, **i32)
        self.counters[0] = staging_slots
        self.counters[_OVF_FREE] = overflow_records
        self.wslot = torch.full((NB,), -1, **i32)
        self.tags = torch.zeros((_N_TAGS, NB), **i32)
        self.free_stack = torch.arange(staging_slots, **i32)
        # One bit per overflow slot (set = in use); bits past the pool are preset.
        words = max(1, -(-overflow_records // 32))
        bits = np.zeros(words * 32, dtype=bool)
        bits[overflow_records:] = True
        self.ovf_bits = torch.from_numpy(
            np.packbits(bits, bitorder="little").view(np.int32).copy()
        ).to(dev)
        self.claim_list = torch.zeros(2 * max_tokens, **i32)
        self.close_list = torch.zeros(2 * max_tokens, **i32)
        # Bookkeeping of this library's prepare: who owns each staging slot,
        # and the blocks seen opening / closing in the current step.
        self.slot_owner = torch.full((staging_slots + transient,), -1, **i32)
        self.seen_list = torch.zeros(2 * max_tokens, **i32)
        # A never-claimed block reads as one all-zero raw record.
        self.null_record = torch.zeros(RAW_RECORD, dtype=torch.uint8, device=dev)
        self.rec_addr = torch.full(
            (L, NB, 2, H), self.null_record.data_ptr(), dtype=torch.int64, device=dev
        )
        self.rec_len = torch.full((L, NB, 2, H), RAW_VAR_LEN, **i32)
        u8 = dict(dtype=torch.uint8, device=dev)
        self.staging = torch.zeros((staging_slots, L, 2, H, RAW_RECORD), **u8)
        self.scratch = torch.zeros((transient, 2, H, RAW_RECORD), **u8)
        self.overflow = torch.zeros((overflow_records, RAW_RECORD), **u8)
        self.fill = torch.zeros((L, NB), **i32)
        self.live = torch.zeros(NB, **i32)
        i64 = dict(dtype=torch.int64, device=dev)
        self.arena_base_dev = torch.tensor(self.arena_base, **i64)
        self.arena_stride_dev = torch.tensor(self.arena_stride, **i64)
        self._poll_host = torch.zeros(
            _N_COUNTERS, dtype=torch.int32, pin_memory=dev.type == "cuda"
        )
        self._poll_event: torch.cuda.Event | None = None
        self._step = 0
        self._native = FpStore(
            counters=self.counters.data_ptr(),
            wslot=self.wslot.data_ptr(),
            tags=self.tags.data_ptr(),
            free_stack=self.free_stack.data_ptr(),
            ovf_bits=self.ovf_bits.data_ptr(),
            claim_list=self.claim_list.data_ptr(),
            close_list=self.close_list.data_ptr(),
            rec_addr=self.rec_addr.data_ptr(),
            rec_len=self.rec_len.data_ptr(),
            staging=self.staging.data_ptr(),
            scratch=self.scratch.data_ptr(),
            overflow=self.overflow.data_ptr(),
            fill=self.fill.data_ptr(),
            slot_owner=self.slot_owner.data_ptr(),
            seen_list=self.seen_list.data_ptr(),
            overflow_records=overflow_records,
            L=L,
            H=H,
            NB=NB,
            S_p=staging_slots,
            S_t=transient,
            ovf_words=words,
            cap=max_tokens,
        )
        self._store_ref = ctypes.byref(self._native)

    def _require_device(self) -> None:
        if self.counters.device.type != "cuda":
            raise RuntimeError("HbmKvStore kernels need CUDA tensors: there is no CPU fallback")

    def memory_usage(self) -> dict[str, int]:
        """Report persistent GPU tensor bytes by component (``hbm_kv.py:303-342``).

        Returns:
            Byte counts for the arena (real row strides), staging, scratch,
            overflow, metadata and codebooks.
        """
        metadata = (
            self.counters,
            self.wslot,
            self.tags,
            self.free_stack,
            self.ovf_bits,
            self.claim_list,
            self.close_list,
            self.slot_owner,
            self.seen_list,
            self.null_record,
            self.rec_addr,
            self.rec_len,
            self.fill,
            self.live,
            self.arena_base_dev,
            self.arena_stride_dev,
        )
        size = lambda t: t.numel() * t.element_size()  # noqa: E731
        return {
            "arena": self.num_blocks * sum(self.arena_stride),
            "staging": size(self.staging),
            "scratch": size(self.scratch),
            "overflow": size(self.overflow),
            "metadata": sum(size(t) for t in metadata),
            "codebooks": sum(
                size(t) for t in (self.tables.rank_of, self.tables.plut, self.tables.slut)
            ),
        }

    def prepare(self, slot_mapping: torch.Tensor, num_tokens: int, live_blocks: np.ndarray) -> None:
        """Start a step: GC, claim staging, list closing blocks (``hbm_kv.py:344-374``).

        Args:
            slot_mapping: int64 ``[>= num_tokens]`` slot ids (negative = pad).
            num_tokens: Tokens to scan.
            live_blocks: int32 ids of the blocks that keep their staging slot
                (the partially written block of each running request).

        Async/thread-safety:
            One host-to-device copy and one kernel; call once per step before
            the first :meth:`write`, outside CUDA graph capture.
        """
        self._require_device()
        if slot_mapping.dtype != torch.int64:
            raise RuntimeError("slot_mapping must be int64")
        self._step = self._step % 0x7FFFFFFE + 1
        n_live = int(live_blocks.size)
        if n_live:
            host = torch.from_numpy(np.ascontiguousarray(live_blocks, dtype=np.int32)).pin_memory()
            self.live[:n_live].copy_(host, non_blocking=True)
        check(
            extension().fp_hbm_prepare(
                self._store_ref, slot_mapping.data_ptr(), num_tokens, self.live.data_ptr(),
                n_live, self._step, stream_ptr(),
            )
        )

    def write(
        self, layer: int, key: torch.Tensor, value: torch.Tensor, slot_mapping: torch.Tensor
    ) -> None:
        """Store one layer's new K / V tokens into their blocks' staging.

        Args:
            layer: Layer index.
            key: BF16 ``[N, H, 128]`` (rows / heads may be strided).
            value: BF16 ``[N, H, 128]``.
            slot_mapping: int64 ``[N]`` slot ids (negative = skip).

        Async/thread-safety:
            One kernel; CUDA-graph safe.
        """
        self._require_device()
        if key.shape[0] == 0:
            return
        if key.stride(2) != 1 or value.stride(2) != 1:
            raise RuntimeError("head dim must be contiguous")
        check(
            extension().fp_hbm_write(
                self._store_ref, key.data_ptr(), key.stride(0), key.stride(1), value.data_ptr(),
                value.stride(0), value.stride(1), slot_mapping.data_ptr(), key.shape[0], layer,
                stream_ptr(),
            )
        )

    def encode(self, layer: int, max_close: int) -> None:
        """Code this layer's records of every block closed this step.

        Args:
            layer: Layer index.
            max_close: Upper bound on blocks closed this step (grid size).

        Async/thread-safety:
            One kernel; CUDA-graph safe for a fixed ``max_close``.
        """
        self._require_device()
        check(
            extension().fp_hbm_encode(
                self._store_ref, self.tables.rank_of.data_ptr(), layer, self.arena_base[layer],
                self.arena_stride[layer], max_close, stream_ptr(),
            )
        )

    def commit(self) -> None:
        """Release the staging of blocks closed this step (after the last layer)."""
        self._require_device()
        check(extension().fp_hbm_commit(self._store_ref, stream_ptr()))

    def gather(self, layer: int, blocks: torch.Tensor, wk: torch.Tensor, wv: torch.Tensor) -> None:
        """Decode blocks of one layer into token-major BF16 pages.

        Args:
            layer: Layer index.
            blocks: int32 ``[P]`` block ids.
            wk: BF16 ``[>= P, 128, H, 128]`` K pages (page ``i`` = ``blocks[i]``).
            wv: BF16 ``[>= P, 128, H, 128]`` V pages.
        """
        self._require_device()
        if blocks.dtype != torch.int32:
            raise RuntimeError("blocks must be int32")
        size = min(wk.numel() * wk.element_size(), wv.numel() * wv.element_size())
        check(
            extension().fp_hbm_gather(
                blocks.data_ptr(), blocks.numel(), self.rec_addr[layer].data_ptr(),
                self.rec_len[layer].data_ptr(), self.tables.plut[layer].data_ptr(),
                self.tables.slut[layer].data_ptr(), wk.data_ptr(), wv.data_ptr(), size,
                self.kv_heads, stream_ptr(),
            )
        )

    @staticmethod
    def gather_status() -> int:
        """Status word of the decompressor (synchronises): bit 0 = a bounded wait ran out."""
        import ctypes

        word = ctypes.c_int32(0)
        check(extension().fp_hbm_gather_status(ctypes.byref(word)))
        return int(word.value)

    def layer_tables(
        self, layer: int
    ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
        """Return ``(rec_addr, rec_len, plut, slut)`` views of one layer."""
        return (
            self.rec_addr[layer],
            self.rec_len[layer],
            self.tables.plut[layer],
            self.tables.slut[layer],
        )

    @property
    def blob_stride(self) -> int:
        """Bytes reserved per block blob (all records raw)."""
        return ap.blob_slot_bytes(self.num_layers, self.kv_heads)

    def export_blocks(self, blocks: torch.Tensor, out: torch.Tensor, stride: int) -> torch.Tensor:
        """Copy closed blocks' records into block blobs (``hbm_kv.py:486-517``).

        Args:
            blocks: int32 ``[n]`` closed block ids.
            out: Contiguous 16-byte aligned uint8 buffer; blob ``i`` at ``i * stride``.
            stride: Bytes between blobs, at least :attr:`blob_stride`, 16-byte multiple.

        Returns:
            int64 ``[n]`` device tensor of blob lengths (``BLOB_ALIGN`` multiples).
        """
        self._require_device()
        if blocks.dtype != torch.int32:
            raise RuntimeError("export blocks must be int32 and lengths int64 [>= n]")
        if out.dtype != torch.uint8 or not out.is_contiguous():
            raise RuntimeError("export buffer must be contiguous 16-byte aligned uint8")
        lengths = torch.empty(blocks.numel(), dtype=torch.int64, device=out.device)
        # Offset of every record in its blob, written by the layout pass for the copy pass.
        scratch = torch.empty(
            (blocks.numel(), self.num_layers * 2 * self.kv_heads), dtype=torch.int64, device=out.device
        )
        check(
            extension().fp_hbm_export(
                blocks.data_ptr(), blocks.numel(), self.rec_addr.data_ptr(),
                self.rec_len.data_ptr(), out.data_ptr(), out.numel(), stride, lengths.data_ptr(),
                scratch.data_ptr(), self.num_layers, self.kv_heads, self.num_blocks,
                self.table_digest, stream_ptr(),
            )
        )
        return lengths

    def import_blocks(
        self, src: torch.Tensor, offsets: torch.Tensor, blocks: torch.Tensor
    ) -> torch.Tensor:
        """Install block blobs into blocks of this store (``hbm_kv.py:519-557``).

        Args:
            src: Contiguous 16-byte aligned uint8 buffer holding the blobs.
            offsets: int64 ``[n]`` byte offsets of the blobs in ``src``.
            blocks: int32 ``[n]`` distinct destination blocks.

        Returns:
            int32 ``[n]`` device status, zero for an installed block (see
            :func:`blob_failures`).
        """
        self._require_device()
        if src.dtype != torch.uint8 or not src.is_contiguous():
            raise RuntimeError("import buffer must be contiguous 16-byte aligned uint8")
        if (
            offsets.dtype != torch.int64
            or offsets.numel() != blocks.numel()
            or blocks.dtype != torch.int32
        ):
            raise RuntimeError("import metadata must be int64 offsets, int32 blocks / status")
        status = torch.zeros(blocks.numel(), dtype=torch.int32, device=src.device)
        # Source and destination address of every record, from the layout and
        # placement passes to the copy pass.
        scratch = torch.empty(
            (2, blocks.numel(), self.num_layers * 2 * self.kv_heads), dtype=torch.int64, device=src.device
        )
        check(
            extension().fp_hbm_import(
                self._store_ref, src.data_ptr(), src.numel(), offsets.data_ptr(),
                blocks.data_ptr(), blocks.numel(), status.data_ptr(), scratch.data_ptr(),
                self.arena_base_dev.data_ptr(), self.arena_stride_dev.data_ptr(),
                self.table_digest, stream_ptr(),
            )
        )
        return status

    def poll(self) -> StoreStats | None:
        """Asynchronously snapshot the counters; raise if data was dropped.

        Each call reads the snapshot taken by the previous call (if its copy has
        finished) and enqueues a new one, so it never blocks the host.

        Raises:
            StoreError: If staging or the overflow pool was exhausted.
        """
        stats = None
        if self._poll_event is not None:
            if not self._poll_event.query():
                return None
            stats = self._stats_from(self._poll_host.numpy())
        self._poll_host.copy_(self.counters, non_blocking=True)
        self._poll_event = torch.cuda.Event()
        self._poll_event.record()
        return stats

    def stats(self) -> StoreStats:
        """Synchronously read the counters (tests and shutdown).

        Raises:
            StoreError: If staging or the overflow pool was exhausted.
        """
        return self._stats_from(self.counters.cpu().numpy())

    def _stats_from(self, c: np.ndarray) -> StoreStats:
        stats = StoreStats(
            encoded=int(c[_ENCODED]),
            fallbacks=int(c[_FALLBACKS]),
            spills=int(c[_SPILLS]),
            err_staging=int(c[_ERR_STAGING]),
            err_overflow=int(c[_ERR_OVERFLOW]),
        )
        if stats.err_staging or stats.err_overflow:
            raise StoreError(
                f"FragPack store dropped KV: staging={stats.err_staging} "
                f"overflow={stats.err_overflow} "
                "(staging must cover one open block per running request; "
                "overflow is sized by FRAGPACK_OVERFLOW)"
            )
        return stats


__all__ = [
    "BLOCK_TOKENS",
    "HEAD_DIM",
    "RAW_RECORD",
    "VAR_SHARE",
    "HbmKvStore",
    "StoreError",
    "StoreStats",
    "active_store",
    "blob_failures",
    "page_bytes",
    "register_store",
]
