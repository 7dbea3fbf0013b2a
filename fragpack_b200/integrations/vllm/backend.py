"""vLLM attention backend over the compressed HBM KV store (B200).

Mirror of the reference's ``fragpack/integrations/vllm/backend.py``: the same
classes (``FragPackAttentionBackend``, ``FragPackMetadataBuilder``,
``FragPackAttentionImpl``, ``FragPackMetadata``, ``PrefillGroup``), the same
per-step flow and the same rejections.  Per step the builder calls
``HbmKvStore.prepare``; per layer the impl writes the new tokens, attends
(decode rows through the fused kernel, prefill rows over a BF16 workspace the
decompressor fills) and encodes the blocks closed this step; the last layer
commits (``backend.py:504-579``).

Two parts:

* an engine-independent core - :class:`PrefillGroup`, :class:`FragPackMetadata`,
  :func:`plan_prefill_groups`, :func:`count_closes`, :func:`run_layer` - that
  needs only torch and this package, so it is tested here without vLLM;
* the vLLM-facing classes, which subclass vLLM's v1 attention interfaces of the
  release the reference pins (0.30.0).  They are built on first access
  (``backend.FragPackAttentionBackend`` etc.), so importing this module never
  imports vLLM.

Differences from the reference, on purpose: compute capability 10 (B200)
instead of 9; prefill rows are attended directly over the compressed records
by :func:`fragpack_b200.ops.prefill_attn.prefill_attention` (the reference
decompresses into the workspace and calls vLLM's FlashAttention-3, which is
SM90-only; that two-step path is kept as ``run_layer(..., fused_prefill=False)``
with torch SDPA per request in FlashAttention's place); the decode workspace
is sized by this package's ``workspace_elems``.
"""

from __future__ import annotations

from dataclasses import dataclass, replace
import os
from typing import Any, Callable

import numpy as np
import torch

from fragpack_b200.integrations.vllm.lifecycle import OpenBlocks
from fragpack_b200.ops.fused_attn_decode import (
    GQA,
    RecordTables,
    decode_attention,
    decode_units,
    workspace_elems,
)
from fragpack_b200.ops.hbm_kv import BLOCK_TOKENS, HEAD_DIM, HbmKvStore, page_bytes, register_store
from fragpack_b200.ops.prefill_attn import prefill_attention as fused_prefill_attention

_POLL_EVERY = 16
_LOG_EVERY = 4096
# Capacity of the raw-record pool when FRAGPACK_OVERFLOW is unset (backend.py:84-88).
_OVERFLOW_RECORDS = 8192

_TRACKER = OpenBlocks(BLOCK_TOKENS)


@dataclass
class PrefillGroup:
    """Prefill rows attended in one workspace pass (``backend.py:94-117``).

    Attributes:
        src_blocks: int32 ``[P]`` blocks decoded into workspace pages ``0..P``.
        block_table: int32 ``[R, max_pages]`` workspace page ids per row.
        store_block_table: int32 ``[R, max_pages]`` the rows' blocks in the store
            (what the fused prefill kernel walks; the workspace is not used then).
        cu_seqlens_q: int32 ``[R + 1]`` query offsets relative to ``tok0``.
        seqused_k: int32 ``[R]`` context lengths.
        tok0: First token of the group in the batch.
        tok1: One past the last token.
        max_seqlen_q: Longest query of the group.
        max_seqlen_k: Longest context of the group.
    """

    src_blocks: torch.Tensor
    block_table: torch.Tensor
    store_block_table: torch.Tensor
    cu_seqlens_q: torch.Tensor
    seqused_k: torch.Tensor
    tok0: int
    tok1: int
    max_seqlen_q: int
    max_seqlen_k: int


@dataclass
class FragPackMetadata:
    """Per-step metadata shared by every layer (``backend.py:120-156``)."""

    store: HbmKvStore
    layer_tables: list[RecordTables]
    layer_index: dict[str, int]
    last_layer: int
    slot_mapping: torch.Tensor
    num_tokens: int
    num_decodes: int
    decode_block_table: torch.Tensor
    decode_seq_lens: torch.Tensor
    units: int
    decode_workspace: tuple[torch.Tensor, torch.Tensor, torch.Tensor]
    max_close: int
    prefills: list[PrefillGroup]
    wk: torch.Tensor
    wv: torch.Tensor


def count_closes(seq_lens: np.ndarray, query_lens: np.ndarray) -> int:
    """Blocks that receive their last token this step (``backend.py:283-286``).

    One per 128-token boundary a request's context crosses.
    """
    seq = np.asarray(seq_lens, np.int64)
    before = np.maximum(seq - np.asarray(query_lens, np.int64), 0)
    return int(np.sum(seq // BLOCK_TOKENS - before // BLOCK_TOKENS))


def plan_prefill_groups(
    block_table: torch.Tensor,
    first: int,
    num_reqs: int,
    query_start: np.ndarray,
    seq_lens: np.ndarray,
    workspace_pages: int,
    device: torch.device,
) -> list[PrefillGroup]:
    """Split the prefill rows into workspace passes (``backend.py:385-446``).

    Rows ``first..num_reqs`` are taken in order; a group closes when the next
    row's context pages would no longer fit the workspace.  Every group decodes
    its rows' blocks into consecutive workspace pages.

    Args:
        block_table: int32 ``[num_reqs, max_pages]`` device block table.
        first: First prefill row (rows before it are decodes).
        num_reqs: Rows of the batch.
        query_start: int64 ``[num_reqs + 1]`` token offsets of the rows.
        seq_lens: int64 ``[num_reqs]`` context lengths after this step.
        workspace_pages: Pages of the BF16 workspace.
        device: Device of the index tensors.
    """
    pages = -(-np.asarray(seq_lens, np.int64) // BLOCK_TOKENS)
    bounds, start, used = [], first, 0
    for row in range(first, num_reqs):
        if used + pages[row] > workspace_pages and row > start:
            bounds.append((start, row))
            start, used = row, 0
        used += int(pages[row])
    bounds.append((start, num_reqs))

    groups = []
    for r0, r1 in bounds:
        count = pages[r0:r1]
        offsets = np.concatenate(([0], np.cumsum(count)))
        total, width, rows = int(offsets[-1]), int(count.max()), r1 - r0
        # Workspace page p holds page (row_of[p], col_of[p]) of the batch's block table.
        row_of = np.repeat(np.arange(r0, r1), count)
        col_of = np.arange(total) - np.repeat(offsets[:-1], count)
        table = np.zeros((rows, width), np.int64)
        for i in range(rows):
            table[i, : count[i]] = np.arange(offsets[i], offsets[i + 1])
        # One host-to-device copy for all five index arrays.
        packed = np.concatenate(
            (row_of, col_of, table.ravel(), query_start[r0 : r1 + 1] - query_start[r0], seq_lens[r0:r1])
        ).astype(np.int64)
        dev = torch.from_numpy(packed)
        if device.type == "cuda":
            dev = dev.pin_memory().to(device, non_blocking=True)
        a, b = total, 2 * total
        c = b + rows * width
        d = c + rows + 1
        src_blocks = block_table[dev[:a], dev[a:b]].to(torch.int32)
        groups.append(
            PrefillGroup(
                src_blocks=src_blocks,
                block_table=dev[b:c].view(rows, width).to(torch.int32),
                store_block_table=src_blocks[dev[b:c]].view(rows, width).contiguous(),
                cu_seqlens_q=dev[c:d].to(torch.int32),
                seqused_k=dev[d:].to(torch.int32),
                tok0=int(query_start[r0]),
                tok1=int(query_start[r1]),
                max_seqlen_q=int((query_start[r0 + 1 : r1 + 1] - query_start[r0:r1]).max()),
                max_seqlen_k=int(np.asarray(seq_lens[r0:r1]).max()),
            )
        )
    return groups


def workspace_prefill_attention(
    query: torch.Tensor,
    wk: torch.Tensor,
    wv: torch.Tensor,
    group: PrefillGroup,
    scale: float,
    out: torch.Tensor,
) -> None:
    """Causal attention of a prefill group over the decompressed workspace.

    Stands where the reference calls ``flash_attn_varlen_func`` with a paged
    workspace (``backend.py:560-575``): row ``r`` attends its last
    ``q_len`` positions of a context of ``seqused_k[r]`` tokens whose pages are
    ``block_table[r]`` of ``wk`` / ``wv``.  Torch SDPA, one call per row.

    Args:
        query: BF16 ``[tok1 - tok0, Hq, 128]`` queries of the group.
        wk, wv: BF16 ``[W, 128, H, 128]`` workspace.
        group: The group.
        scale: Softmax scale.
        out: BF16 output, same shape as ``query``.
    """
    starts = group.cu_seqlens_q.tolist()
    lengths = group.seqused_k.tolist()
    heads = wk.shape[2]
    q_per_kv = query.shape[1] // heads
    for row, context in enumerate(lengths):
        q0, q1 = starts[row], starts[row + 1]
        if q1 == q0:
            continue
        pages = group.block_table[row, : -(-context // BLOCK_TOKENS)].long()
        keys = wk[pages].reshape(-1, heads, HEAD_DIM)[:context]
        values = wv[pages].reshape(-1, heads, HEAD_DIM)[:context]
        q = query[q0:q1].transpose(0, 1).unsqueeze(0)  # [1, Hq, n, 128]
        k = keys.transpose(0, 1).repeat_interleave(q_per_kv, 0).unsqueeze(0)
        v = values.transpose(0, 1).repeat_interleave(q_per_kv, 0).unsqueeze(0)
        n = q1 - q0
        # Query i is position context - n + i: it sees keys up to and including itself.
        mask = torch.ones(n, context, dtype=torch.bool, device=query.device).tril(context - n)
        res = torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=mask, scale=scale)
        out[q0:q1] = res[0].transpose(0, 1)


def run_layer(
    md: FragPackMetadata,
    layer: int,
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    output: torch.Tensor,
    scale: float,
    prefill_attention: Callable[..., None] = workspace_prefill_attention,
    fused_prefill: bool = True,
) -> torch.Tensor:
    """One layer of a step: write new KV, attend, encode closed blocks (``backend.py:536-579``).

    Args:
        md: Step metadata.
        layer: Layer index.
        query: BF16 ``[T, Hq, 128]``; decode rows first.
        key, value: BF16 ``[T, H, 128]`` new tokens.
        output: BF16 ``[T, Hq, 128]`` output buffer.
        scale: Softmax scale.
        prefill_attention: ``(query, wk, wv, group, scale, out)`` for one prefill group
            over the decompressed workspace (used when ``fused_prefill`` is false).
        fused_prefill: Attend prefill rows directly over the compressed records
            (one tensor-core kernel per group, no workspace) instead of
            decompressing into the workspace first.

    Returns:
        ``output``.

    Async/thread-safety:
        Enqueues on the current stream; decode-only steps are CUDA-graph safe.
    """
    store = md.store
    n = md.num_tokens
    store.write(layer, key[:n], value[:n], md.slot_mapping[:n])
    nd = md.num_decodes
    if nd:
        decode_attention(
            query[:nd], md.layer_tables[layer], md.decode_block_table, md.decode_seq_lens, scale,
            md.units, output[:nd], md.decode_workspace, replan=layer == 0,
        )
    for group in md.prefills:
        if fused_prefill:
            fused_prefill_attention(
                query[group.tok0 : group.tok1], md.layer_tables[layer], group.store_block_table,
                group.cu_seqlens_q, group.seqused_k, scale, output[group.tok0 : group.tok1],
                group.max_seqlen_q,
            )
            continue
        store.gather(layer, group.src_blocks, md.wk, md.wv)
        prefill_attention(query[group.tok0 : group.tok1], md.wk, md.wv, group, scale,
                          output[group.tok0 : group.tok1])
    store.encode(layer, md.max_close)
    if layer == md.last_layer:
        store.commit()
    return output


def check_impl_arguments(
    num_heads: int,
    head_size: int,
    num_kv_heads: int | None,
    alibi_slopes: Any,
    sliding_window: Any,
    logits_soft_cap: Any,
    is_decoder: bool,
    kv_sharing_target_layer_name: Any,
) -> int:
    """The rejections of ``FragPackAttentionImpl.__init__`` (``backend.py:478-497``).

    Returns:
        The KV head count.

    Raises:
        ValueError: For anything but plain causal, unshared decoder
            self-attention with head size 128 and a query group dividing 8.
    """
    num_kv_heads = num_kv_heads or num_heads
    if num_heads % num_kv_heads or GQA % (num_heads // num_kv_heads) or head_size != HEAD_DIM:
        raise ValueError(f"FragPack attention needs a GQA group dividing {GQA} and head size {HEAD_DIM}")
    if alibi_slopes is not None or sliding_window is not None or logits_soft_cap:
        raise ValueError("FragPack attention supports plain causal attention only")
    if not is_decoder or kv_sharing_target_layer_name is not None:
        raise ValueError("FragPack attention supports unshared decoder self-attention only")
    return num_kv_heads


def supports_compute_capability(capability: Any) -> bool:
    """True on compute capability 10.x (the kernels are built for sm_100a only)."""
    return getattr(capability, "major", None) == 10


def customize_spec(spec: Any) -> Any:
    """Size a block as one record page per layer (``backend.py:615-631``).

    Returns ``spec`` with one head slot of ``page_bytes(H) / 128`` bytes per token.
    """
    if spec.state_content_bytes is not None:
        return spec
    return replace(spec, num_head_slots=1,
                   state_content_bytes=page_bytes(spec.num_kv_heads) // BLOCK_TOKENS)


# ---------------------------------------------------------------------------
# vLLM-facing classes, bound on first access.
# ---------------------------------------------------------------------------
_BOUND: dict[str, Any] = {}
_LAZY = ("FragPackAttentionBackend", "FragPackMetadataBuilder", "FragPackAttentionImpl")


def _bind_vllm() -> dict[str, Any]:
    """Import vLLM's v1 attention interfaces and build the three classes."""
    from vllm.config import get_layers_from_vllm_config
    from vllm.distributed import get_tensor_model_parallel_rank
    from vllm.model_executor.layers.attention import Attention
    from vllm.model_executor.models.utils import extract_layer_index
    from vllm.v1.attention.backend import (
        AttentionBackend,
        AttentionCGSupport,
        AttentionImpl,
        AttentionMetadataBuilder,
        AttentionType,
    )
    from vllm.v1.attention.backends.utils import split_decodes_and_prefills
    from vllm.v1.kv_cache_interface import KVCacheLayout

    from fragpack_b200.compression.attn_tables import load_tables
    from fragpack_b200.integrations.vllm.capacity import FragPackCapacity, publish_capacity
    from fragpack_b200.integrations.vllm.compat import install_tracker, require_supported_vllm
    from fragpack_b200.logging import init_logger

    logger = init_logger(__name__)

    class FragPackMetadataBuilder(AttentionMetadataBuilder):
        """Builds :class:`FragPackMetadata`; owns the store and workspaces (``backend.py:159-446``)."""

        _cudagraph_support = AttentionCGSupport.UNIFORM_SINGLE_TOKEN_DECODE

        def __init__(self, kv_cache_spec, layer_names, vllm_config, device) -> None:
            super().__init__(kv_cache_spec, layer_names, vllm_config, device)
            require_supported_vllm(use_v2_model_runner=vllm_config.use_v2_model_runner)
            if vllm_config.speculative_config is not None:
                raise ValueError("FragPack attention does not support speculative decoding")
            if vllm_config.cache_config.block_size != BLOCK_TOKENS:
                raise ValueError(f"FragPack attention needs --block-size {BLOCK_TOKENS}")
            self._init_reorder_batch_threshold(1, supports_spec_as_decode=False)
            install_tracker(_TRACKER, use_v2_model_runner=vllm_config.use_v2_model_runner)

            sched = vllm_config.scheduler_config
            capture = vllm_config.compilation_config.max_cudagraph_capture_size or 0
            self.max_tokens = max(sched.max_num_batched_tokens, capture)
            self.kv_heads = kv_cache_spec.num_kv_heads
            order = sorted(layer_names, key=extract_layer_index)
            self.layer_names = order
            self.layer_index = {name: i for i, name in enumerate(order)}
            self.num_sms = torch.cuda.get_device_properties(device).multi_processor_count
            self.max_reqs = sched.max_num_seqs
            opart, ml, plan = workspace_elems(
                self.kv_heads, decode_units(max(self.max_reqs, capture), self.kv_heads, self.num_sms)
            )
            self.decode_workspace = (
                torch.empty(opart, dtype=torch.float32, device=device),
                torch.empty(ml, dtype=torch.float32, device=device),
                torch.empty(plan, dtype=torch.int32, device=device),
            )
            self.workspace_pages = -(-vllm_config.model_config.max_model_len // BLOCK_TOKENS)
            shape = (self.workspace_pages, BLOCK_TOKENS, self.kv_heads, HEAD_DIM)
            self.wk = torch.empty(shape, dtype=torch.bfloat16, device=device)
            self.wv = torch.empty(shape, dtype=torch.bfloat16, device=device)

            path = os.environ.get("FRAGPACK_TABLES")
            if not path:
                raise ValueError("FRAGPACK_TABLES must point at calibrated FragPack tables (.npz)")
            # Tensor-parallel rank r holds the KV heads [r * H, (r + 1) * H).
            rank = get_tensor_model_parallel_rank()
            heads = slice(rank * self.kv_heads, (rank + 1) * self.kv_heads)
            self.tables = load_tables(path, device, heads)
            if self.tables.plut.shape[2] != self.kv_heads:
                raise ValueError(f"FragPack tables {path} do not cover KV heads {heads.start}..{heads.stop}")
            self.store: HbmKvStore | None = None
            self.store_key: tuple[int, int] | None = None
            self.layer_tables: list[RecordTables] = []
            self.steps = 0

        def build(self, common_prefix_len, common_attn_metadata, fast_build=False) -> FragPackMetadata:
            """Prepare the store for this step and build the metadata (raises ``StoreError`` on data loss)."""
            return self._build(common_attn_metadata, capture=False)

        def build_for_cudagraph_capture(self, common_attn_metadata) -> FragPackMetadata:
            """Capture metadata with the replay's launch shapes; store state is not touched."""
            return self._build(common_attn_metadata, capture=True)

        def _build(self, cam, capture: bool) -> FragPackMetadata:
            store = self._store()
            num_reqs = cam.num_reqs
            nd, npf, _, _ = split_decodes_and_prefills(cam, decode_threshold=1)
            qsl = cam.query_start_loc_cpu.numpy().astype(np.int64)
            seq = cam.seq_lens_cpu_upper_bound.numpy().astype(np.int64)[:num_reqs]
            qlen = qsl[1 : num_reqs + 1] - qsl[:num_reqs]
            num_tokens = min(int(qsl[num_reqs]), cam.slot_mapping.shape[0])
            max_close = min(max(count_closes(seq, qlen), nd), self.max_tokens)
            if not capture:
                store.prepare(cam.slot_mapping, num_tokens, _TRACKER.live_blocks())
                self.steps += 1
                if self.steps % _POLL_EVERY == 0:
                    stats = store.poll()
                    if stats is not None and self.steps % _LOG_EVERY == 0:
                        logger.info("FragPack store: %s", stats)
            prefills: list[PrefillGroup] = []
            if npf and not capture:
                prefills = plan_prefill_groups(cam.block_table_tensor, nd, num_reqs, qsl, seq,
                                               self.workspace_pages, self.device)
            return FragPackMetadata(
                store=store, layer_tables=self.layer_tables, layer_index=self.layer_index,
                last_layer=len(self.layer_names) - 1, slot_mapping=cam.slot_mapping,
                num_tokens=num_tokens, num_decodes=nd, decode_block_table=cam.block_table_tensor[:nd],
                decode_seq_lens=cam.seq_lens[:nd],
                units=decode_units(max(nd, 1), self.kv_heads, self.num_sms),
                decode_workspace=self.decode_workspace, max_close=max_close, prefills=prefills,
                wk=self.wk, wv=self.wv,
            )

        def _store(self) -> HbmKvStore:
            layers = get_layers_from_vllm_config(self.vllm_config, Attention, self.layer_names)
            caches = [layers[name].kv_cache for name in self.layer_names]
            if caches[0].numel() == 0:
                raise RuntimeError("FragPack attention built metadata before the KV cache was bound")
            key = (caches[0].data_ptr(), caches[0].shape[0])
            if self.store is None or key != self.store_key:
                # Every running request keeps at most one block open across steps.
                self.store = HbmKvStore(
                    caches, self.kv_heads, self.tables, self.max_tokens, staging_slots=self.max_reqs,
                    overflow_records=int(os.environ.get("FRAGPACK_OVERFLOW", _OVERFLOW_RECORDS)),
                )
                self.store_key = key
                register_store(self.store)
                self.layer_tables = [RecordTables(*self.store.layer_tables(i)) for i in range(len(caches))]
                memory = self.store.memory_usage()
                memory["prefill_workspace"] = sum(t.numel() * t.element_size() for t in (self.wk, self.wv))
                memory["decode_workspace"] = sum(t.numel() * t.element_size() for t in self.decode_workspace)
                publish_capacity(
                    FragPackCapacity(
                        blocks=self.store.num_blocks, block_tokens=BLOCK_TOKENS,
                        layers=self.store.num_layers, kv_heads=self.kv_heads,
                        page_bytes=self.store.arena_stride[0],
                        raw_page_bytes=2 * self.kv_heads * BLOCK_TOKENS * HEAD_DIM * 2, memory=memory,
                    )
                )
                logger.info(
                    "FragPack store: %d layers x %d blocks, %d B/block-layer (raw %d), %d staging slots, "
                    "%d overflow records",
                    len(caches), self.store.num_blocks, page_bytes(self.kv_heads),
                    2 * self.kv_heads * BLOCK_TOKENS * HEAD_DIM * 2, self.store.staging.shape[0],
                    self.store.overflow.shape[0],
                )
            return self.store

    class FragPackAttentionImpl(AttentionImpl):
        """Decoder self-attention over the compressed HBM store (``backend.py:449-579``)."""

        def __init__(self, num_heads, head_size, scale, num_kv_heads=None, alibi_slopes=None,
                     sliding_window=None, kv_cache_dtype="auto", logits_soft_cap=None,
                     attn_type=AttentionType.DECODER, kv_sharing_target_layer_name=None, **kwargs) -> None:
            self.num_kv_heads = check_impl_arguments(
                num_heads, head_size, num_kv_heads, alibi_slopes, sliding_window, logits_soft_cap,
                attn_type == AttentionType.DECODER, kv_sharing_target_layer_name,
            )
            self.num_heads = num_heads
            self.head_size = head_size
            self.scale = float(scale)
            self.kv_cache_dtype = kv_cache_dtype

        def forward(self, layer, query, key, value, kv_cache, attn_metadata, output,
                    output_scale=None, output_block_scale=None) -> torch.Tensor:
            """Write this layer's new KV, attend, and encode closed blocks; ``kv_cache`` is unused."""
            if output_scale is not None or output_block_scale is not None:
                raise NotImplementedError("FragPack attention does not fuse output quantization")
            if attn_metadata is None:  # profiling run
                return output.zero_()
            index = attn_metadata.layer_index[layer.layer_name]
            return run_layer(attn_metadata, index, query, key, value, output, self.scale)

    class FragPackAttentionBackend(AttentionBackend):
        """Compressed HBM KV cache backend (``--attention-backend CUSTOM``; ``backend.py:582-641``)."""

        accept_output_buffer = True
        forward_includes_kv_cache_update = True
        supported_dtypes = [torch.bfloat16]
        supported_kv_cache_dtypes = ["auto", "bfloat16"]

        @staticmethod
        def get_supported_kernel_block_sizes() -> list[int]:
            return [BLOCK_TOKENS]

        @staticmethod
        def get_name() -> str:
            return "CUSTOM"

        @staticmethod
        def get_impl_cls():
            return FragPackAttentionImpl

        @staticmethod
        def get_builder_cls():
            return FragPackMetadataBuilder

        @classmethod
        def get_supported_head_sizes(cls) -> list[int]:
            return [HEAD_DIM]

        @classmethod
        def customize_spec(cls, spec):
            return customize_spec(spec)

        @classmethod
        def supported_kv_cache_layouts(cls):
            return (KVCacheLayout.LBNHC,)

        @classmethod
        def supports_compute_capability(cls, capability) -> bool:
            return supports_compute_capability(capability)

    return {
        "FragPackAttentionBackend": FragPackAttentionBackend,
        "FragPackMetadataBuilder": FragPackMetadataBuilder,
        "FragPackAttentionImpl": FragPackAttentionImpl,
    }


def __getattr__(name: str) -> Any:
    if name in _LAZY:
        if not _BOUND:
            _BOUND.update(_bind_vllm())
        return _BOUND[name]
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


__all__ = [
    "FragPackAttentionBackend",
    "FragPackAttentionImpl",
    "FragPackMetadata",
    "FragPackMetadataBuilder",
    "PrefillGroup",
    "check_impl_arguments",
    "count_closes",
    "customize_spec",
    "plan_prefill_groups",
    "run_layer",
    "supports_compute_capability",
    "workspace_prefill_attention",
]
