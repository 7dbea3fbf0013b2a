"""Host-side contracts of the vLLM backend mirror (no GPU, no vLLM).

The engine-independent core is tested directly; the vLLM-facing classes are
bound against fake modules injected at the import paths of the vLLM release the
reference pins, and must keep the reference's names, flags and rejections
(``fragpack/integrations/vllm/backend.py:449-641``).
"""

from __future__ import annotations

from dataclasses import dataclass
import sys
from types import ModuleType, SimpleNamespace

import numpy as np
import pytest
import torch

from fragpack_b200.integrations.vllm import backend
from fragpack_b200.ops.hbm_kv import page_bytes


def test_importing_the_backend_does_not_import_vllm() -> None:
    import subprocess

    code = (
        "import sys; import fragpack_b200.integrations.vllm.backend as b; "
        "assert b.PrefillGroup and b.FragPackMetadata and b.run_layer; "
        "assert not any(m == 'vllm' or m.startswith('vllm.') for m in sys.modules)"
    )
    subprocess.run([sys.executable, "-c", code], check=True, cwd=str(__import__("pathlib").Path(__file__).parents[1]))


def test_count_closes_counts_crossed_block_boundaries() -> None:
    # contexts after the step / new tokens this step
    seq = np.array([128, 129, 127, 300, 1])
    qlen = np.array([1, 1, 127, 300, 1])
    # 127->128 closes one; 128->129 none; 0->127 none; 0->300 closes two; 0->1 none
    assert backend.count_closes(seq, qlen) == 3


def test_prefill_groups_pack_rows_into_workspace_passes() -> None:
    table = torch.arange(40, dtype=torch.int32).view(4, 10)
    qsl = np.array([0, 1, 201, 351, 451], np.int64)   # row 0 is a decode
    seq = np.array([500, 200, 150, 612], np.int64)
    groups = backend.plan_prefill_groups(table, 1, 4, qsl, seq, workspace_pages=5, device=torch.device("cpu"))
    # pages per prefill row: 2, 2, 5 -> [rows 1-2] fit 5 pages, row 3 needs its own pass
    assert [(g.tok0, g.tok1) for g in groups] == [(1, 351), (351, 451)]
    g = groups[0]
    assert g.src_blocks.tolist() == [10, 11, 20, 21]
    assert g.block_table.tolist() == [[0, 1], [2, 3]]
    assert g.cu_seqlens_q.tolist() == [0, 200, 350]
    assert g.seqused_k.tolist() == [200, 150]
    assert (g.max_seqlen_q, g.max_seqlen_k) == (200, 200)
    assert groups[1].src_blocks.tolist() == [30, 31, 32, 33, 34]
    assert groups[1].max_seqlen_k == 612


def test_impl_argument_rejections() -> None:
    ok = dict(alibi_slopes=None, sliding_window=None, logits_soft_cap=None, is_decoder=True,
              kv_sharing_target_layer_name=None)
    assert backend.check_impl_arguments(32, 128, 8, **ok) == 8
    assert backend.check_impl_arguments(8, 128, None, **ok) == 8
    for heads, size, kv in ((32, 64, 8), (24, 128, 8), (48, 128, 4), (10, 128, 4)):
        with pytest.raises(ValueError):
            backend.check_impl_arguments(heads, size, kv, **ok)
    for bad in (dict(alibi_slopes=[1.0]), dict(sliding_window=4096), dict(logits_soft_cap=30.0),
                dict(is_decoder=False), dict(kv_sharing_target_layer_name="layers.0")):
        with pytest.raises(ValueError):
            backend.check_impl_arguments(32, 128, 8, **{**ok, **bad})


def test_capability_and_spec() -> None:
    assert backend.supports_compute_capability(SimpleNamespace(major=10, minor=0))
    assert not backend.supports_compute_capability(SimpleNamespace(major=9, minor=0))

    @dataclass(frozen=True)
    class Spec:
        num_kv_heads: int
        num_head_slots: int = 8
        state_content_bytes: int | None = None

    sized = backend.customize_spec(Spec(num_kv_heads=8))
    assert sized.num_head_slots == 1 and sized.state_content_bytes == page_bytes(8) // 128
    kept = Spec(num_kv_heads=8, state_content_bytes=77)
    assert backend.customize_spec(kept) is kept


@pytest.fixture
def fake_vllm(monkeypatch):
    """Fake modules at the import paths the backend binds."""
    def module(name, **attrs):
        mod = ModuleType(name)
        for key, value in attrs.items():
            setattr(mod, key, value)
        monkeypatch.setitem(sys.modules, name, mod)
        return mod

    class Base:
        def __init__(self, *a, **k):
            pass

    module("vllm")
    module("vllm.config", get_layers_from_vllm_config=lambda *a: {})
    module("vllm.distributed", get_tensor_model_parallel_rank=lambda: 0)
    module("vllm.model_executor")
    module("vllm.model_executor.layers")
    module("vllm.model_executor.layers.attention", Attention=object)
    module("vllm.model_executor.models")
    module("vllm.model_executor.models.utils", extract_layer_index=lambda name: int(name.split(".")[-1]))
    module("vllm.v1")
    module("vllm.v1.attention")
    module("vllm.v1.attention.backend", AttentionBackend=Base, AttentionImpl=Base,
           AttentionMetadataBuilder=Base,
           AttentionCGSupport=SimpleNamespace(UNIFORM_SINGLE_TOKEN_DECODE="uniform-single-token"),
           AttentionType=SimpleNamespace(DECODER="decoder", ENCODER="encoder"))
    module("vllm.v1.attention.backends")
    module("vllm.v1.attention.backends.utils", split_decodes_and_prefills=lambda *a, **k: (0, 0, 0, 0))
    module("vllm.v1.kv_cache_interface", KVCacheLayout=SimpleNamespace(LBNHC="LBNHC"))
    monkeypatch.setattr(backend, "_BOUND", {})
    yield
    backend._BOUND.clear()


def test_bound_classes_keep_the_reference_contract(fake_vllm) -> None:
    cls = backend.FragPackAttentionBackend
    assert cls.get_name() == "CUSTOM"
    assert cls.accept_output_buffer and cls.forward_includes_kv_cache_update
    assert cls.supported_dtypes == [torch.bfloat16]
    assert cls.supported_kv_cache_dtypes == ["auto", "bfloat16"]
    assert cls.get_supported_kernel_block_sizes() == [128]
    assert cls.get_supported_head_sizes() == [128]
    assert cls.supported_kv_cache_layouts() == ("LBNHC",)
    assert cls.get_impl_cls() is backend.FragPackAttentionImpl
    assert cls.get_builder_cls() is backend.FragPackMetadataBuilder
    assert backend.FragPackMetadataBuilder._cudagraph_support == "uniform-single-token"

    impl = cls.get_impl_cls()(32, 128, 0.088, num_kv_heads=8)
    assert impl.num_kv_heads == 8 and impl.scale == pytest.approx(0.088)
    with pytest.raises(ValueError):
        cls.get_impl_cls()(32, 128, 0.088, num_kv_heads=8, attn_type="encoder")
    out = torch.ones(3, 32, 128)
    assert impl.forward(None, None, None, None, None, None, out) is out and not out.any()
    with pytest.raises(NotImplementedError):
        impl.forward(None, None, None, None, None, None, out, output_scale=torch.ones(1))
