"""``vllm.general_plugins`` entry point (reference: ``fragpack/integrations/vllm/plugin.py:9-31``).

Registers the backend class path for ``AttentionBackendEnum.CUSTOM`` lazily:
nothing of the kernels, torch or CUDA is imported here.
"""

from __future__ import annotations

from fragpack_b200.integrations.vllm.compat import require_supported_vllm

BACKEND_PATH = "fragpack_b200.integrations.vllm.backend.FragPackAttentionBackend"


def register() -> None:
    """Validate the installed vLLM release and register the CUSTOM backend by path.

    Raises:
        RuntimeError: If the installed vLLM distribution is unsupported.
    """
    require_supported_vllm()
    from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend

    register_backend(AttentionBackendEnum.CUSTOM, BACKEND_PATH)
