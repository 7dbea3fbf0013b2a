"""Release gate and scheduler hook for vLLM's V2 model runner.

Reference: ``fragpack/integrations/vllm/compat.py:20-112``.  The attention
backend is not given the scheduler output, so the worker's
``GPUModelRunner.execute_model`` is wrapped once to feed every real step to the
:class:`~fragpack_b200.integrations.vllm.lifecycle.OpenBlocks` tracker before
the forward runs.  This is a patch of one specific release, hence the exact
version check.  Importing this module imports neither torch nor vLLM.
"""

from __future__ import annotations

import functools
from importlib import metadata
from typing import TYPE_CHECKING, Any

if TYPE_CHECKING:
    from fragpack_b200.integrations.vllm.lifecycle import OpenBlocks

SUPPORTED_VLLM_VERSION = "0.30.0+cu129"
_installed_tracker: "OpenBlocks | None" = None


def require_supported_vllm(*, use_v2_model_runner: bool | None = None) -> str:
    """Reject an unsupported vLLM distribution or a non-V2 runner.

    Args:
        use_v2_model_runner: Resolved runner choice when known; ``None`` checks
            the distribution only (plugin discovery).

    Returns:
        The supported version string.

    Raises:
        RuntimeError: vLLM absent or another version.
        ValueError: The runner choice is not V2.
    """
    try:
        installed = metadata.version("vllm")
    except metadata.PackageNotFoundError as exc:
        raise RuntimeError(
            f"FragPack requires vllm=={SUPPORTED_VLLM_VERSION}; vLLM is not installed"
        ) from exc
    if installed != SUPPORTED_VLLM_VERSION:
        raise RuntimeError(
            f"FragPack requires vllm=={SUPPORTED_VLLM_VERSION}; found {installed}. "
            "Its V2 lifecycle adapter is release-specific."
        )
    if use_v2_model_runner is not None and not use_v2_model_runner:
        raise ValueError("FragPack attention needs the V2 model runner")
    return installed


def install_tracker(tracker: "OpenBlocks", *, use_v2_model_runner: bool) -> None:
    """Wrap ``GPUModelRunner.execute_model`` once so that ``tracker`` sees every real step.

    Installing the same tracker again is a no-op; a different tracker is an
    error (the backend would otherwise read a stale one).  Dummy runs
    (``dummy_run=True``) are not tracked.

    Raises:
        RuntimeError: Unsupported distribution, or another tracker is installed.
        ValueError: The runner is not V2.
    """
    global _installed_tracker
    require_supported_vllm(use_v2_model_runner=use_v2_model_runner)
    if _installed_tracker is tracker:
        return
    if _installed_tracker is not None:
        raise RuntimeError("FragPack V2 lifecycle adapter already has a tracker")

    from vllm.v1.worker.gpu.model_runner import GPUModelRunner

    inner = GPUModelRunner.execute_model

    @functools.wraps(inner)
    def execute_model(self: Any, scheduler_output: Any, *args: Any, **kwargs: Any) -> Any:
        if not kwargs.get("dummy_run", False):
            tracker.update(scheduler_output)
        return inner(self, scheduler_output, *args, **kwargs)

    GPUModelRunner.execute_model = execute_model
    _installed_tracker = tracker
