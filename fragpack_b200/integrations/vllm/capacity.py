"""Host-only allocation snapshot of one worker's store.

Reference: ``fragpack/integrations/vllm/capacity.py:12-77``.
"""

from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any

_CAPACITY: "FragPackCapacity | None" = None


@dataclass(frozen=True)
class FragPackCapacity:
    """Allocated capacity of a worker's attention store.

    Attributes:
        blocks: Allocated blocks, including the engine's reserved null block.
        block_tokens: Token slots per block.
        layers: Attention layers on this worker.
        kv_heads: KV heads per layer on this worker.
        page_bytes: Allocated bytes per block-layer.
        raw_page_bytes: BF16 bytes of the same block-layer.
        memory: Persistent tensor bytes by component (``HbmKvStore.memory_usage``).
    """

    blocks: int
    block_tokens: int
    layers: int
    kv_heads: int
    page_bytes: int
    raw_page_bytes: int
    memory: dict[str, int]

    def to_dict(self) -> dict[str, Any]:
        """Independent, serialisable copy."""
        return asdict(self)


def publish_capacity(capacity: FragPackCapacity) -> None:
    """Publish the snapshot after a store is created or rebound."""
    global _CAPACITY
    _CAPACITY = capacity


def get_capacity() -> "FragPackCapacity | None":
    """The published snapshot, or ``None`` before the store exists."""
    return _CAPACITY
