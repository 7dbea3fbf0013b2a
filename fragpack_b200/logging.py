"""Logger helper (reference: ``fragpack/logging.py:15-51``).

``FRAGPACK_LOG_LEVEL`` selects the level of the ``fragpack_b200`` logger tree.
"""

from __future__ import annotations

import logging
import os

_ROOT = "fragpack_b200"
_configured = False


def init_logger(name: str) -> logging.Logger:
    """Return a logger under the package root, configuring the root once.

    Args:
        name: Usually ``__name__``.

    Returns:
        The logger.
    """
    global _configured
    if not _configured:
        root = logging.getLogger(_ROOT)
        level = os.environ.get("FRAGPACK_LOG_LEVEL", "").upper()
        if level:
            root.setLevel(getattr(logging, level, logging.INFO))
        if not root.handlers:
            handler = logging.StreamHandler()
            handler.setFormatter(
                logging.Formatter("%(levelname)s %(asctime)s [%(name)s] %(message)s")
            )
            root.addHandler(handler)
            root.propagate = False
        _configured = True
    if not name.startswith(_ROOT):
        name = f"{_ROOT}.{name}"
    return logging.getLogger(name)


__all__ = ["init_logger"]
