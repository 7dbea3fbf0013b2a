"""Compile the CPU oracle (test infrastructure only) into a shared library.

Run as ``python -m oracle.build``.  Tries the system ``gcc`` with OpenMP first
and falls back to a serial build when no OpenMP runtime is installed.
"""

from __future__ import annotations

import os
from pathlib import Path
import shutil
import subprocess

_DIR = Path(__file__).resolve().parent
SOURCE = _DIR / "fragpack_oracle.c"
LIBRARY = _DIR / "libfragpack_oracle.so"


def build(force: bool = False) -> Path:
    """Build ``libfragpack_oracle.so`` next to its source if it is stale.

    Args:
        force: Rebuild even when the library is newer than the source.

    Returns:
        Path of the shared library.

    Raises:
        RuntimeError: If no C compiler could build it.
    """
    if (
        not force
        and LIBRARY.exists()
        and LIBRARY.stat().st_mtime >= SOURCE.stat().st_mtime
    ):
        return LIBRARY
    compilers = [c for c in ("/usr/bin/gcc", shutil.which("gcc"), os.environ.get("CC"), "cc") if c]
    errors = []
    for openmp in (["-fopenmp"], []):
        for cc in compilers:
            cmd = [cc, "-O2", "-fPIC", "-std=c11", *openmp, "-shared", "-o", str(LIBRARY), str(SOURCE)]
            done = subprocess.run(cmd, capture_output=True, text=True)
            if done.returncode == 0:
                return LIBRARY
            errors.append(f"{' '.join(cmd)}: {done.stderr.strip()[:200]}")
    raise RuntimeError("could not build the oracle:\n" + "\n".join(errors))


if __name__ == "__main__":
    print(build(force=True))
