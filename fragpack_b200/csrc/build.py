"""Build the C-ABI shared library of the sm_100a kernels with nvcc.

Run as ``python -m fragpack_b200.csrc.build``.  The library is written next to
the Python wrappers (``fragpack_b200/ops/libfragpack_b200.so``) so that it is
found without an install step.
"""

from __future__ import annotations

from pathlib import Path
import shutil
import subprocess
import sys

_DIR = Path(__file__).resolve().parent
SOURCES = ("hbm_kv.cu", "lifecycle.cu", "decode_attn.cu", "blob.cu", "prefill_attn.cu")
HEADERS = ("fp_common.cuh", "fp_pipe.cuh", "fp_store.cuh", "fp_api.h", "../../include/fragpack_b200.h")
LIBRARY = _DIR.parent / "ops" / "libfragpack_b200.so"
NVCC_FLAGS = (
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-O3",
    "-std=c++17",
    "-lineinfo",
    "--use_fast_math",
    "-Xcompiler",
    "-fPIC",
    "-shared",
)


def _stale() -> bool:
    if not LIBRARY.exists():
        return True
    built = LIBRARY.stat().st_mtime
    files = [_DIR / s for s in SOURCES] + [_DIR / h for h in HEADERS] + [Path(__file__)]
    return any(f.exists() and f.stat().st_mtime > built for f in files)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the kernels for sm_100a if the library is missing or stale.

    Args:
        force: Rebuild unconditionally.
        verbose: Pass ``-Xptxas -v`` and echo the compiler output.

    Returns:
        Path of the shared library.

    Raises:
        RuntimeError: If nvcc is missing or the build fails.
    """
    if not force and not _stale():
        return LIBRARY
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        raise RuntimeError("nvcc not found; the kernels cannot be built")
    sources = [str(_DIR / s) for s in SOURCES if (_DIR / s).exists()]
    cmd = [nvcc, *NVCC_FLAGS, *(("-Xptxas", "-v") if verbose else ()), "-o", str(LIBRARY), *sources]
    done = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or done.returncode:
        sys.stderr.write(done.stdout + done.stderr)
    if done.returncode:
        raise RuntimeError(f"nvcc failed ({done.returncode}): {' '.join(cmd)}")
    return LIBRARY


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv))
