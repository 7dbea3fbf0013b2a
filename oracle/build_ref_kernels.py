"""TEST INFRASTRUCTURE - builds the reference's own CUDA extension for sm_100a.

The reference ships its decode-attention and store kernels as three source
files (``fragpack/ops/fragpack_ext.cpp``, ``fused_attn_decode.cu``,
``hbm_kv.cu``) that it JIT-compiles with ``torch.utils.cpp_extension.load``
(``fragpack/ops/fragpack_ext.py:14-32``).  This recipe compiles those files
where they lie in a reference checkout, unmodified, with the same flags plus
the sm_100a target, and writes only into ``oracle/_ref/fragpack_cuda/``.  No
reference source is copied.

The result is the same-GPU comparison arm of ``bench.py`` (``--impl
reference-gpu``): the reference's kernels reading the very records this
library wrote.  Nothing in the product imports it.

    python -m oracle.build_ref_kernels [/path/to/reference]
"""

from __future__ import annotations

import importlib.util
import os
from pathlib import Path
import sys

OUT = Path(__file__).resolve().parent / "_ref" / "fragpack_cuda"
NAME = "fragpack_cuda"
SOURCES = ("fragpack_ext.cpp", "fused_attn_decode.cu", "hbm_kv.cu")


def reference_root() -> Path:
    """The reference checkout: ``$FRAGPACK_REFERENCE``, else ``reference`` beside this repository."""
    env = os.environ.get("FRAGPACK_REFERENCE")
    return Path(env) if env else Path(__file__).resolve().parents[2] / "reference"


def built() -> Path | None:
    """Path of the built module, or None."""
    hits = sorted(OUT.glob(f"{NAME}*.so"))
    return hits[0] if hits else None


def build(reference: str | None = None) -> Path | None:
    """Compile the reference extension if a checkout is present.

    Returns:
        The shared object, or None when there is neither a checkout nor an
        earlier build.
    """
    ops = (Path(reference) if reference else reference_root()) / "fragpack" / "ops"
    if not all((ops / s).exists() for s in SOURCES):
        return built()
    newest = max((ops / s).stat().st_mtime for s in (*SOURCES, "fragpack_common.cuh"))
    have = built()
    if have is not None and have.stat().st_mtime >= newest:
        return have
    from torch.utils.cpp_extension import load

    OUT.mkdir(parents=True, exist_ok=True)
    # The arch comes from the -gencode flag below; this only stops torch from
    # probing for a GPU (there is none where this runs).
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    load(
        name=NAME,
        sources=[str(ops / s) for s in SOURCES],
        extra_include_paths=[str(ops)],
        extra_cuda_cflags=["-O3", "--use_fast_math", "-lineinfo",
                           "-gencode", "arch=compute_100a,code=sm_100a"],
        build_directory=str(OUT),
        is_python_module=False,
        verbose=False,
    )
    return built()


def module():
    """Import the built extension (the reference's ``fragpack_cuda`` module)."""
    so = built()
    if so is None:
        raise RuntimeError("the reference CUDA extension has not been built (oracle/build_ref_kernels.py)")
    import torch  # noqa: F401  (the extension links against libtorch)

    spec = importlib.util.spec_from_file_location(NAME, so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else None))
