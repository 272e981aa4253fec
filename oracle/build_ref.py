"""Build the UNMODIFIED reference tile-encoder extension (test infrastructure only).

This compiles the reference's own sources where they lie (``qsrt/csrc/sqg_quantize.cpp`` and
``qsrt/csrc/sqg_quantize.cu`` under the reference checkout) for sm_100a with the reference's
own flags (``qsrt/sqg_quantizer.py:359-380``: ``-O3 --use_fast_math -lineinfo``) and writes
the result to ``oracle/_ref/``.  Nothing is copied into this repository.  The resulting
extension is the GPU-side ground truth used by the ``gpu`` parity tests to pin both the CPU
restatement in ``oracle/viterbi_oracle.c`` and the product kernels; the product never loads it.

Usage:  python oracle/build_ref.py [/path/to/reference]
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

REF_NAME = "qsrt_ref_sqg_ext"


def default_reference_root() -> str:
    """The reference checkout: ``$QSRT_REFERENCE_ROOT`` or the ``reference`` folder beside the repository."""

    return os.environ.get("QSRT_REFERENCE_ROOT", str(Path(__file__).resolve().parents[2] / "reference"))


def build(reference_root: str | None = None, verbose: bool = False) -> Path | None:
    root = Path(reference_root or default_reference_root())
    csrc = root / "qsrt" / "csrc"
    out = Path(__file__).resolve().parent / "_ref"
    if not (csrc / "sqg_quantize.cu").exists():
        return None
    out.mkdir(parents=True, exist_ok=True)
    target = out / f"{REF_NAME}.so"
    newest = max(p.stat().st_mtime for p in csrc.rglob("*") if p.is_file())
    if target.exists() and target.stat().st_mtime >= newest:
        return target
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", "4")
    from torch.utils.cpp_extension import load

    load(
        name=REF_NAME,
        sources=[str(csrc / "sqg_quantize.cpp"), str(csrc / "sqg_quantize.cu")],
        extra_include_paths=[str(csrc)],
        extra_cflags=["-O3"],
        extra_cuda_cflags=[
            "-O3",
            "--use_fast_math",
            "-lineinfo",
            "-gencode",
            "arch=compute_100a,code=sm_100a",
            "-Xcudafe",
            "--diag_suppress=177",
            "-Xcudafe",
            "--diag_suppress=20012",
        ],
        build_directory=str(out),
        is_python_module=False,
        verbose=verbose,
    )
    return target if target.exists() else None


if __name__ == "__main__":
    result = build(*(sys.argv[1:2]), verbose=True)
    print("built:", result)
