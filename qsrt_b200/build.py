"""Build ``libqsrt_b200.so`` (hand-written sm_100a kernels + C ABI) in-tree with nvcc."""

from __future__ import annotations

import subprocess
import sys
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
CSRC = PACKAGE / "csrc"
LIBRARY = PACKAGE / "libqsrt_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-diag-suppress", "177",
]


def cutlass_include() -> Path | None:
    """CUTLASS / CuTe header tree used by the tcgen05 kernels (vendored inside site-packages)."""

    import importlib.util

    for package, relative in (("flashinfer", "data/cutlass/include"), ("tilelang", "3rdparty/cutlass/include")):
        spec = importlib.util.find_spec(package)
        if spec is None or not spec.submodule_search_locations:
            continue
        candidate = Path(list(spec.submodule_search_locations)[0]) / relative
        if (candidate / "cute" / "arch" / "mma_sm100_umma.hpp").exists():
            return candidate
    return None


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def needs_build() -> bool:
    if not LIBRARY.exists():
        return True
    built = LIBRARY.stat().st_mtime
    inputs = list(CSRC.glob("*")) + [PACKAGE.parent / "include" / "qsrt_b200.h"]
    return any(p.stat().st_mtime > built for p in inputs if p.is_file())


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` for sm_100a and link the shared library."""

    if not force and not needs_build():
        return LIBRARY
    objects = []
    build_dir = PACKAGE / "build"
    build_dir.mkdir(exist_ok=True)
    procs = []
    cutlass = cutlass_include()
    extra = ["-I", str(cutlass)] if cutlass is not None else ["-DQSRTB_NO_CUTLASS"]
    for src in sources():
        obj = build_dir / (src.stem + ".o")
        objects.append(obj)
        cmd = ["nvcc", *NVCC_FLAGS, "-I", str(PACKAGE.parent / "include"), "-c", str(src), "-o", str(obj)]
        if src.name.endswith("_tc.cu"):
            cmd[1:1] = extra
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, proc in procs:
        out, _ = proc.communicate()
        if verbose or proc.returncode:
            sys.stderr.write(out)
        if proc.returncode:
            raise RuntimeError(f"nvcc failed on {src.name}")
    link = ["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIBRARY),
            *map(str, objects), "-lcudart"]
    subprocess.run(link, check=True)
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
