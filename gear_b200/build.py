"""Build libgear_b200.so in-tree with nvcc for sm_100a.

    python -m gear_b200.build [--force] [--verbose]

The library links the CUDA runtime statically and has no other dependency
(NCCL is resolved at run time from the process, see csrc/comm.cc), so the built
file can be loaded from Python (ctypes), C or C++ alike.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB = PKG / "lib" / "libgear_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--fmad=true",
]


def sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cc")))


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found: libgear_b200.so cannot be built on this machine")
    return exe


def nccl_include() -> list[str]:
    """Directory of nccl.h (types only; the functions are looked up at run time)."""
    cands = [Path("/usr/include/nccl.h")]
    try:
        import importlib.util
        spec = importlib.util.find_spec("nvidia.nccl")
        if spec and spec.submodule_search_locations:
            cands.append(Path(list(spec.submodule_search_locations)[0]) / "include" / "nccl.h")
    except Exception:
        pass
    for c in cands:
        if c.exists():
            return ["-I", str(c.parent)]
    raise RuntimeError("nccl.h not found (needed for its type definitions)")


def needs_build() -> bool:
    if not LIB.exists():
        return True
    deps = sources() + list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + [ROOT / "include" / "gear_b200.h"]
    return any(d.stat().st_mtime > LIB.stat().st_mtime for d in deps)


def build(force: bool = False, verbose: bool = False, defines: list[str] | None = None,
          out: Path | None = None) -> Path:
    """Build the library; `defines` (-D flags) and `out` make tuning variants beside the default."""
    global LIB
    variant = bool(defines or out)
    lib_path = Path(out) if out else LIB
    if not force and not variant and not needs_build():
        return LIB
    LIB_default, LIB = LIB, lib_path
    try:
        return _build(verbose, defines or [])
    finally:
        LIB = LIB_default


def _build(verbose: bool, defines: list[str]) -> Path:
    LIB.parent.mkdir(parents=True, exist_ok=True)
    objdir = LIB.parent / ("obj_" + LIB.stem if defines else "obj")
    objdir.mkdir(exist_ok=True)
    nvcc = _nvcc()
    objs = []
    procs = []
    for src in sources():
        obj = objdir / (src.stem + ".o")
        objs.append(obj)
        cmd = [nvcc, *NVCC_FLAGS, *[f"-D{d}" for d in defines], "-I", str(ROOT / "include"), "-I", str(CSRC),
               *nccl_include(),
               "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        if src.suffix == ".cc":
            cmd[1:1] = ["-x", "cu"]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- {src.name}\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed; see output above")
    link = [nvcc, "-shared", "-o", str(LIB), *map(str, objs), "-cudart", "static", "-ldl", "-lpthread",
            "-gencode", "arch=compute_100a,code=sm_100a"]
    subprocess.check_call(link)
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
