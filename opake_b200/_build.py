"""In-tree build of the native libraries (nvcc for the sm_100a kernels, g++ for the host-only accountant).

The shared objects are written next to the Python package (``opake_b200/_C``) so that they travel with a
snapshot of the source tree; nothing is installed into site-packages and no JIT cache is used.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
OUT = Path(__file__).resolve().parent / "_C"

KERNEL_LIB = OUT / "libopake_kernels.so"
# same sources with -DOPK_DEBUG_BOUNDS: data-dependent indices are checked, a bad one is recorded and its access skipped
KERNEL_LIB_DEBUG = OUT / "libopake_kernels_debug.so"
ACCOUNTING_LIB = OUT / ("_opake_accounting" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-DOPK_SM100A",
]


def _newer(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(s.stat().st_mtime <= t for s in sources)


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found; cannot build the sm_100a kernels")
    return exe


def build_kernels(force: bool = False, verbose: bool = False, debug_bounds: bool = False) -> Path:
    """Compile every ``csrc/kernels/*.cu`` into one shared library for sm_100a (``debug_bounds``: the checked variant)."""
    src_dir = CSRC / "kernels"
    target = KERNEL_LIB_DEBUG if debug_bounds else KERNEL_LIB
    extra = ["-DOPK_DEBUG_BOUNDS"] if debug_bounds else []
    suffix = ".dbg.o" if debug_bounds else ".o"
    cu = sorted(src_dir.glob("*.cu"))
    deps = cu + sorted(src_dir.glob("*.cuh")) + sorted(src_dir.glob("*.h"))
    if not force and _newer(target, deps):
        return target
    OUT.mkdir(parents=True, exist_ok=True)
    objs = []
    jobs = []
    for f in cu:
        obj = OUT / (f.stem + suffix)
        if not force and _newer(obj, [f] + [d for d in deps if d.suffix in (".cuh", ".h")]):
            objs.append(obj)
            continue
        cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-c", str(f), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        jobs.append((f, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for f, proc in jobs:
        out, _ = proc.communicate()
        if verbose and out:
            print(out)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed for {f.name}:\n{out}")
    link = [_nvcc(), "-shared", "-o", str(target), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a",
            "-Xcompiler", "-fPIC"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}")
    return target


def build_accounting(force: bool = False) -> Path:
    """Compile the torch-free C++ privacy accountant (pybind11 module)."""
    src_dir = CSRC / "accounting"
    cpp = sorted(src_dir.glob("*.cpp"))
    if not cpp:
        return ACCOUNTING_LIB
    deps = cpp + sorted(src_dir.glob("*.hpp"))
    if not force and _newer(ACCOUNTING_LIB, deps):
        return ACCOUNTING_LIB
    import pybind11

    OUT.mkdir(parents=True, exist_ok=True)
    cmd = [
        os.environ.get("CXX", "g++"), "-O3", "-std=c++17", "-shared", "-fPIC", "-pthread", "-fvisibility=hidden",
        f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}", f"-I{src_dir}",
        *map(str, cpp), "-o", str(ACCOUNTING_LIB),
    ]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"accountant build failed:\n{r.stdout}")
    return ACCOUNTING_LIB


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_kernels(force=force, verbose=verbose)
    build_kernels(force=force, debug_bounds=True)
    build_accounting(force=force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built:", KERNEL_LIB, ACCOUNTING_LIB if ACCOUNTING_LIB.exists() else "(no accountant sources yet)")
