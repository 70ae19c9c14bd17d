"""Builds the native library in-tree: librecuda_b200/lib/libdriverapi.so.

One shared object holds both layers: the CUDA kernels with their `lcb_*` C-ABI launchers
(csrc/kernels, compiled by nvcc for sm_100a only) and the C++ host layer that implements the
`libreCu*` API on top of them (csrc/driverapi).  The CUDA runtime is linked statically; the CUDA
driver and NCCL are resolved at run time, so the library loads on a machine without a GPU.

Run as `python -m librecuda_b200.build` or call `build()`.
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
OBJ = ROOT / "build" / "obj"
LIB = PKG / "lib" / "libdriverapi.so"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA_HOME / "bin" / "nvcc")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", f"-I{ROOT / 'include'}", f"-I{CSRC / 'kernels'}", f"-I{CSRC / 'driverapi'}"]


def _sources():
    cu = sorted((CSRC / "kernels").glob("*.cu"))
    cpp = sorted((CSRC / "driverapi").glob("*.cpp"))
    return cu, cpp


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(d).stat().st_mtime <= t for d in deps)


def _compile(src: Path, verbose: bool) -> Path:
    obj = OBJ / (src.stem + ".o")
    headers = list((ROOT / "include").glob("*.h")) + list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh"))
    if _newer(obj, [src, *headers]):
        return obj
    cmd = [NVCC, *ARCH, *COMMON, "-Xcompiler", "-fPIC,-Wall,-fvisibility=default", "-c", str(src), "-o", str(obj)]
    if src.suffix == ".cu":
        cmd += ["-Xptxas", "-v"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    (OBJ / (src.stem + ".log")).write_text(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
    if verbose:
        print(f"compiled {src.relative_to(ROOT)}", file=sys.stderr)
    return obj


def build(verbose: bool = False) -> Path:
    """Compile and link libdriverapi.so (incremental).  Returns its path."""
    OBJ.mkdir(parents=True, exist_ok=True)
    LIB.parent.mkdir(parents=True, exist_ok=True)
    cu, cpp = _sources()
    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose), [*cu, *cpp]))
    if not _newer(LIB, objs):
        cmd = [NVCC, *ARCH, "-shared", "-cudart", "static", "-o", str(LIB), *map(str, objs), "-ldl", "-lpthread"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed: {' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
        if verbose:
            print(f"linked {LIB.relative_to(ROOT)}", file=sys.stderr)
    return LIB


if __name__ == "__main__":
    print(build(verbose=True))
