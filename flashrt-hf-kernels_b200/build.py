#!/usr/bin/env python3
"""Build the native pieces in-tree (sm_100a only).

  lib/libflashrt_b200.so              the C-ABI library (nvcc; no torch types)
  torch-ext/flashrt_b200_core/_C.so   the torch operator library (g++; links the C-ABI library)

`python build.py` builds what is out of date; `python build.py --force` rebuilds.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
CSRC = HERE / "csrc"
LIB = HERE / "lib" / "libflashrt_b200.so"
EXT = HERE / "torch-ext" / "flashrt_b200_core" / "_C.so"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", f"-I{ROOT / 'include'}", f"-I{CSRC}"]


def newer(target: Path, sources) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(s).stat().st_mtime <= t for s in sources)


def run(cmd):
    print("+", " ".join(str(c) for c in cmd), flush=True)
    subprocess.run([str(c) for c in cmd], check=True)


def build_lib(force=False, verbose=False):
    cus = sorted(CSRC.glob("*.cu"))
    deps = cus + sorted(CSRC.glob("*.cuh")) + [ROOT / "include" / "flashrt_b200.h"]
    if not force and newer(LIB, deps):
        return LIB
    LIB.parent.mkdir(parents=True, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objs = []
    procs = []
    for cu in cus:
        obj = LIB.parent / (cu.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-c", cu, "-o", obj]
        print("+", " ".join(str(c) for c in cmd), flush=True)
        procs.append(subprocess.Popen([str(c) for c in cmd]))
        objs.append(obj)
    for pr in procs:
        if pr.wait() != 0:
            raise RuntimeError("nvcc failed")
    run([nvcc, "-shared", "-Wno-deprecated-gpu-targets", "-o", LIB, *objs])
    return LIB


def build_ext(force=False):
    src = HERE / "torch-ext" / "torch_binding.cpp"
    if not src.exists():
        return None
    deps = [src, HERE / "torch-ext" / "registration.h", ROOT / "include" / "flashrt_b200.h", LIB]
    if not force and newer(EXT, deps):
        return EXT
    import torch
    from torch.utils import cpp_extension as ce
    inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{ROOT / 'include'}", f"-I{HERE / 'torch-ext'}",
                                                    "-I/usr/local/cuda/include"]
    import sysconfig
    inc.append(f"-I{sysconfig.get_paths()['include']}")
    torch_lib = Path(torch.__file__).parent / "lib"
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=_C",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", *inc, str(src), "-o", str(EXT),
           f"-L{LIB.parent}", "-lflashrt_b200", f"-Wl,-rpath,$ORIGIN/../../lib",
           f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda",
           ]
    run(cmd)
    return EXT


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="pass -Xptxas -v")
    ap.add_argument("--no-ext", action="store_true")
    a = ap.parse_args()
    print(build_lib(a.force, a.verbose))
    if not a.no_ext:
        print(build_ext(a.force))


if __name__ == "__main__":
    main()
