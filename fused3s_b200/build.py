"""In-tree build of the two binaries of this package (no JIT cache, no install step):

* ``libf3s_b200.so``  -- the CUDA kernels and the C ABI (``include/f3s_b200.h``), built with
  nvcc for sm_100a only; depends on nothing but the CUDA runtime.
* ``F3S.<abi>.so``    -- the PyTorch extension module named ``F3S`` (the reference's module
  name, src/setup.py:4-26), a thin binding over the C ABI.

``python -m fused3s_b200.build`` builds both; ``--force`` rebuilds.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
LIB = PKG / "libf3s_b200.so"
CUDA_SOURCES = ["abi.cu", "forward.cu", "backward.cu", "preprocess.cu", "probe.cu", "sddmm_umma.cu"]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    return str(Path(home) / "bin" / "nvcc")


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def ext_path() -> Path:
    return PKG / ("F3S" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_lib(force: bool = False, verbose: bool = False) -> Path:
    deps = [CSRC / s for s in CUDA_SOURCES] + [CSRC / "common.cuh", CSRC / "attn_common.cuh", INCLUDE / "f3s_b200.h"]
    if force or _stale(LIB, deps):
        objs = []
        for s in CUDA_SOURCES:
            obj = CSRC / (Path(s).stem + ".o")
            if force or _stale(obj, [CSRC / s, CSRC / "common.cuh", CSRC / "attn_common.cuh", INCLUDE / "f3s_b200.h"]):
                cmd = [_nvcc(), "-O3", "-std=c++17", *ARCH_FLAGS, "-lineinfo", "-Xcompiler", "-fPIC",
                       "-Xptxas", "-v" if verbose else "-O3", "-c", str(CSRC / s), "-o", str(obj)]
                subprocess.run(cmd, check=True)
            objs.append(str(obj))
        cmd = [_nvcc(), "-shared", *ARCH_FLAGS, "-o", str(LIB), *objs]
        subprocess.run(cmd, check=True)
    return LIB


def build_ext(force: bool = False) -> Path:
    import torch
    from torch.utils import cpp_extension as ce

    out = ext_path()
    src = CSRC / "f3s_torch.cpp"
    if force or _stale(out, [src, INCLUDE / "f3s_b200.h", LIB]):
        inc = []
        for p in ce.include_paths("cuda"):
            inc += ["-isystem", p]
        inc += ["-isystem", sysconfig.get_paths()["include"]]
        libdirs = ce.library_paths("cuda")
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=F3S",
               "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
               *inc, str(src), "-o", str(out),
               *[f"-L{d}" for d in libdirs], f"-L{PKG}",
               "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
               "-lcudart", "-lf3s_b200", "-Wl,-rpath,$ORIGIN"]
        subprocess.run(cmd, check=True)
    return out


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_lib(force, verbose)
    build_ext(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print("built", LIB, ext_path())
