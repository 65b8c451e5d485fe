"""TEST INFRASTRUCTURE -- recipe that compiles the UNMODIFIED reference extension for sm_100a.

Reads the reference's three compiled sources where they lie (``src/F3S.cpp``,
``src/F3S_kernel.cu``, ``src/utils.cu`` of the reference checkout named by the environment
variable ``F3S_REFERENCE_DIR``, or the default location below) and writes only into
``oracle/_ref/`` (git-ignored):

* ``F3S_ref.<abi>.so``      -- the reference as it is, module name ``F3S_ref``; flags are the
  reference's own (src/setup.py:12-21) plus ``-gencode arch=compute_100a,code=sm_100a``.
* ``F3S_ref_rowfix.<abi>.so`` -- the same with ONE token of ``fill_edgeToRow`` changed
  (src/utils.cu:348, stride ``gridDim.x`` -> ``blockDim.x``) so that every edge gets its
  row.  The patched copy of utils.cu lives in a temporary directory, never in this tree.

Nothing is copied into the repository.  The built modules are checkers: the GPU tests
compare this package's TC-block arrays and attention output with theirs, and
tests/golden/make_golden_gpu.py dumps their outputs as golden fixtures.

The reference's own build system (setup.py) is not run; this script issues the nvcc / g++
commands itself.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
import tempfile
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
# the reference checkout: F3S_REFERENCE_DIR, else a directory named "reference" beside this repository
REF = Path(os.environ.get("F3S_REFERENCE_DIR", HERE.parent.parent / "reference")) / "src"
NVCC = str(Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "bin" / "nvcc")
REF_NVCC_FLAGS = ["-O3", "-use_fast_math", "-ftz=true", "-prec-div=false", "-prec-sqrt=false", "-lineinfo"]


def _common_flags(name: str):
    import torch
    from torch.utils import cpp_extension as ce

    inc = []
    for p in ce.include_paths("cuda"):
        inc += ["-isystem", p]
    inc += ["-isystem", sysconfig.get_paths()["include"], "-I", str(REF)]
    defs = [f"-DTORCH_EXTENSION_NAME={name}", "-DTORCH_API_INCLUDE_EXTENSION_H",
            f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    return inc, defs, ce.library_paths("cuda")


def _compile(src: Path, obj: Path, name: str):
    inc, defs, _ = _common_flags(name)
    if src.suffix == ".cu":
        cmd = [NVCC, "-std=c++17", *REF_NVCC_FLAGS, "-gencode", "arch=compute_100a,code=sm_100a",
               "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__",
               "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "--expt-relaxed-constexpr",
               "-Xcompiler", "-fPIC", *defs, *inc, "-c", str(src), "-o", str(obj)]
    else:
        cmd = ["g++", "-O3", "-std=c++17", "-fPIC", *defs, *inc, "-c", str(src), "-o", str(obj)]
    subprocess.run(cmd, check=True)
    return obj


def _link(objs, name: str) -> Path:
    _, _, libdirs = _common_flags(name)
    out = OUT / (name + sysconfig.get_config_var("EXT_SUFFIX"))
    cmd = ["g++", "-shared", "-o", str(out), *map(str, objs), *[f"-L{d}" for d in libdirs],
           "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    subprocess.run(cmd, check=True)
    return out


def build(force: bool = False) -> list[Path]:
    """Build both modules if the reference sources are present; return what exists."""
    suffix = sysconfig.get_config_var("EXT_SUFFIX")
    targets = [OUT / ("F3S_ref" + suffix), OUT / ("F3S_ref_rowfix" + suffix)]
    if not REF.exists():
        return [t for t in targets if t.exists()]
    if not force and all(t.exists() for t in targets):
        return targets
    OUT.mkdir(exist_ok=True)
    with tempfile.TemporaryDirectory(prefix="f3s_ref_build_") as tmp:
        tmp = Path(tmp)
        text = (REF / "utils.cu").read_text()
        needle = "eid < nodePointer[nid + 1]; eid += gridDim.x"
        assert text.count(needle) == 1, "fill_edgeToRow loop not found where expected"
        (tmp / "utils_rowfix.cu").write_text(text.replace(needle, "eid < nodePointer[nid + 1]; eid += blockDim.x"))
        jobs = []
        with ThreadPoolExecutor(max_workers=4) as ex:
            for name in ("F3S_ref", "F3S_ref_rowfix"):
                # the module name is baked into F3S.cpp through TORCH_EXTENSION_NAME
                jobs.append(ex.submit(_compile, REF / "F3S.cpp", tmp / f"{name}_F3S.o", name))
            jobs.append(ex.submit(_compile, REF / "F3S_kernel.cu", tmp / "F3S_kernel.o", "F3S_ref"))
            jobs.append(ex.submit(_compile, REF / "utils.cu", tmp / "utils.o", "F3S_ref"))
            jobs.append(ex.submit(_compile, tmp / "utils_rowfix.cu", tmp / "utils_rowfix.o", "F3S_ref"))
            for j in jobs:
                j.result()
        _link([tmp / "F3S_ref_F3S.o", tmp / "F3S_kernel.o", tmp / "utils.o"], "F3S_ref")
        _link([tmp / "F3S_ref_rowfix_F3S.o", tmp / "F3S_kernel.o", tmp / "utils_rowfix.o"], "F3S_ref_rowfix")
    return targets


def load(name: str = "F3S_ref"):
    """Import a built reference module (None if it has not been built)."""
    import importlib.util

    import torch  # noqa: F401  (the module links against torch)

    path = OUT / (name + sysconfig.get_config_var("EXT_SUFFIX"))
    if not path.exists():
        return None
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
