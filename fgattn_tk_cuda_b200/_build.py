"""In-tree build of the native pieces: the C-ABI CUDA library and the torch operator extension."""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libfgattn_b200.so"
EXT = PKG / "spattn" / "cuda_attn.so"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17", "--shared",
              "-Xcompiler", "-fPIC"]


def _newer(target: Path, sources) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(s).stat().st_mtime <= t for s in sources)


def _nvcc() -> str:
    cand = os.environ.get("CUDA_HOME", "/usr/local/cuda") + "/bin/nvcc"
    return cand if os.path.exists(cand) else "nvcc"


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """nvcc-compile csrc/fgattn_capi.cu (which includes every kernel header) for sm_100a."""
    sources = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + \
        [PKG.parent / "include" / "fgattn_b200.h"]
    if not force and _newer(LIB, sources):
        return LIB
    cmd = [_nvcc(), *NVCC_FLAGS, "-o", str(LIB), str(CSRC / "fgattn_capi.cu")]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    subprocess.run(cmd, check=True)
    return LIB


def build_extension(force: bool = False) -> Path:
    """g++-compile csrc/extension.cpp (torch operator registrations + pybind module) against the
    C ABI; it contains no device code."""
    import torch
    from torch.utils import cpp_extension as ce

    src = CSRC / "extension.cpp"
    if not force and _newer(EXT, [src, PKG.parent / "include" / "fgattn_b200.h"]):
        return EXT
    build_library()
    inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{PKG.parent / 'include'}"]
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc.append(f"-I{cuda_home}/include")
    import sysconfig
    inc.append(f"-I{sysconfig.get_paths()['include']}")
    torch_lib = Path(torch.__file__).parent / "lib"
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-DTORCH_EXTENSION_NAME=cuda_attn",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           *inc, str(src), "-o", str(EXT), f"-L{torch_lib}", f"-L{PKG}", "-lfgattn_b200", "-lc10", "-lc10_cuda",
           "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
           f"-Wl,-rpath,{torch_lib}", "-Wl,-rpath,$ORIGIN/..", "-Wl,-rpath,$ORIGIN"]
    subprocess.run(cmd, check=True)
    return EXT


if __name__ == "__main__":
    build_library(force="--force" in sys.argv, verbose="-v" in sys.argv)
    if "--ext" in sys.argv:
        build_extension(force="--force" in sys.argv)
