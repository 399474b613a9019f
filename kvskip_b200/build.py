"""In-tree build of the CUDA library and its PyTorch front.

    python -m kvskip_b200.build            # builds what is out of date
    python -m kvskip_b200.build --force

Products (next to this file, git-ignored; in the directory $KVSKIP_BUILD when that variable is set,
the reference's name for its build directory, kernels/kvskip.py:33):
    libkvskip_b200.so   nvcc, sm_100a only, no framework dependency: the C ABI of include/kvskip_b200.h
    _kvskip_ext.so      g++, the pybind11/ATen module over it (links libkvskip_b200.so via $ORIGIN)
"""

import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
ROOT = PKG.parent


def out_dir() -> Path:
    """Where the two shared objects live: $KVSKIP_BUILD if set (created on demand), else the package."""
    d = os.environ.get("KVSKIP_BUILD")
    if not d:
        return PKG
    p = Path(d).expanduser().resolve()
    p.mkdir(parents=True, exist_ok=True)
    return p


LIB = out_dir() / "libkvskip_b200.so"
EXT = out_dir() / "_kvskip_ext.so"

NVCC_FLAGS = ["-O3", "--use_fast_math", "-lineinfo", "-std=c++17",
              "-gencode", "arch=compute_100a,code=sm_100a",
              "-shared", "-Xcompiler", "-fPIC"]


def _newer(target: Path, sources) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in sources)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(map(str, cmd)), flush=True)
    r = subprocess.run(list(map(str, cmd)), capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"build step failed ({r.returncode}): {' '.join(map(str, cmd))}\n{r.stdout}\n{r.stderr}")
    if verbose and (r.stdout or r.stderr):
        print(r.stdout, r.stderr, flush=True)


def build_lib(force=False, verbose=False, ptxas_v=False) -> Path:
    srcs = [CSRC / "kvskip_b200.cu", *CSRC.glob("*.cuh"), ROOT / "include" / "kvskip_b200.h"]
    if force or _newer(LIB, srcs):
        nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
        flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if ptxas_v else [])
        _run([nvcc, *flags, CSRC / "kvskip_b200.cu", "-o", LIB], verbose or ptxas_v)
    return LIB


def build_ext(force=False, verbose=False) -> Path:
    srcs = [CSRC / "torch_binding.cpp", ROOT / "include" / "kvskip_b200.h"]
    if force or _newer(EXT, srcs):
        import torch
        from torch.utils.cpp_extension import include_paths, library_paths
        cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
        inc = include_paths("cuda") + [sysconfig.get_paths()["include"], f"{cuda_home}/include"]
        libdirs = library_paths("cuda") + [f"{cuda_home}/lib64"]
        cxx = "/usr/bin/g++" if Path("/usr/bin/g++").exists() else (shutil.which("g++") or "g++")
        cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-Wno-deprecated-declarations",
               "-DTORCH_EXTENSION_NAME=_kvskip_ext", "-DTORCH_API_INCLUDE_EXTENSION_H",
               f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
               *[f"-I{p}" for p in inc], CSRC / "torch_binding.cpp",
               *[f"-L{p}" for p in libdirs], f"-L{LIB.parent}",
               "-lkvskip_b200", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
               "-Wl,-rpath,$ORIGIN", *[f"-Wl,-rpath,{p}" for p in library_paths("cuda")],
               "-o", EXT]
        _run(cmd, verbose)
    return EXT


def build_all(force=False, verbose=False):
    build_lib(force, verbose)
    build_ext(force, verbose)
    return LIB, EXT


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
    print("built", LIB, EXT)
