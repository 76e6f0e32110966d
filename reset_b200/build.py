"""In-tree build of the native libraries.

``libnvfp4r_b200.so``  the CUDA kernels behind the C ABI of ``include/nvfp4r_b200.h``
                       (nvcc, sm_100a only, no PyTorch dependency).
``_C*.so``             the PyTorch extension that registers ``torch.ops.nvfp4r.*`` and
                       forwards to the C ABI (host C++ only).

Both are written next to this file so that they travel with the source tree.
``python -m reset_b200.build`` builds what is out of date; ``--force`` rebuilds.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
LIB_NAME = "libnvfp4r_b200.so"
EXT_NAME = "_C" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so")

CUDA_SOURCES = ["api.cu", "quant.cu", "gemv.cu", "gemv_rows.cu", "reset_step.cu", "gemm_tcgen05.cu", "linear_packed.cu",
                "no_alloc.cu", "decode_ops.cu", "peer_allreduce.cu", "lm_head_reset.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: set NVCC or put it on PATH")


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print("+", " ".join(str(c) for c in cmd), flush=True)
    res = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"build step failed ({res.returncode}):\n{' '.join(map(str, cmd))}\n"
                           f"{res.stdout}\n{res.stderr}")
    return res


def build_cuda_library(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """nvcc -> libnvfp4r_b200.so (one object per .cu so unchanged files are reused)."""
    out = PKG / LIB_NAME
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    sources = [CSRC / s for s in CUDA_SOURCES if (CSRC / s).exists()]
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)
    objs = []
    for src in sources:
        obj = objdir / (src.stem + ".o")
        if force or _stale(obj, [src, *headers]):
            cmd = [_nvcc(), *NVCC_FLAGS, "-I", INCLUDE, "-c", src, "-o", obj]
            if ptxas_info:
                cmd += ["-Xptxas", "-v"]
            res = _run(cmd, verbose)
            if ptxas_info:
                print(res.stderr)
        objs.append(obj)
    if force or _stale(out, objs):
        _run([_nvcc(), "-shared", "-o", out, *objs, "-lcudart_static"], verbose)
    return out


def build_torch_extension(force: bool = False, verbose: bool = False) -> Path:
    """g++ -> _C.so linking libtorch and libnvfp4r_b200.so (found via $ORIGIN)."""
    import torch
    from torch.utils import cpp_extension as ce

    out = PKG / EXT_NAME
    src = CSRC / "torch_bindings.cpp"
    if not (force or _stale(out, [src, INCLUDE / "nvfp4r_b200.h", PKG / LIB_NAME])):
        return out
    inc = [f"-I{p}" for p in ce.include_paths("cuda")] + [f"-I{INCLUDE}",
                                                          f"-I{sysconfig.get_paths()['include']}"]
    torch_lib = Path(torch.__file__).parent / "lib"
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           "-DTORCH_EXTENSION_NAME=_C", *inc, str(src), "-o", str(out),
           f"-L{PKG}", "-l:" + LIB_NAME, f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-lc10",
           "-lc10_cuda", "-ltorch_cuda", "-ltorch_python",
           "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    cuda_home = Path(_nvcc()).parent.parent
    cmd += [f"-L{cuda_home / 'lib64'}", "-lcudart"]
    _run(cmd, verbose)
    return out


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_cuda_library(force=force, verbose=verbose)
    if (CSRC / "torch_bindings.cpp").exists():
        build_torch_extension(force=force, verbose=verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
    print("built:", PKG / LIB_NAME)
