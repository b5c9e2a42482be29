"""In-tree build of the CUDA library (`libhfuse_b200.so`) for sm_100a.

`python -m hfuse_b200.build` compiles every `.cu` under `csrc/` with nvcc
(cross-compiling works without a GPU) and links one shared library beside
this file.  Objects are cached under `csrc/_obj/` and rebuilt when a source
or any header is newer.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "_obj")
LIB = os.path.join(HERE, "libhfuse_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; the CUDA library cannot be built")


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers_mtime() -> float:
    m = 0.0
    for root in (CSRC, os.path.join(HERE, "..", "include")):
        for f in os.listdir(root):
            if f.endswith((".cuh", ".h", ".inc")):
                m = max(m, os.path.getmtime(os.path.join(root, f)))
    return m


def _compile(src: str, verbose: bool) -> str:
    obj = os.path.join(OBJ, src[:-3] + ".o")
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
    if verbose:
        sys.stderr.write(r.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    hdr = _headers_mtime()
    todo, objs = [], []
    for src in _sources():
        obj = os.path.join(OBJ, src[:-3] + ".o")
        objs.append(obj)
        newest = max(hdr, os.path.getmtime(os.path.join(CSRC, src)))
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < newest:
            todo.append(src)
    if todo:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
            list(ex.map(lambda s: _compile(s, verbose), todo))
    if todo or not os.path.exists(LIB):
        cmd = [_nvcc(), "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
               "-Xcompiler", "-fPIC", "-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


TORCH_EXT = os.path.join(HERE, "_torch_ext.so")


def build_torch_ext(force: bool = False) -> str:
    """The PyTorch extension (torch.ops.hfuse_b200.*): one host-only C++ file compiled with g++
    against the installed torch headers and linked to libhfuse_b200.so beside it."""
    import torch
    from torch.utils import cpp_extension as ce
    src = os.path.join(CSRC, "torch_ext.cpp")
    hdr = os.path.join(HERE, "..", "include", "hfuse_b200.h")
    if not force and os.path.exists(TORCH_EXT) and os.path.getmtime(TORCH_EXT) >= max(
            os.path.getmtime(src), os.path.getmtime(hdr)):
        return TORCH_EXT
    build()
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_inc = os.path.join(os.path.dirname(os.path.dirname(_nvcc())), "include")
    cmd = ["/usr/bin/g++", "-O2", "-std=c++17", "-fPIC", "-shared", src, "-o", TORCH_EXT,
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", "-DTORCH_EXTENSION_NAME=_torch_ext",
           *[f"-I{p}" for p in ce.include_paths()], f"-I{cuda_inc}",
           f"-L{tlib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
           f"-L{HERE}", "-lhfuse_b200", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{tlib}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"torch extension build failed:\n{r.stdout}\n{r.stderr[-4000:]}")
    return TORCH_EXT


FUSER = os.path.join(HERE, "fuser")


def build_fuser(force: bool = False) -> str:
    """The C++ host program over the C ABI (csrc/fuser_main.cpp), the counterpart of the
    reference's `fuser` binary.  Host-only code: g++ plus the CUDA runtime."""
    src = os.path.join(CSRC, "fuser_main.cpp")
    if not force and os.path.exists(FUSER) and os.path.getmtime(FUSER) >= os.path.getmtime(src):
        return FUSER
    build()
    cuda = os.path.dirname(os.path.dirname(_nvcc()))
    cmd = ["/usr/bin/g++", "-O2", "-std=c++17", src, "-o", FUSER, f"-I{cuda}/include", f"-L{HERE}", "-lhfuse_b200",
           f"-L{cuda}/lib64", "-lcudart", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{cuda}/lib64"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"fuser build failed:\n{r.stdout}\n{r.stderr[-4000:]}")
    return FUSER


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--torch-ext" in sys.argv:
        print(build_torch_ext(force="--force" in sys.argv))
    if "--fuser" in sys.argv:
        print(build_fuser(force="--force" in sys.argv))
