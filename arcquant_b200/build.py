"""In-tree build of the native parts (no network, no pip):

  libarcq.so   CUDA kernels + C ABI, nvcc -gencode arch=compute_100a,code=sm_100a
  agemm*.so    the reference's `agemm` operator module as a torch C++ extension over that ABI

Run as ``python -m arcquant_b200.build``; add ``--ptxas`` to print register and
shared-memory usage.  nvcc cross-compiles, so this works on a machine without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(ROOT, "include")
LIB = os.path.join(HERE, "libarcq.so")
CUDA_SOURCES = ["arcq_api.cu", "arcq_quant.cu", "arcq_gemm.cu", "arcq_layer.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-I" + INCLUDE, "-I" + CSRC]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _newer(target: str, sources) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _cuda_sources():
    return [os.path.join(CSRC, s) for s in CUDA_SOURCES if os.path.exists(os.path.join(CSRC, s))]


def build_lib(force: bool = False, ptxas: bool = False) -> str:
    srcs = _cuda_sources()
    deps = srcs + [os.path.join(CSRC, "arcq_internal.h"), os.path.join(INCLUDE, "arcq.h")]
    if not force and _newer(LIB, deps):
        return LIB
    objs = []
    procs = []
    for s in srcs:
        o = os.path.join(CSRC, os.path.basename(s)[:-3] + ".o")
        cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas else []) + ["-c", s, "-o", o]
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(o)
    for s, p in procs:
        out, _ = p.communicate()
        if ptxas or p.returncode:
            sys.stderr.write(out)
        if p.returncode:
            raise RuntimeError(f"nvcc failed on {s}")
    subprocess.check_call([_nvcc(), "-shared", "-Wno-deprecated-gpu-targets", "-o", LIB] + objs + ["-lcudart"])
    return LIB


def build_agemm(force: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension as ce

    suffix = sysconfig.get_config_var("EXT_SUFFIX")
    target = os.path.join(HERE, "agemm" + suffix)
    src = os.path.join(CSRC, "agemm_ext.cpp")
    if not force and _newer(target, [src, os.path.join(INCLUDE, "arcq.h")]):
        return target
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_home = os.path.dirname(os.path.dirname(_nvcc()))
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=agemm",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           src, "-o", target, "-I" + INCLUDE, "-I" + sysconfig.get_paths()["include"],
           "-I" + os.path.join(cuda_home, "include")]
    cmd += ["-I" + p for p in ce.include_paths()]
    cmd += ["-L" + torch_lib, "-L" + HERE, "-larcq", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
            "-ltorch_python", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + torch_lib, "-w"]
    subprocess.check_call(cmd)
    return target


def build_all(force: bool = False, ptxas: bool = False):
    lib = build_lib(force=force, ptxas=ptxas)
    ext = build_agemm(force=force)
    return lib, ext


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv, ptxas="--ptxas" in sys.argv))
