"""In-tree build of the two shared libraries of the package (sm_100a only).

  libb200moe.so       - the CUDA kernels behind the C ABI declared in include/b200moe.h (nvcc, no torch)
  libb200_moe_ops.so  - TORCH_LIBRARY(my_ops): the reference's custom-op surface, calling the C ABI

Both land next to this file so that they travel with the source tree; nothing is cached elsewhere.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
ROOT = os.path.dirname(HERE)
NATIVE_LIB = os.path.join(HERE, "libb200moe.so")
OPS_LIB = os.path.join(HERE, "libb200_moe_ops.so")
CU_SOURCES = ["route.cu", "permute.cu", "gemm_simple.cu", "gemm_tc.cu", "gemm_bf16_tc.cu", "experts.cu", "ep.cu",
              "ep_p2p.cu"]
NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("build step failed: " + " ".join(cmd[:3]) + " ...")
    if verbose and (r.stdout or r.stderr):
        print(r.stdout + r.stderr)


def build_native(force=False, verbose=False):
    srcs = [os.path.join(CSRC, s) for s in CU_SOURCES]
    deps = srcs + [os.path.join(CSRC, h) for h in ("common.cuh", "internal.h", "tc_ptx.cuh")] + [
        os.path.join(ROOT, "include", "b200moe.h")]
    if not force and not _newer(NATIVE_LIB, deps):
        return NATIVE_LIB
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    cmd = [nvcc, "-O3", "-std=c++17", *NVCC_ARCH, "-lineinfo", "-Xcompiler", "-fPIC", "-shared",
           *srcs, "-o", NATIVE_LIB]
    _run(cmd, verbose)
    return NATIVE_LIB


def build_torch_ops(force=False, verbose=False):
    build_native(force=force, verbose=verbose)
    src = os.path.join(CSRC, "my_ops.cpp")
    if not force and not _newer(OPS_LIB, [src, NATIVE_LIB, os.path.join(ROOT, "include", "b200moe.h")]):
        return OPS_LIB
    import torch
    from torch.utils import cpp_extension as ce
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc = []
    for p in ce.include_paths() + [os.path.join(cuda_home, "include")]:
        inc += ["-isystem", p]
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-Wno-deprecated-declarations",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           *inc, src, "-o", OPS_LIB, f"-L{tlib}", f"-L{HERE}", "-lc10", "-lc10_cuda", "-ltorch_cpu",
           "-ltorch_cuda", "-ltorch", "-lb200moe", f"-L{os.path.join(cuda_home, 'lib64')}", "-lcudart",
           "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{tlib}"]
    _run(cmd, verbose)
    return OPS_LIB


def build_all(force=False, verbose=False):
    build_native(force=force, verbose=verbose)
    build_torch_ops(force=force, verbose=verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
