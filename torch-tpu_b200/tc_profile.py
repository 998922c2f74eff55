"""Per-role cycle accounting of the tcgen05 GEMM kernels (the counterpart of the reference's op-level timing switch,
torch_tpu/csrc/core/OpTimer.h:3-10, one level down: inside the kernel).

    python torch-tpu_b200/tc_profile.py [tokens] [workload]

Builds a second copy of the kernel library with -DMOE_TC_PROFILE (clock64 reads around every wait and work section
of the producer, MMA and epilogue roles), runs the layer once to fill the workspace, then each GEMM alone, and
prints the average cycles per CTA and per K block.  Numbers are for reading the pipeline, not for benchmarking: the
instrumentation itself costs a few percent.
"""
import ctypes
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, ROOT)
PROF_LIB = os.path.join(HERE, "libb200moe_prof.so")
NAMES = ["producer wait(empty)", "mma wait(full)", "mma wait(tmem_empty)", "mma total", "epilogue wait(done)",
         "epilogue wake->buffer released", "epilogue rest (FMAs after release, tile end)", "epilogue total",
         "  first two TMEM loads + wait", "  FMAs + two more loads + wait", "  loop top (scale products, next scale loads)", "  fence + release"]


def build():
    from importlib import import_module
    b = import_module("torch_tpu_b200.build")
    srcs = [os.path.join(b.CSRC, s) for s in b.CU_SOURCES]
    if os.path.exists(PROF_LIB) and all(os.path.getmtime(s) < os.path.getmtime(PROF_LIB) for s in srcs):
        return
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    subprocess.run([nvcc, "-O3", "-std=c++17", "-DMOE_TC_PROFILE", *b.NVCC_ARCH, "-lineinfo", "-Xcompiler", "-fPIC",
                    "-shared", *srcs, "-o", PROF_LIB], check=True)


def main():
    T = int(sys.argv[1]) if len(sys.argv) > 1 else 4096
    wlname = sys.argv[2] if len(sys.argv) > 2 else "mixtral"
    import torch_tpu_b200  # noqa: F401
    build()
    from torch_tpu_b200 import lib as L
    L.LIB_PATH = PROF_LIB
    import numpy as np
    import torch
    import bench
    from torch_tpu_b200 import ops
    wl = bench.WORKLOADS[wlname]
    layer = bench.build_layer(wl, T, "cuda:0", 0)
    x = bench.make_x(T, wl["H"], "cuda:0", 1).to("cuda:0")
    for _ in range(3):
        layer.forward(x)
    torch.cuda.synchronize()
    lib = L.lib()
    lib.b200moe_debug_read_tc_profile.argtypes = [ctypes.c_void_p]
    wg, wu, wd, sg, su, sd = layer.w
    n_sm = torch.cuda.get_device_properties(0).multi_processor_count
    offs = None
    for label, mask, KB, NT in (("gate/up GEMM", 16 | 64 | 128, wl["H"] // 128, wl["I"] // 128),
                                ("down GEMM", 16 | 32 | 128, wl["I"] // 128, (wl["H"] + 255) // 256)):
        ops.experts(layer.out[:T], x, wg, wu, wd, sg, su, sd, layer.ids[:T], layer.topk_w[:T], shared=None,
                    workspace=layer.workspace, reserved=mask)
        torch.cuda.synchronize()
        buf = np.zeros(256 * 12, dtype=np.int64)
        lib.b200moe_debug_read_tc_profile(buf.ctypes.data)
        a = buf.reshape(256, 12)[:n_sm].mean(0)
        cnt = torch.bincount(layer.ids[:T].flatten().long(), minlength=wl["E"])
        mtiles = int(((cnt + 127) // 128).sum())
        kblocks = mtiles * NT * KB / n_sm
        print(f"{label}: T={T} {wlname}, {mtiles} m-tiles x {NT} n-tiles x {KB} K blocks = {kblocks:.0f} K blocks per CTA")
        for n, v in zip(NAMES, a):
            print(f"    {n:48s} {v:12.0f} cycles  {v / kblocks:8.0f} per K block")


if __name__ == "__main__":
    main()
