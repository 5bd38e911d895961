"""TEST INFRASTRUCTURE ONLY: build the reference project's own CUDA kernels into oracle/_ref/libraf_ref_kernels.so.

The reference's kernel sources are compiled from where they lie (nothing is copied into this repository):

    src/op/dialect/cuda/kernels/tutel_moe_dispatch.cu   gating locations, encode/decode and their gradients, batch-
                                                         prioritized locations, merge_masks, redispatch
    src/op/dialect/cuda/kernels/multi_tensor_lans.cu    LANS (L2 norms, stage 1, stage 2)

together with raf_ref_entry.cu of this folder (unmangled entry points) and stub/raf/device.h (a stand-in for one header of
the reference that needs TVM and dlpack, un-vendored submodules).  The result travels to the GPU machine as a built file;
the reference tree does not, so the GPU tests load the library and skip when it is absent.

    python oracle/ref_build/build_ref.py [reference root]
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(os.path.dirname(HERE), "_ref")
LIB = os.path.join(OUT, "libraf_ref_kernels.so")
KERNELS = "src/op/dialect/cuda/kernels"
DEFAULT_ROOT = os.environ.get("LANCET_REFERENCE_ROOT", "/root/reference")   # where the reference tree is mounted, if at all
SOURCES = ("tutel_moe_dispatch.cu", "multi_tensor_lans.cu")


def build(ref_root=None, verbose=False):
    """Returns the library path, or None when the reference tree or nvcc is not available."""
    kdir = os.path.join(ref_root or DEFAULT_ROOT, KERNELS)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not all(os.path.exists(os.path.join(kdir, s)) for s in SOURCES) or not os.path.exists(nvcc):
        return None
    os.makedirs(OUT, exist_ok=True)
    srcs = [os.path.join(kdir, s) for s in SOURCES] + [os.path.join(HERE, "raf_ref_entry.cu")]
    newest = max(os.path.getmtime(p) for p in srcs + [os.path.join(HERE, "stub", "raf", "device.h"), __file__])
    if os.path.exists(LIB) and os.path.getmtime(LIB) >= newest:
        return LIB
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-w", "-shared", "-Xcompiler", "-fPIC",
           "-I", os.path.join(HERE, "stub"), "-I", kdir, "-o", LIB] + srcs
    if verbose:
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(*(sys.argv[1:2]), verbose=True))
