"""Builds oracle/_ref/libref_winograd.so from the REFERENCE's own sources.  TEST INFRASTRUCTURE ONLY.

The reference's non-fused Winograd kernels (src/winograd_nonfused.cu), its cuBLAS GEMM wrapper (src/gemm.cpp) and its
im2row lowering (src/im2row.cu) are compiled unmodified, where they lie under the reference tree, against the stand-in header in oracle/ref_shim/ and the
type header of this repository, and linked with oracle/ref_harness.cu.  The reference targets sm_61 and does not
compile natively for sm >= 80 (its bfloat16 number class is empty there), so the device code is emitted as compute_75
PTX, which the driver JIT-compiles on the B200.  The output is a comparator for the GPU parity tests; nothing of the
product loads it and no reference source is copied into this repository.
"""
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
# AVOCADO_REFERENCE_ROOT names the checkout of the reference; the default is where this project's build container mounts it
REFERENCE_ROOT = os.environ.get("AVOCADO_REFERENCE_ROOT", "/root/reference")
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libref_winograd.so")


def build(force=False):
    sources = [os.path.join(REFERENCE_ROOT, "src", "winograd_nonfused.cu"), os.path.join(REFERENCE_ROOT, "src", "gemm.cpp"),
               os.path.join(REFERENCE_ROOT, "src", "im2row.cu"), os.path.join(HERE, "ref_harness.cu")]
    if not all(os.path.exists(s) for s in sources):
        raise RuntimeError("reference sources not found under %s" % REFERENCE_ROOT)
    shim = os.path.join(HERE, "ref_shim", "Avocado", "backend_descriptors.hpp")
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= max(os.path.getmtime(s) for s in sources + [shim]):
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = [nvcc, "-shared", "-o", LIB, "-std=c++14", "--expt-relaxed-constexpr", "-DCUDA_BACKEND", "-DNDEBUG", "-O2", "-x", "cu",
           "-gencode", "arch=compute_75,code=compute_75", "-Xcompiler", "-fPIC", "-I", os.path.join(REFERENCE_ROOT, "include"),
           "-I", os.path.join(HERE, "ref_shim"), "-I", os.path.join(ROOT, "include"), "-I", os.path.join(REFERENCE_ROOT, "src")] + sources + ["-lcublas"]
    result = subprocess.run(cmd, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError("building the reference comparator failed:\n" + result.stdout[-4000:] + result.stderr[-4000:])
    return LIB


if __name__ == "__main__":
    print(build(force=True))
