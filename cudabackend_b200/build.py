"""Builds libAvocadoCudaBackend.so, the C-ABI library, from cudabackend_b200/csrc with nvcc for sm_100a.

The library is linked in-tree (cudabackend_b200/lib/) so that it travels with a copy of the repository;
nothing is installed.  Objects are rebuilt only when a source or header is newer than the object.
Run as ``python -m cudabackend_b200.build`` or call :func:`build`.
"""
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "cudabackend_b200", "csrc")
OBJ_DIR = os.path.join(ROOT, "cudabackend_b200", "build")
LIB_DIR = os.path.join(ROOT, "cudabackend_b200", "lib")
LIB_NAME = "libAvocadoCudaBackend.so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC,-fvisibility=hidden",
                "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-DCUDA_BACKEND"]


def library_path():
    return os.path.join(LIB_DIR, LIB_NAME)


def _nvcc():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the CUDA extension cannot be built")
    return nvcc


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))


def _newest_header_mtime():
    newest = 0.0
    for base in (CSRC, os.path.join(ROOT, "include", "Avocado")):
        for f in os.listdir(base):
            if f.endswith((".h", ".hpp", ".cuh")):
                newest = max(newest, os.path.getmtime(os.path.join(base, f)))
    return newest


def _compile(nvcc, src, obj, verbose, extra):
    cmd = [nvcc, "-c", os.path.join(CSRC, src), "-o", obj] + ARCH_FLAGS + COMMON_FLAGS + extra
    if src.endswith(".cpp"):
        cmd += ["-x", "cu"]
    result = subprocess.run(cmd, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, result.stdout, result.stderr))
    if verbose and (result.stdout or result.stderr):
        sys.stderr.write(result.stdout + result.stderr)
    return src


def build(force=False, verbose=False, ptxas_info=False):
    """Compiles every source under csrc/ for sm_100a and links the shared library. Returns its path."""
    nvcc = _nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    os.makedirs(LIB_DIR, exist_ok=True)
    header_mtime = _newest_header_mtime()
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    objects, jobs = [], []
    for src in _sources():
        obj = os.path.join(OBJ_DIR, os.path.splitext(src)[0] + ".o")
        objects.append(obj)
        stale = force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(os.path.join(CSRC, src)), header_mtime)
        if stale:
            jobs.append((src, obj))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            for done in pool.map(lambda job: _compile(nvcc, job[0], job[1], verbose or ptxas_info, extra), jobs):
                if verbose:
                    print("compiled", done)
    lib = library_path()
    if jobs or not os.path.exists(lib):
        cmd = [nvcc, "-shared", "-o", lib] + objects + ARCH_FLAGS + ["-Xcompiler", "-fPIC", "-cudart", "static"]
        result = subprocess.run(cmd, capture_output=True, text=True)
        if result.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (result.stdout, result.stderr))
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv))
