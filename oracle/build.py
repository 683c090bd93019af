"""Compiles the CPU oracle (oracle/conv_oracle.c) into oracle/_build/liboracle.so with gcc.

Test infrastructure only: the product never loads this library.
"""
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(OUT_DIR, "liboracle.so")


def build(force=False):
    src = os.path.join(HERE, "conv_oracle.c")
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(src):
        return LIB
    gcc = shutil.which("gcc")
    if gcc is None:
        raise RuntimeError("gcc not found: the oracle cannot be built")
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = [gcc, "-O2", "-fopenmp", "-ffp-contract=off", "-fno-fast-math", "-shared", "-fPIC", "-o", LIB, src, "-lm"]
    result = subprocess.run(cmd, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError("gcc failed:\n" + result.stdout + result.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
