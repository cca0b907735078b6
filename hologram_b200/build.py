"""Build libhologram_b200.so (sm_100a only) in-tree with nvcc.

Run: python hologram_b200/build.py [--force] [--verbose]   (by path: importing the package needs the built library)
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libhologram_b200.so")
SOURCES = ["api.cu", "lut.cu", "glue.cu", "attention.cu", "gemm.cu", "quant_gemv.cu", "tp.cu", "session.cu", "addressed.cpp", "pool.cpp", "archive.cpp", "blake3.cpp", "label.cpp"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fno-fast-math", "--expt-relaxed-constexpr",
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _deps(src):
    deps = [src]
    for name in os.listdir(CSRC):
        if name.endswith((".h", ".cuh")):
            deps.append(os.path.join(CSRC, name))
    deps.append(os.path.join(HERE, "..", "include", "hologram_b200.h"))
    return deps


def build(force=False, verbose=False):
    objs = []
    procs = []
    for name in SOURCES:
        src = os.path.join(CSRC, name)
        obj = os.path.join(CSRC, os.path.splitext(name)[0] + ".o")
        objs.append(obj)
        newest = max(os.path.getmtime(d) for d in _deps(src))
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < newest:
            cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
            procs.append((name, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for name, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- {name} ---\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if force or procs or not os.path.exists(LIB):
        cmd = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + objs + ["-ldl"]
        subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
