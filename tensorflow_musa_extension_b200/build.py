"""Builds libmusa_plugin_kernels.so (the sm_100a launcher layer) in-tree.

    python -m tensorflow_musa_extension_b200.build [--force] [--verbose]

The library is compiled with nvcc for sm_100a only and is written next to this
file, where `_loader.py` looks first.  nvcc cross-compiles, so no GPU is needed
to build.  This stands where the reference's CMake `mcc` device-code step does
(CMakeLists.txt:188-234 of the reference project).
"""
import argparse
import hashlib
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
BUILD_DIR = os.path.join(PKG_DIR, "build")
LIB_NAME = "libmusa_plugin_kernels.so"
LIB_PATH = os.path.join(PKG_DIR, LIB_NAME)

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA toolkit is required to build "
                           + LIB_NAME)
    return exe


def sources():
    out = []
    for root, _, files in os.walk(CSRC):
        for f in sorted(files):
            if f.endswith((".cu", ".cc")):
                out.append(os.path.join(root, f))
    return sorted(out)


def _headers_digest():
    h = hashlib.sha256()
    hdrs = []
    for root, _, files in os.walk(CSRC):
        hdrs += [os.path.join(root, f) for f in files if f.endswith((".h", ".cuh"))]
    hdrs.append(os.path.join(PKG_DIR, "..", "include", "musa_plugin_kernels.h"))
    for p in sorted(hdrs):
        with open(p, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force=False, verbose=False):
    """Compiles every source under csrc/ and links the shared library."""
    os.makedirs(BUILD_DIR, exist_ok=True)
    nvcc = _nvcc()
    stamp = _headers_digest()
    objs = []
    relinked = force or not os.path.exists(LIB_PATH)
    for src in sources():
        rel = os.path.relpath(src, CSRC).replace(os.sep, "_")
        obj = os.path.join(BUILD_DIR, rel + ".o")
        tag = obj + ".stamp"
        with open(src, "rb") as fh:
            want = hashlib.sha256(fh.read() + stamp.encode()).hexdigest()
        have = open(tag).read() if os.path.exists(tag) else ""
        if force or have != want or not os.path.exists(obj):
            cmd = [nvcc] + NVCC_FLAGS + ["-x", "cu", "-c", src, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
                print(" ".join(cmd), flush=True)
            subprocess.run(cmd, check=True)
            with open(tag, "w") as fh:
                fh.write(want)
            relinked = True
        objs.append(obj)
    if relinked:
        cmd = [nvcc, "-shared", "-o", LIB_PATH] + objs + ["-lpthread"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
    sys.exit(0)
