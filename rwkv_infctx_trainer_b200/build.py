"""Build libwkv_b200.so (the C-ABI library, sm_100a only) in-tree with nvcc.

    python -m rwkv_infctx_trainer_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libwkv_b200.so")
STAMP = LIB + ".digest"
SOURCES = ["wkv_api.cu", "wkv4.cu", "wkv4_par.cu", "wkv56_scalar.cu", "wkv56_chunked.cu", "wkv56_chunked_bwd.cu",
           "timemix_fused.cu"]
HEADERS = ["wkv_common.cuh", os.path.join("..", "..", "include", "wkv_b200.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math", "-Xcompiler", "-fPIC"]


def have_nvcc() -> bool:
    return bool(shutil.which("nvcc")) or os.path.exists("/usr/local/cuda/bin/nvcc")


def _source_digest() -> str:
    """sha256 over the names and contents of everything the library is compiled from"""
    h = hashlib.sha256()
    files = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith((".cu", ".cuh", ".h"))]
    files.append(os.path.join(PKG, "..", "include", "wkv_b200.h"))
    for f in files:
        h.update(os.path.basename(f).encode())
        with open(f, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _stale() -> bool:
    """The library is current when the digest recorded beside it at build time matches the
    sources (file times are not used: they do not survive a copy of the tree)."""
    if not os.path.exists(LIB) or not os.path.exists(STAMP):
        return True
    with open(STAMP) as f:
        return f.read().strip() != _source_digest()


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or older than its sources."""
    if not force and not _stale():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libwkv_b200.so")
    objs = []
    bdir = os.path.join(PKG, "build")
    os.makedirs(bdir, exist_ok=True)
    procs = []
    for s in SOURCES:
        obj = os.path.join(bdir, s.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, s), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd), flush=True)
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
        objs.append(obj)
    for s, p in procs:
        out = p.communicate()[0].decode()
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {s}:\n{out}")
        if verbose and out:
            print(out)
    # link beside the target and move into place: another process may be loading the library
    tmp = f"{LIB}.{os.getpid()}.tmp"
    subprocess.check_call([nvcc, "-shared", "-o", tmp, *objs])
    os.replace(tmp, LIB)
    with open(STAMP + f".{os.getpid()}", "w") as f:
        f.write(_source_digest())
    os.replace(STAMP + f".{os.getpid()}", STAMP)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
