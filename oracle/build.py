"""TEST INFRASTRUCTURE ONLY -- build recipes for the CPU oracle and for the
unmodified reference CUDA kernels used as a second checker on a GPU.

``build_naive()`` compiles ``wkv_naive.c`` (this directory) with gcc into
``oracle/libwkv_naive.so``.

``build_ref()`` compiles the RWKV-infctx-trainer project's own WKV ``.cu``
files, unchanged and from where they lie in the read-only project checkout,
for sm_100a, each together with a few lines of ``extern "C"`` glue from
``ref_glue/`` (ours), into ``oracle/_ref/*.so``.  Nothing is copied out of the
project tree; only the built objects land in ``oracle/_ref/`` (git-ignored).
It is a no-op when the checkout or nvcc is absent (e.g. on a GPU box, where the
prebuilt objects are used).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.environ.get("WKV_REFERENCE_ROOT", "/root/reference")
NAIVE_SO = os.path.join(HERE, "libwkv_naive.so")
REF_DIR = os.path.join(HERE, "_ref")


def _newer(target: str, *sources: str) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources if os.path.exists(s))


def build_naive(force: bool = False) -> str:
    src = os.path.join(HERE, "wkv_naive.c")
    if not force and _newer(NAIVE_SO, src):
        return NAIVE_SO
    cmd = ["gcc", "-O2", "-fPIC", "-shared", "-std=c99", "-o", NAIVE_SO, src, "-lm"]
    subprocess.check_call(cmd)
    return NAIVE_SO


# (output name, reference source relative to the project root, glue file, defines)
_REF_TARGETS = [
    ("libref_wkv4.so", "RWKV-v4neo/cuda/wkv_cuda_bf16.cu", "glue_v4.cu", ["-DTmax=2048"]),
    ("libref_wkv5.so", "RWKV-v5/src/module/cuda/wkv5_cuda.cu", "glue_v5.cu", ["-D_N_=64"]),
    ("libref_wkv6state.so", "RWKV-v6/src/module/cuda/wkv6state_cuda_v1.cu", "glue_v6.cu",
     ["-D_N_=64", "-D_T_=4096"]),
]


def build_ref(force: bool = False) -> list[str]:
    """Compile the project's CUDA WKV kernels for sm_100a into oracle/_ref/."""
    if not os.path.isdir(REF_ROOT) or shutil.which("nvcc") is None:
        return [os.path.join(REF_DIR, t[0]) for t in _REF_TARGETS
                if os.path.exists(os.path.join(REF_DIR, t[0]))]
    import torch
    from torch.utils import cpp_extension

    os.makedirs(REF_DIR, exist_ok=True)
    incs = [f"-I{p}" for p in cpp_extension.include_paths()]
    built = []
    for name, rel, glue, defs in _REF_TARGETS:
        src = os.path.join(REF_ROOT, rel)
        gsrc = os.path.join(HERE, "ref_glue", glue)
        out = os.path.join(REF_DIR, name)
        if not force and _newer(out, src, gsrc):
            built.append(out)
            continue
        cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "--use_fast_math",
               "-std=c++17", "-shared", "-Xcompiler", "-fPIC", "-w",
               "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
               *defs, *incs, src, gsrc, "-o", out]
        subprocess.check_call(cmd)
        built.append(out)
    return built


if __name__ == "__main__":
    print(build_naive(force="--force" in sys.argv))
    if "--ref" in sys.argv:
        for p in build_ref(force="--force" in sys.argv):
            print(p)
