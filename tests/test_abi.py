"""The C-ABI library: loads, exports every symbol include/wkv_b200.h declares,
and rejects bad arguments with an error code before touching the GPU."""
import ctypes
import os
import re

import rwkv_infctx_trainer_b200._lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "wkv_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b(wkv[0-9a-z_]*)\s*\(", text))


def test_library_exports_every_declared_symbol():
    lib = L.load()
    names = declared_functions()
    assert names, "no declarations found"
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/wkv_b200.h but not exported"
    assert set(L.EXPORTS) <= names
    assert lib.wkv_version().decode().endswith("sm_100a")


def test_error_codes_without_gpu():
    lib = L.load()
    assert lib.wkv6_forward(None, None) == 1  # WKV_ERR_NULL
    a = L.WkvArgs()
    a.B, a.T, a.H, a.N = 1, 4, 1, 32
    assert lib.wkv6_forward(ctypes.byref(a), None) == 2  # head size other than 64
    a.N = 64
    a.dtype = 9
    assert lib.wkv5_forward(ctypes.byref(a), None) == 3
    a.dtype = L.WKV_BF16
    assert lib.wkv6_forward(ctypes.byref(a), None) == 1  # u is NULL
    buf = (ctypes.c_char * 4096)()
    base = ctypes.addressof(buf)
    base += (-base) % 16
    for f in ("r", "k", "v", "w", "u", "y"):
        setattr(a, f, base)
    a.r = base + 2
    assert lib.wkv6_forward(ctypes.byref(a), None) == 4  # misaligned
    assert lib.wkv4_forward(-1, 1, 1, 0, None, None, None, None, None, None, None, None, 0, None) == 2
    assert lib.wkv4_forward(1, 1, 1, 0, None, None, None, None, None, None, None, None, 0, None) == 1
    assert lib.wkv4_backward_workspace(2, 100, 8) == 2 * 7 * 3 * 8 * 4      # short: one thread per chain
    assert lib.wkv4_forward_workspace(2, 100, 8) == 0
    assert lib.wkv4_forward_workspace(2, 256, 8) == 2 * 2 * 4 * 3 * 8 * 4   # 64-token pieces
    assert b"workspace" in lib.wkv_error_string(5)
    # empty batch is a no-op, not an error
    a = L.WkvArgs()
    a.N = 64
    assert lib.wkv6_forward(ctypes.byref(a), None) == 0


def test_struct_matches_header_field_order():
    text = open(os.path.join(ROOT, "include", "wkv_b200.h")).read()
    body = text[text.index("typedef struct wkv_args {"):text.index("} wkv_args_t;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = []
    for decl in body.split("{", 1)[1].split(";"):
        decl = decl.strip()
        if not decl:
            continue
        names = re.sub(r"^(const\s+)?(void|float|int|size_t)\s*", "", decl)
        fields += [n.strip().lstrip("*") for n in names.split(",")]
    assert fields == [f[0] for f in L.WkvArgs._fields_]


def test_handover_buffer_size_without_gpu():
    """wkv56_state_ckpt_bytes: chunk-start states + scaled r + chunk decays + the per-chunk mild
    flags, each 256-byte aligned; 0 when the call would not run on the chunked kernels"""
    lib = L.load()
    a = L.WkvArgs()
    a.B, a.T, a.H, a.N, a.dtype, a.w_kind = 2, 200, 3, 64, L.WKV_BF16, L.WKV_W_RAW
    al = lambda x: (x + 255) // 256 * 256
    n = (200 + 63) // 64
    want = (al(2 * 3 * (n + 1) * 64 * 64 * 2) + al(2 * 200 * 3 * 64 * 2) + al(2 * 3 * n * 64 * 4)
            + al(2 * 3 * n))
    assert lib.wkv56_state_ckpt_bytes(ctypes.byref(a), 1) == want
    a.dtype = L.WKV_F32          # fp32 I/O runs on the token-serial kernels: nothing to hand over
    assert lib.wkv56_state_ckpt_bytes(ctypes.byref(a), 1) == 0
