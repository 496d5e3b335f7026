"""ctypes binding of libwkv_b200.so (declared in include/wkv_b200.h).

The library is the product: if it cannot be loaded this module raises, there is
no PyTorch or CPU fallback behind any op of this package.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import build as _build

WKV_F32, WKV_BF16, WKV_F16 = 0, 1, 2
WKV_W_RAW, WKV_W_NEGEXP = 0, 1
WKV_STATE_KV, WKV_STATE_VK = 0, 1
WKV_PATH_AUTO, WKV_PATH_SCALAR, WKV_PATH_CHUNKED = 0, 1, 2
WKV_GROUP_STATES_NONE, WKV_GROUP_STATES_SAVE, WKV_GROUP_STATES_USE = 0, 1, 2

DTYPE_CODE = {torch.float32: WKV_F32, torch.bfloat16: WKV_BF16, torch.float16: WKV_F16}

_vp = ctypes.c_void_p


class WkvArgs(ctypes.Structure):
    _fields_ = [
        ("B", ctypes.c_int), ("T", ctypes.c_int), ("H", ctypes.c_int), ("N", ctypes.c_int),
        ("dtype", ctypes.c_int), ("w_kind", ctypes.c_int), ("state_layout", ctypes.c_int),
        ("path", ctypes.c_int),
        ("r", _vp), ("k", _vp), ("v", _vp), ("w", _vp), ("u", _vp), ("state_in", _vp),
        ("y", _vp), ("state_out", _vp),
        ("gy", _vp), ("gstate_out", _vp),
        ("gr", _vp), ("gk", _vp), ("gv", _vp), ("gw", _vp), ("gu", _vp), ("gstate_in", _vp),
        ("workspace", _vp), ("workspace_bytes", ctypes.c_size_t),
        ("state_ckpt", _vp), ("state_ckpt_bytes", ctypes.c_size_t),
        ("time_groups", ctypes.c_int),
        ("group_states", _vp), ("group_states_bytes", ctypes.c_size_t), ("group_states_mode", ctypes.c_int),
    ]


EXPORTS = [
    "wkv_error_string", "wkv_version", "wkv56_uses_chunked", "wkv56_state_ckpt_bytes",
    "wkv4_forward_workspace", "wkv4_forward", "wkv4_backward_workspace", "wkv4_backward",
    "wkv4_backward_static_limit", "wkv4_backward_static",
    "wkv4_state_ckpt_bytes", "wkv4_forward_ckpt", "wkv4_backward_ckpt",
    "wkv5_forward_workspace", "wkv5_backward_workspace", "wkv5_forward", "wkv5_backward",
    "wkv6_forward_workspace", "wkv6_backward_workspace", "wkv6_forward", "wkv6_backward",
    "wkv_selftest_wait_timeout", "wkv56_selftest_abort", "wkv56_group_states_bytes",
    "wkv_lnx_gate_forward", "wkv_lnx_gate_backward_workspace", "wkv_lnx_gate_backward",
    "wkv_ddlerp_forward", "wkv_ddlerp_backward_workspace", "wkv_ddlerp_backward",
]

_lib = None


def load() -> ctypes.CDLL:
    """Load the in-tree library.  Where nvcc exists it is first rebuilt if it is missing or older
    than its sources; where it does not (a GPU box that received a prebuilt copy) the file is
    taken as it is, and a missing file is an error."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB
    if _build.have_nvcc():
        path = _build.build()
    elif not os.path.exists(path):
        raise ImportError(f"{path} is missing and there is no nvcc to build it")
    lib = ctypes.CDLL(path)
    if any(not hasattr(lib, name) for name in EXPORTS):
        # a library from older sources: rebuild once (raises if nvcc is absent)
        path = _build.build(force=True)
        lib = ctypes.CDLL(path)
        missing = [name for name in EXPORTS if not hasattr(lib, name)]
        if missing:
            raise ImportError(f"{path} lacks symbols {missing}")
    lib.wkv_error_string.restype = ctypes.c_char_p
    lib.wkv_error_string.argtypes = [ctypes.c_int]
    lib.wkv_version.restype = ctypes.c_char_p
    i, f = ctypes.c_int, _vp
    lib.wkv4_forward_workspace.restype = ctypes.c_size_t
    lib.wkv4_forward_workspace.argtypes = [i, i, i]
    lib.wkv4_forward.restype = i
    lib.wkv4_forward.argtypes = [i, i, i, i, f, f, f, f, f, f, f, _vp, ctypes.c_size_t, _vp]
    lib.wkv4_backward_workspace.restype = ctypes.c_size_t
    lib.wkv4_backward_workspace.argtypes = [i, i, i]
    lib.wkv4_backward.restype = i
    lib.wkv4_backward.argtypes = [i, i, i, i] + [f] * 12 + [_vp, ctypes.c_size_t, _vp]
    lib.wkv4_state_ckpt_bytes.restype = ctypes.c_size_t
    lib.wkv4_state_ckpt_bytes.argtypes = [i, i, i]
    lib.wkv4_forward_ckpt.restype = i
    lib.wkv4_forward_ckpt.argtypes = [i, i, i, i, f, f, f, f, f, f, f, _vp, ctypes.c_size_t, _vp, ctypes.c_size_t, _vp]
    lib.wkv4_backward_ckpt.restype = i
    lib.wkv4_backward_ckpt.argtypes = [i, i, i, i] + [f] * 12 + [_vp, ctypes.c_size_t, _vp, ctypes.c_size_t, _vp]
    lib.wkv4_backward_static_limit.restype = ctypes.c_size_t
    lib.wkv4_backward_static_limit.argtypes = []
    lib.wkv4_backward_static.restype = i
    lib.wkv4_backward_static.argtypes = [i, i, i, i] + [f] * 12 + [_vp]
    lib.wkv56_uses_chunked.restype = i
    lib.wkv56_uses_chunked.argtypes = [ctypes.POINTER(WkvArgs), i]
    lib.wkv56_group_states_bytes.restype = ctypes.c_size_t
    lib.wkv56_group_states_bytes.argtypes = [ctypes.POINTER(WkvArgs)]
    lib.wkv56_state_ckpt_bytes.restype = ctypes.c_size_t
    lib.wkv56_state_ckpt_bytes.argtypes = [ctypes.POINTER(WkvArgs), i]
    lib.wkv_selftest_wait_timeout.restype = i
    lib.wkv_selftest_wait_timeout.argtypes = [_vp, ctypes.c_uint, _vp]
    lib.wkv56_selftest_abort.restype = i
    lib.wkv56_selftest_abort.argtypes = [ctypes.POINTER(WkvArgs), i, i, i, i, ctypes.c_uint, _vp]
    fl, sz = ctypes.c_float, ctypes.c_size_t
    lib.wkv_lnx_gate_forward.restype = i
    lib.wkv_lnx_gate_forward.argtypes = [i, i, f, f, f, f, fl, f, _vp]
    lib.wkv_lnx_gate_backward_workspace.restype = sz
    lib.wkv_lnx_gate_backward_workspace.argtypes = [i, i]
    lib.wkv_lnx_gate_backward.restype = i
    lib.wkv_lnx_gate_backward.argtypes = [i, i, f, f, f, f, fl, f, f, f, f, f, _vp, sz, _vp]
    lib.wkv_ddlerp_forward.restype = i
    lib.wkv_ddlerp_forward.argtypes = [i, i, i, i, f, f, f, f, f, _vp]
    lib.wkv_ddlerp_backward_workspace.restype = sz
    lib.wkv_ddlerp_backward_workspace.argtypes = [i, i, i, i]
    lib.wkv_ddlerp_backward.restype = i
    lib.wkv_ddlerp_backward.argtypes = [i, i, i, i] + [f] * 10 + [_vp, sz, _vp]
    for v in ("wkv5", "wkv6"):
        for d in ("forward", "backward"):
            fn = getattr(lib, f"{v}_{d}")
            fn.restype = i
            fn.argtypes = [ctypes.POINTER(WkvArgs), _vp]
            ws = getattr(lib, f"{v}_{d}_workspace")
            ws.restype = ctypes.c_size_t
            ws.argtypes = [ctypes.POINTER(WkvArgs)]
    _lib = lib
    return lib


def check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what}: {load().wkv_error_string(code).decode()} (code {code})")


def ptr(t):
    return None if t is None else t.data_ptr()


def stream_handle(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(*tensors) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("wkv_b200 ops run on CUDA tensors only (there is no CPU path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError("all tensors of one WKV call must live on the same device")
    return dev
