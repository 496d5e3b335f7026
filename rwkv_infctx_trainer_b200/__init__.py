"""B200 (sm_100a) implementation of the RWKV WKV time-mix recurrence (v4/v5/v6),
behind the op interfaces of RWKV-infctx-trainer.  Importing the package loads
libwkv_b200.so; there is no fallback if that fails."""
from . import _lib
from ._lib import (WKV_PATH_AUTO, WKV_PATH_CHUNKED, WKV_PATH_SCALAR, WKV_STATE_KV, WKV_STATE_VK,
                   WKV_W_NEGEXP, WKV_W_RAW)
from .timemix import ddlerp, lnx_gate
from .timemix_block import RWKV_TimeMix, RWKV_TimeMix6_0, RWKV_TimeMix_v4, TimeMixState
from .wkv4 import WKVFunction, register_torch_op, wkv, wkv_op
from .wkv5 import RUN_WKV5_CUDA, WKV5, WKV5_CUDA, wkv5, wkv5_cuda_kernel
from .wkv6 import (RUN_WKV6STATE_CUDA, WKV6, WKV6STATE_CUDA, wkv6, wkv6_cuda_kernel,
                   wkv6state_cuda_kernel)

_lib.load()
register_torch_op()

__all__ = [
    "WKVFunction", "wkv", "wkv_op", "register_torch_op",
    "WKV5", "wkv5", "WKV5_CUDA", "RUN_WKV5_CUDA", "wkv5_cuda_kernel",
    "WKV6", "wkv6", "WKV6STATE_CUDA", "RUN_WKV6STATE_CUDA", "wkv6state_cuda_kernel",
    "wkv6_cuda_kernel", "lnx_gate", "ddlerp", "RWKV_TimeMix", "RWKV_TimeMix6_0",
    "RWKV_TimeMix_v4", "TimeMixState",
]
