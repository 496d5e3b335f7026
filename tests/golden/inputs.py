"""Deterministic synthetic inputs for the WKV parity tests and fixtures.

A counter-based generator (splitmix64 hash of seed and element index, then
Box-Muller) written out in numpy integer arithmetic, so the same seed gives the
same numbers on every machine and numpy version.  The fixtures under this
directory store only outputs; tests rebuild the inputs from here.
"""
from __future__ import annotations

import numpy as np

_M = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix(z: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = (z + np.uint64(0x9E3779B97F4A7C15)) & _M
        z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M
        z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M
        return z ^ (z >> np.uint64(31))


def uniform01(shape, seed: int, stream: int = 0) -> np.ndarray:
    n = int(np.prod(shape))
    with np.errstate(over="ignore"):
        base = _splitmix(np.array([seed * 1000003 + stream * 7919 + 12345], dtype=np.uint64))[0]
        idx = np.arange(n, dtype=np.uint64) * np.uint64(2654435761) + base
    bits = _splitmix(idx)
    return ((bits >> np.uint64(11)).astype(np.float64) + 0.5) / float(1 << 53)


def uniform(shape, seed: int, lo: float, hi: float, stream: int = 0) -> np.ndarray:
    return (lo + (hi - lo) * uniform01(shape, seed, stream)).reshape(shape)


def normal(shape, seed: int, mean: float = 0.0, std: float = 1.0, stream: int = 0) -> np.ndarray:
    u1 = uniform01(shape, seed, stream * 2 + 101)
    u2 = uniform01(shape, seed, stream * 2 + 102)
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return (mean + std * z).reshape(shape)


def wkv56_case(variant: str, B: int, T: int, H: int, N: int, seed: int,
               state: bool = True, gstate: bool = True) -> dict:
    """Inputs with the distributions the benchmark configurations name:
    r,k,v,gy ~ N(0,1); u ~ U(-1,1); v5 decay parameter d ~ U(-6,-1) per
    (head, channel); v6 decay parameter x ~ N(-0.6, 0.5) per (b,t,c);
    the decay itself is exp(-exp(.))."""
    C = H * N
    d = dict(
        r=normal((B, T, C), seed, stream=1), k=normal((B, T, C), seed, stream=2),
        v=normal((B, T, C), seed, stream=3), gy=normal((B, T, C), seed, stream=4),
        u=uniform((H, N), seed, -1.0, 1.0, stream=5),
    )
    if variant == "v6":
        d["x"] = normal((B, T, C), seed, mean=-0.6, std=0.5, stream=6)
    else:
        d["x"] = uniform((H, N), seed, -6.0, -1.0, stream=6)
    d["state_in"] = (normal((B, H, N, N), seed, std=0.5, stream=7) if state
                     else np.zeros((B, H, N, N)))
    d["gstate_out"] = (normal((B, H, N, N), seed, std=0.5, stream=8) if gstate
                       else np.zeros((B, H, N, N)))
    return d


def wkv4_case(B: int, T: int, C: int, seed: int, state: bool = True, gstate: bool = True) -> dict:
    """k,v,gy ~ N(0,1); time_decay ~ U(-5,1) (w = -exp(time_decay)); time_first u ~ U(-1,1).
    A non-trivial carried state is made by the caller by running a first segment."""
    return dict(
        k=normal((B, T, C), seed, stream=1), v=normal((B, T, C), seed, stream=2),
        gy=normal((B, T, C), seed, stream=3),
        td=uniform((C,), seed, -5.0, 1.0, stream=4), u=uniform((C,), seed, -1.0, 1.0, stream=5),
    )
