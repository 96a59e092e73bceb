"""TEST INFRASTRUCTURE ONLY -- Python face of the CPU projection oracle.

Two independent restatements of the matrix the reference's fast_jl kernel
defines (fast_jl/random.cuh:13-60, fast_jl/fast_jl_kernel.cuh:34-45,60-87,
121-127, fast_jl/fast_jl.cu:42):

* ``jl_oracle.c`` walks the kernel's own structure (a 16x32 factor tile per
  warp per 16 features, streams advanced sequentially);
* ``matrix_entries_closed_form`` below evaluates the closed form
  "element (f, n) is bit b of draw r of stream (c, tile)" with numpy.

They are cross-checked against each other and against golden vectors from the
compiled reference kernel.  Only tests, the smoke check and the benchmark's
CPU-baseline leg may import this module.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "jl_oracle.c")
_SO = os.path.join(_HERE, "libjl_oracle.so")

RADEMACHER, NORMAL = 0, 1
_DT = {np.dtype(np.float16): 0, np.dtype(np.float32): 2, np.dtype(np.float64): 3}


def build(force: bool = False) -> str:
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(_SRC):
        subprocess.check_call(["gcc", "-O2", "-fopenmp", "-ffp-contract=off", "-shared", "-fPIC",
                               _SRC, "-o", _SO, "-lm"])
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        l = ctypes.CDLL(build())
        u32, u64, vp, i = ctypes.c_uint32, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_int
        l.tbo_xorwow_draws.argtypes = [u32, u32, vp]
        l.tbo_xorwow_draws.restype = None
        l.tbo_box_muller.argtypes = [u32, u32, vp]
        l.tbo_box_muller.restype = None
        l.tbo_feature_tile_size.argtypes = [u64, u32]
        l.tbo_feature_tile_size.restype = u32
        l.tbo_matrix_rows.argtypes = [i, u64, u32, u32, u32, vp, u32, vp]
        l.tbo_matrix_rows.restype = i
        l.tbo_project.argtypes = [i, vp, i, u64, u64, u64, u32, u32, u32, i, vp]
        l.tbo_project.restype = i
        l.tbo_project_column_groups.argtypes = [i, vp, i, u64, u64, u64, u32, u32, i, vp, u32, vp]
        l.tbo_project_column_groups.restype = i
        _lib = l
    return _lib


def _ptype(p):
    if p in (RADEMACHER, "rademacher"):
        return RADEMACHER
    if p in (NORMAL, "normal"):
        return NORMAL
    raise ValueError(p)


def xorwow_draws(seed: int, n: int) -> np.ndarray:
    out = np.empty(n, np.uint32)
    lib().tbo_xorwow_draws(seed & 0xFFFFFFFF, n, out.ctypes.data)
    return out


def box_muller(x: int, y: int) -> np.ndarray:
    out = np.empty(2, np.float32)
    lib().tbo_box_muller(x, y, out.ctypes.data)
    return out


def feature_tile_size(F: int, tiles: int) -> int:
    return lib().tbo_feature_tile_size(F, tiles)


def matrix_rows(ptype, F: int, N: int, seed: int, tiles: int, feats) -> np.ndarray:
    """Rows P[f, :] (float32; +-1 or fp16-representable normals) for the given features."""
    feats = np.ascontiguousarray(np.asarray(feats, dtype=np.uint64))
    out = np.empty((len(feats), N), np.float32)
    rc = lib().tbo_matrix_rows(_ptype(ptype), F, N, seed, tiles, feats.ctypes.data, len(feats),
                               out.ctypes.data)
    if rc:
        raise ValueError(f"tbo_matrix_rows failed: {rc}")
    return out


def matrix(ptype, F: int, N: int, seed: int, tiles: int) -> np.ndarray:
    return matrix_rows(ptype, F, N, seed, tiles, np.arange(F))


def project(ptype, grads, N: int, seed: int, tiles: int, round_f16: bool = False) -> np.ndarray:
    """fp64-accumulated projection of ``grads`` [B, F] (numpy fp16/fp32/fp64, or a
    uint16 array holding bf16 bit patterns with ``dtype`` attribute trick below)."""
    g = np.ascontiguousarray(grads)
    if g.dtype == np.uint16:  # bf16 bit patterns
        dt = 1
    else:
        dt = _DT[g.dtype]
    B, F = g.shape
    out = np.empty((B, N), np.float64)
    rc = lib().tbo_project(_ptype(ptype), g.ctypes.data, dt, B, F, F, N, seed, tiles,
                           int(round_f16), out.ctypes.data)
    if rc:
        raise ValueError(f"tbo_project failed: {rc}")
    return out


def project_column_groups(ptype, grads, seed: int, tiles: int, groups, round_f16: bool = False) -> np.ndarray:
    """The columns ``32 g .. 32 g + 31`` for every ``g`` in ``groups`` of the fp64-accumulated projection
    (``[B, 32 * len(groups)]``, groups side by side): a few columns of a projection whose full oracle would
    take minutes.  Columns do not depend on the projection dimension."""
    g = np.ascontiguousarray(grads)
    dt = 1 if g.dtype == np.uint16 else _DT[g.dtype]
    groups = np.ascontiguousarray(np.asarray(groups, dtype=np.uint32))
    B, F = g.shape
    out = np.empty((B, 32 * len(groups)), np.float64)
    rc = lib().tbo_project_column_groups(_ptype(ptype), g.ctypes.data, dt, B, F, F, seed, tiles, int(round_f16),
                                         groups.ctypes.data, len(groups), out.ctypes.data)
    if rc:
        raise ValueError(f"tbo_project_column_groups failed: {rc}")
    return out


# --------------------------------------------------------------------------
# numpy twin: closed form, independent of the C code's structure
# --------------------------------------------------------------------------

def _np_seed(seed):
    """XORWOW state after curand_init(seed, 0, 0), vectorised over uint32 seeds."""
    seed = np.asarray(seed, dtype=np.uint32)
    with np.errstate(over="ignore"):
        s0 = seed ^ np.uint32(0xAAD26B49)
        t0 = np.uint32(1099087573) * s0
        t1 = np.uint32((2591861531 * 0xF7DCEFDD) & 0xFFFFFFFF)
        v = [np.uint32(123456789) + t0, np.uint32(362436069) ^ t0,
             np.full_like(t0, (521288629 + int(t1)) & 0xFFFFFFFF),
             np.full_like(t0, 88675123 ^ int(t1)), np.uint32(5783321) + t0]
        d = np.uint32(6615241) + t1 + t0
    return v, d


def _np_next(v, d):
    with np.errstate(over="ignore"):
        t = v[0] ^ (v[0] >> np.uint32(2))
        v4 = (v[4] ^ (v[4] << np.uint32(4))) ^ (t ^ (t << np.uint32(1)))
        v = [v[1], v[2], v[3], v[4], v4]
        d = d + np.uint32(362437)
        return v, d, v4 + d


def matrix_entries_closed_form(ptype, F, N, seed, tiles, feats) -> np.ndarray:
    """Same contract as ``matrix_rows``; Rademacher only needs integer work, the
    Gaussian branch uses numpy float32 math (so it is looser than the C twin)."""
    p = _ptype(ptype)
    tiles = min(F, tiles)
    fts = (F - 1) // tiles + 1
    n = np.arange(N, dtype=np.int64)
    nl = n & 31
    out = np.empty((len(feats), N), np.float32)
    for i, f in enumerate(feats):
        by, t = divmod(int(f), fts)
        r, k = t >> 4, t & 15
        L = (nl >> 1) + 16 * (k & 1)
        c = (n & ~31) + L
        S = (seed + 658105236 * c + 359124577 * by) & 0xFFFFFFFF
        v, d = _np_seed(S.astype(np.uint32))
        if p == RADEMACHER:
            for _ in range(r + 1):
                v, d, draw = _np_next(v, d)
            bit = (draw >> (2 * (k >> 1) + (nl & 1)).astype(np.uint32)) & np.uint32(1)
            out[i] = np.where(bit == 1, 1.0, -1.0)
        else:
            q = 8 * r + (k >> 1)
            for _ in range(2 * q + 1):
                v, d, x = _np_next(v, d)
            v, d, y = _np_next(v, d)
            inv = np.float32(2.3283064e-10)
            inv2pi = np.float32(2.3283064e-10) * np.float32(6.2831855)
            u = (x.astype(np.float64) * np.float64(inv) + np.float64(inv / 2)).astype(np.float32)
            w = (y.astype(np.float64) * np.float64(inv2pi) + np.float64(inv2pi / 2)).astype(np.float32)
            s = np.sqrt(np.float32(-2.0) * np.log(u)).astype(np.float32)
            val = np.where((nl & 1) == 0, np.sin(w) * s, np.cos(w) * s).astype(np.float32)
            out[i] = val.astype(np.float16).astype(np.float32)
    return out
