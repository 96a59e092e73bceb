"""Drop-in for the reference's ``fast_jl`` extension module.

Same six callables with the same positional signature
``(input, N, seed, num_feature_tiles) -> float32 CUDA tensor [B, N]``
(fast_jl/fast_jl.cu:81-110), backed by the sm_100a kernels behind the C ABI.
The 8 / 16 / 32 suffix (rows per launch in the reference) is only a name here:
every entry point takes any number of rows; one generation of the matrix serves up to 256 rows
(Rademacher) or 512 rows (Gaussian) of the batch.

To make an unmodified ``trak`` pick this module up::

    import sys, trak_b200.fast_jl
    sys.modules["fast_jl"] = trak_b200.fast_jl
"""
import os

import torch

from . import _lib

_STRICT = os.environ.get("TRAK_B200_STRICT", "1") != "0"
_DTYPES = {torch.float16: _lib.TB_F16, torch.bfloat16: _lib.TB_BF16, torch.float32: _lib.TB_F32}
_workspaces = {}
_MAX_CACHED_WORKSPACES = 8  # per process; streams come and go, their workspaces should not pile up


def _u32(name, v):
    if isinstance(v, bool) or not isinstance(v, int):
        try:
            v = v.__index__()
        except Exception:
            raise TypeError(f"{name} must be an unsigned 32-bit integer, got {type(v).__name__}")
    if v < 0 or v > 0xFFFFFFFF:
        raise TypeError(f"{name} must be an unsigned 32-bit integer, got {v}")
    return v


def _workspace(device, stream, nbytes):
    key = (device.index, stream)
    ws = _workspaces.pop(key, None)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
    _workspaces[key] = ws  # most recently used last
    while len(_workspaces) > _MAX_CACHED_WORKSPACES:
        _workspaces.pop(next(iter(_workspaces)))
    return ws


def free_workspaces():
    """Drops the cached per-(device, stream) workspaces and the matrices kept by the stored-matrix mode."""
    _workspaces.clear()
    _stored.clear()


class StoredMatrix:
    """The projection matrix of ``(F, N, seed, num_feature_tiles, proj_type)`` materialised in device memory
    (``2 * N`` bytes per feature: 91.6 GB for F = 11,173,962 and N = 4096), for ``project(..., matrix=...)``.
    ``dtype`` is the gradients' dtype it will be used with (fp32 gradients are rounded to fp16 on the way in,
    so they take the fp16 form).  Entries are bit for bit what ``project`` generates on the fly."""

    def __init__(self, F, N, seed, num_feature_tiles, proj_type, dtype=torch.float16, device="cuda"):
        dev = torch.device(device)
        if dev.type != "cuda":
            raise RuntimeError("StoredMatrix needs a CUDA device")
        if dev.index is None:
            dev = torch.device("cuda", torch.cuda.current_device())
        self.F, self.N = int(F), _u32("N", N)
        self.seed, self.tiles = _u32("seed", seed), _u32("num_feature_tiles", num_feature_tiles)
        self.proj_type, self.device = int(proj_type), dev
        self.elem = _lib.TB_BF16 if dtype == torch.bfloat16 else _lib.TB_F16
        l = _lib.lib()
        nbytes = l.tb_matrix_bytes(self.F, self.N, max(self.tiles, 1))
        if nbytes == 0:
            _lib.check(_lib.TB_ERR_BAD_PROJ_DIM if self.N % 512 else 2)
        self.data = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            stream = torch.cuda.current_stream(dev).cuda_stream
            _lib.check(l.tb_matrix_generate(dev.index, stream, self.F, self.N, self.seed, self.tiles, self.proj_type,
                                            self.elem, self.data.data_ptr(), nbytes))
            _lib.device_status(dev.index)

    @staticmethod
    def nbytes(F, N, num_feature_tiles):
        return _lib.lib().tb_matrix_bytes(int(F), int(N), int(num_feature_tiles))

    def matches(self, input, N, num_feature_tiles):
        elem = _lib.TB_BF16 if input.dtype == torch.bfloat16 else _lib.TB_F16
        return input.shape[1] == self.F and N == self.N and num_feature_tiles == self.tiles and \
            elem == self.elem and input.device == self.device


def project(input, N, seed, num_feature_tiles, proj_type, *, alpha=1.0, out=None, accumulate=False,
            strict=None, allow_strided=False, matrix=None):
    """``alpha * input @ P`` with the fast_jl matrix P(seed, num_feature_tiles, proj_type).

    ``out`` (float32 [B, N], rows 16-byte aligned) and ``accumulate`` let callers
    sum parameter chunks in place; ``alpha`` folds a normalisation into the same
    pass.  With ``strict`` (default: env TRAK_B200_STRICT, on) the call waits for
    the kernels and raises if one of them gave up a bounded wait.  With
    ``allow_strided`` the rows may be further apart than their length (a column
    slice of a wider buffer); the six ``project_*`` entry points keep the
    reference's contiguity check.  With ``matrix`` (a ``StoredMatrix`` made for the
    same shape, seed, tile count, type and 16-bit gradient format) the matrix is
    read from device memory instead of being regenerated.
    """
    if not isinstance(input, torch.Tensor) or not input.is_cuda:
        raise RuntimeError("input must be a CUDA tensor")
    if input.dim() != 2:
        raise RuntimeError("input must be 2D")
    if not input.is_contiguous():
        if not (allow_strided and input.stride(1) == 1 and input.stride(0) >= input.shape[1]):
            raise RuntimeError("input must be contiguous")
    if input.dtype not in _DTYPES:
        raise RuntimeError("input must be fp16 or fp32 (bf16 is accepted as well)")
    N = _u32("N", N)
    seed = _u32("seed", seed)
    num_feature_tiles = _u32("num_feature_tiles", num_feature_tiles)
    B, F = input.shape
    if B == 0 or F == 0:
        raise RuntimeError("input must not be empty")
    l = _lib.lib()
    dev = input.device
    if out is None:
        out = torch.empty((B, N), dtype=torch.float32, device=dev)
        accumulate = False
    else:
        if out.device != dev or out.dtype != torch.float32 or out.dim() != 2 or out.shape[0] != B \
                or out.shape[1] != N or out.stride(1) != 1:
            raise RuntimeError("out must be a float32 [B, N] tensor on the input's device")
    dt = _DTYPES[input.dtype]
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        nbytes = l.tb_project_workspace_bytes(dt, B, F, N, max(num_feature_tiles, 1))
        ws = _workspace(dev, stream, max(nbytes, 256))
        if matrix is not None:
            if not matrix.matches(input, N, num_feature_tiles) or matrix.seed != seed or \
                    matrix.proj_type != int(proj_type):
                raise RuntimeError("the stored matrix was made for another shape, seed, type or gradient dtype")
            rc = l.tb_project_cached(dev.index, stream, input.data_ptr(), dt, B, F, input.stride(0), out.data_ptr(),
                                     out.stride(0), N, num_feature_tiles, matrix.data.data_ptr(), matrix.data.numel(),
                                     float(alpha), int(bool(accumulate)), ws.data_ptr(), ws.numel())
        else:
            rc = l.tb_project(dev.index, stream, input.data_ptr(), dt, B, F, input.stride(0),
                              out.data_ptr(), out.stride(0), N, seed, num_feature_tiles,
                              int(proj_type), float(alpha), int(bool(accumulate)), ws.data_ptr(),
                              ws.numel())
        _lib.check(rc)
        if _STRICT if strict is None else strict:
            _lib.device_status(dev.index)
    return out


def project_segments(tensors, N, seed, num_feature_tiles, proj_type, *, alpha=1.0, out=None, accumulate=False,
                     strict=None, matrix=None):
    """Projects the per-sample gradient whose sample b is the concatenation of ``t[b].reshape(-1)`` over
    ``tensors`` (a list of CUDA tensors ``[B, *shape]``, one dtype, each with contiguous samples) without
    first copying them into one ``[B, D]`` matrix.  A tensor with fewer than two dimensions contributes one
    feature per sample, as in the reference's ``vectorize`` (trak/utils.py:100-102).  Same result as
    ``project(torch.cat([t.reshape(B, -1) for t in tensors], 1), ...)``."""
    if not tensors:
        raise RuntimeError("no gradient tensors")
    first = tensors[0]
    B, dev, dtype = first.shape[0], first.device, first.dtype
    if dtype not in _DTYPES or not first.is_cuda:
        raise RuntimeError("gradients must be CUDA tensors of dtype fp16, bf16 or fp32")
    N = _u32("N", N)
    seed = _u32("seed", seed)
    num_feature_tiles = _u32("num_feature_tiles", num_feature_tiles)
    segs = (_lib.Segment * len(tensors))()
    keep = []
    F = 0
    for i, t in enumerate(tensors):
        if t.device != dev or t.dtype != dtype or t.shape[0] != B:
            raise RuntimeError("all gradient tensors must share device, dtype and batch size")
        flat = t.reshape(B, 1) if t.dim() < 2 else t.flatten(start_dim=1)
        if flat.shape[1] == 0:
            raise RuntimeError("empty parameter")
        if flat.stride(1) != 1 or (B > 1 and flat.stride(0) < flat.shape[1]):
            flat = flat.contiguous()
        keep.append(flat)
        segs[i].ptr = flat.data_ptr()
        segs[i].numel = flat.shape[1]
        segs[i].row_stride = flat.stride(0) if B > 1 else flat.shape[1]
        F += flat.shape[1]
    l = _lib.lib()
    if out is None:
        out = torch.empty((B, N), dtype=torch.float32, device=dev)
        accumulate = False
    elif out.device != dev or out.dtype != torch.float32 or tuple(out.shape) != (B, N) or out.stride(1) != 1:
        raise RuntimeError("out must be a float32 [B, N] tensor on the gradients' device")
    dt = _DTYPES[dtype]
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        nbytes = l.tb_project_segments_workspace_bytes(dt, B, F, N, max(num_feature_tiles, 1), len(tensors))
        ws = _workspace(dev, stream, max(nbytes, 256))
        if matrix is not None:
            elem = _lib.TB_BF16 if dtype == torch.bfloat16 else _lib.TB_F16
            if (matrix.F, matrix.N, matrix.tiles, matrix.elem, matrix.device) != (F, N, num_feature_tiles, elem, dev) \
                    or matrix.seed != seed or matrix.proj_type != int(proj_type):
                raise RuntimeError("the stored matrix was made for another shape, seed, type or gradient dtype")
            rc = l.tb_project_segments_cached(dev.index, stream, segs, len(tensors), dt, B, out.data_ptr(), out.stride(0),
                                              N, num_feature_tiles, matrix.data.data_ptr(), matrix.data.numel(),
                                              float(alpha), int(bool(accumulate)), ws.data_ptr(), ws.numel())
        else:
            rc = l.tb_project_segments(dev.index, stream, segs, len(tensors), dt, B, out.data_ptr(), out.stride(0), N,
                                       seed, num_feature_tiles, int(proj_type), float(alpha), int(bool(accumulate)),
                                       ws.data_ptr(), ws.numel())
        _lib.check(rc)
        if _STRICT if strict is None else strict:
            _lib.device_status(dev.index)
    return out


# ---- opt-in: keep the Gaussian matrix in device memory between calls of the six entry points -----------------
# The reference's CudaProjector calls project_normal_* once per batch with the same (seed, num_feature_tiles) for a
# whole checkpoint (trak/projectors.py:414-440).  With TRAK_B200_STORE_MATRIX=1 (or store_matrices(True)) the
# entry points generate that matrix once per device and read it afterwards (StoredMatrix), when it fits next to
# what the process already holds; otherwise, and for the Rademacher matrix (cheaper to regenerate than to read),
# nothing changes.
_store = os.environ.get("TRAK_B200_STORE_MATRIX", "0") not in ("", "0")
_stored = {}          # device index -> StoredMatrix (one per device: the matrices are tens of GB)
_does_not_fit = set()
_STORE_HEADROOM = 2 << 30   # bytes left to the caller after the matrix is allocated


def store_matrices(on: bool = True):
    """Turns the stored-matrix mode of ``project_normal_*`` on or off; off also frees the matrices."""
    global _store
    _store = bool(on)
    if not _store:
        _stored.clear()
        _does_not_fit.clear()


def _auto_matrix(input, N, seed, num_feature_tiles):
    if not (_store and isinstance(input, torch.Tensor) and input.is_cuda and input.dim() == 2
            and input.dtype in _DTYPES and input.shape[0] > 0 and input.shape[1] > 0):
        return None   # project() raises the reference's error for it
    dev = input.device
    elem = _lib.TB_BF16 if input.dtype == torch.bfloat16 else _lib.TB_F16
    key = (dev.index, input.shape[1], N, seed, num_feature_tiles, elem)
    m = _stored.get(dev.index)
    if m is not None and (dev.index, m.F, m.N, m.seed, m.tiles, m.elem) == key:
        return m
    if key in _does_not_fit:
        return None
    try:
        need = StoredMatrix.nbytes(input.shape[1], _u32("N", N), max(_u32("num_feature_tiles", num_feature_tiles), 1))
        _u32("seed", seed)
    except TypeError:
        return None
    if need == 0:
        return None
    _stored.pop(dev.index, None)
    m = None
    free, _ = torch.cuda.mem_get_info(dev)
    free += torch.cuda.memory_reserved(dev) - torch.cuda.memory_allocated(dev)   # blocks torch can reuse
    if len(_does_not_fit) > 64:
        _does_not_fit.clear()
    if need + _STORE_HEADROOM > free:
        _does_not_fit.add(key)
        return None
    try:
        m = StoredMatrix(input.shape[1], N, seed, num_feature_tiles, _lib.TB_NORMAL, dtype=input.dtype, device=dev)
    except torch.cuda.OutOfMemoryError:
        _does_not_fit.add(key)
        return None
    _stored[dev.index] = m
    return m


def project_rademacher_8(input, N, seed, num_feature_tiles):
    return project(input, N, seed, num_feature_tiles, _lib.TB_RADEMACHER)


def project_rademacher_16(input, N, seed, num_feature_tiles):
    return project(input, N, seed, num_feature_tiles, _lib.TB_RADEMACHER)


def project_rademacher_32(input, N, seed, num_feature_tiles):
    return project(input, N, seed, num_feature_tiles, _lib.TB_RADEMACHER)


def project_normal_8(input, N, seed, num_feature_tiles):
    return project(input, N, seed, num_feature_tiles, _lib.TB_NORMAL,
                   matrix=_auto_matrix(input, N, seed, num_feature_tiles))


def project_normal_16(input, N, seed, num_feature_tiles):
    return project(input, N, seed, num_feature_tiles, _lib.TB_NORMAL,
                   matrix=_auto_matrix(input, N, seed, num_feature_tiles))


def project_normal_32(input, N, seed, num_feature_tiles):
    return project(input, N, seed, num_feature_tiles, _lib.TB_NORMAL,
                   matrix=_auto_matrix(input, N, seed, num_feature_tiles))
