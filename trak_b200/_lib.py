"""ctypes binding of ``libtrakb200.so`` (the C ABI declared in ``include/trak_b200.h``).

There is no fallback: if the shared library is missing or a call fails, the
caller gets an exception.
"""
import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtrakb200.so")

TB_F16, TB_BF16, TB_F32 = 0, 1, 2
TB_RADEMACHER, TB_NORMAL = 0, 1
TB_OK = 0
TB_ERR_BAD_PROJ_DIM = 3
TB_ERR_DEVICE_TIMEOUT = 7
TB_ERR_NOT_SPD = 10

_lib = None
_lock = threading.Lock()

_i, _i64, _u32 = ctypes.c_int, ctypes.c_int64, ctypes.c_uint32
_vp, _sz, _f = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_float
_i32 = ctypes.c_int32


class Segment(ctypes.Structure):
    """tb_segment: one parameter's per-sample gradients ([B, numel], rows row_stride apart)."""
    _fields_ = [("ptr", ctypes.c_void_p), ("numel", ctypes.c_int64), ("row_stride", ctypes.c_int64)]


# name -> (restype, argtypes); one entry per function include/trak_b200.h declares
SIGNATURES = {
    "tb_version": (_i, []),
    "tb_strerror": (ctypes.c_char_p, [_i]),
    "tb_last_cuda_error": (ctypes.c_char_p, []),
    "tb_device_status": (_i, [_i, ctypes.POINTER(_u32)]),
    "tb_selftest_wait_timeout": (_i, [_i, _vp, _u32]),
    "tb_selftest_sqrt": (_i, [_i, _vp, ctypes.c_uint64, ctypes.c_uint64, _vp]),
    "tb_project_workspace_bytes": (_sz, [_i, _i64, _i64, _u32, _u32]),
    "tb_profile_events": (_i, [_vp, _vp]),
    "tb_project_segments_workspace_bytes": (_sz, [_i, _i64, _i64, _u32, _u32, _i32]),
    "tb_project_segments": (_i, [_i, _vp, ctypes.POINTER(Segment), _i32, _i, _i64, _vp, _i64, _u32, _u32, _u32,
                                 _i, _f, _i, _vp, _sz]),
    "tb_gram_workspace_bytes": (_sz, [_i, _i64, _i64]),
    "tb_gram": (_i, [_i, _vp, _vp, _i, _i64, _i64, _i64, _vp, _i64, _i, _vp, _sz]),
    "tb_spd_inverse_workspace_bytes": (_sz, [_i64]),
    "tb_spd_inverse": (_i, [_i, _vp, _vp, _i64, _i64, _f, _i, _vp, _vp, _sz]),
    "tb_gemm_nt_workspace_bytes": (_sz, [_i, _i64, _i64, _i64]),
    "tb_gemm_nt": (_i, [_i, _vp, _vp, _i64, _vp, _i64, _i, _i64, _i64, _i64, _vp, _i64, _vp, _f, _i, _vp, _sz]),
    "tb_matrix_bytes": (_sz, [_i64, _u32, _u32]),
    "tb_matrix_generate": (_i, [_i, _vp, _i64, _u32, _u32, _u32, _i, _i, _vp, _sz]),
    "tb_project_cached": (_i, [_i, _vp, _vp, _i, _i64, _i64, _i64, _vp, _i64, _u32, _u32, _vp, _sz, _f, _i, _vp, _sz]),
    "tb_project_segments_cached": (_i, [_i, _vp, ctypes.POINTER(Segment), _i32, _i, _i64, _vp, _i64, _u32, _u32, _vp,
                                        _sz, _f, _i, _vp, _sz]),
    "tb_finalize_scores": (_i, [_i, _vp, _vp, _i64, _vp, _i64, _i64, _f, _vp, _i, _i64]),
    "tb_project_static": (_i, [_i, _vp, _vp, _i, _i64, _i64, _i64, _vp, _i64, _u32, _u32, _u32, _i, _f, _i]),
    "tb_project": (_i, [_i, _vp, _vp, _i, _i64, _i64, _i64, _vp, _i64, _u32, _u32, _u32, _i, _f, _i,
                        _vp, _sz]),
}


def lib():
    """The loaded library.  Raises ImportError (with the build hint) when absent."""
    global _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise ImportError(
                    f"{LIB_PATH} not found: build it with `python -m trak_b200.build` "
                    "(needs nvcc; the kernels are sm_100a only and there is no CPU fallback)")
            l = ctypes.CDLL(LIB_PATH)
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(l, name)
                fn.restype = res
                fn.argtypes = args
            _lib = l
    return _lib


class DeviceTimeout(RuntimeError):
    pass


class NotPositiveDefinite(RuntimeError):
    """tb_spd_inverse met a non-positive Cholesky pivot (torch.linalg.inv of the reference would
    return garbage or raise on such a matrix)."""


def check(rc: int) -> None:
    """Maps a status code to the exception type the reference raises for it:
    ValueError for a bad projection dimension (std::invalid_argument in
    fast_jl/fast_jl_kernel.cuh:113-115), RuntimeError otherwise."""
    if rc == TB_OK:
        return
    l = lib()
    msg = l.tb_strerror(rc).decode()
    if rc == TB_ERR_BAD_PROJ_DIM:
        raise ValueError(msg)
    if rc == 6:
        msg = f"CUDA error: {l.tb_last_cuda_error().decode()}"
    if rc == TB_ERR_DEVICE_TIMEOUT:
        raise DeviceTimeout(msg)
    if rc == TB_ERR_NOT_SPD:
        raise NotPositiveDefinite(msg)
    raise RuntimeError(f"trak_b200: {msg} (code {rc})")


def device_status(device: int) -> None:
    """Synchronises the device and raises DeviceTimeout if a kernel gave up a wait."""
    detail = _u32(0)
    rc = lib().tb_device_status(device, ctypes.byref(detail))
    if rc == TB_ERR_DEVICE_TIMEOUT:
        raise DeviceTimeout(f"trak_b200: a bounded wait inside a kernel ran out (status {detail.value})")
    check(rc)
