"""tb_project_static: the projection for hosts that cannot allocate device memory (their
memory belongs to another component's pool, or they must avoid the device-wide
synchronisation of cudaMalloc / cudaFree).  Its scratch is a fixed array inside the library.

The tests drive the C ABI directly with ctypes: the workspace-free entry point must give
exactly what tb_project gives with a caller-provided workspace (same kernels, same fixed
summation order, so the comparison is bit for bit), on calls in a row (later ones reuse the
array with the earlier calls' bytes still in it), must not change the amount of free device
memory, and must refuse shapes whose scratch does not fit.  This file sorts last so that a run
stopping at the first failure has already run every other test.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 1e-3  # per row ||a - b|| / ||b|| against the fp64 oracle, the tolerance of the other projection tests
STATIC_BYTES = 32 * 1024 * 1024
CODES = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


def _with_workspace(lib, dev, g, N, seed, tiles, ptype, alpha=1.0, out=None):
    B, F = g.shape
    acc = out is not None
    if out is None:
        out = torch.empty(B, N, device=dev, dtype=torch.float32)
    dt = CODES[g.dtype]
    nbytes = lib.tb_project_workspace_bytes(dt, B, F, N, tiles)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    rc = lib.tb_project(dev.index, stream, g.data_ptr(), dt, B, F, g.stride(0), out.data_ptr(), N, N, seed,
                        tiles, ptype, alpha, int(acc), ws.data_ptr(), ws.numel())
    assert rc == 0, lib.tb_strerror(rc)
    torch.cuda.synchronize(dev)
    return out


def _static(lib, dev, g, N, seed, tiles, ptype, alpha=1.0, out=None):
    B, F = g.shape
    acc = out is not None
    if out is None:
        out = torch.empty(B, N, device=dev, dtype=torch.float32)
    stream = torch.cuda.current_stream(dev).cuda_stream
    rc = lib.tb_project_static(dev.index, stream, g.data_ptr(), CODES[g.dtype], B, F, g.stride(0), out.data_ptr(),
                               N, N, seed, tiles, ptype, alpha, int(acc))
    assert rc == 0, lib.tb_strerror(rc)
    torch.cuda.synchronize(dev)
    return out


def _grads(dev, B, F, dtype):
    g = torch.randn(B, F, device=dev, generator=torch.Generator(device=dev).manual_seed(F + B)) * 1e-2
    return g.to(dtype)


def test_static_scratch_projection_matches_workspace_projection(cuda):
    from trak_b200 import _lib
    lib = _lib.lib()
    # calls in a row with different shapes, dtypes, seeds and projection types
    cases = [(16, 50021, 1024, 17, 148, 0, torch.float16), (5, 9000, 512, 3, 108, 1, torch.float16),
             (12, 30011, 512, 5, 148, 1, torch.bfloat16), (9, 20000, 1024, 9, 64, 0, torch.float32)]
    for B, F, N, seed, tiles, ptype, dtype in cases:
        assert lib.tb_project_workspace_bytes(CODES[dtype], B, F, N, tiles) <= STATIC_BYTES
        g = _grads(cuda, B, F, dtype)
        got = _static(lib, cuda, g, N, seed, tiles, ptype)
        want = _with_workspace(lib, cuda, g, N, seed, tiles, ptype)
        assert torch.equal(got, want)
    # and the first shape once more, now over the other calls' leftovers
    B, F, N, seed, tiles, ptype, dtype = cases[0]
    g = _grads(cuda, B, F, dtype)
    assert torch.equal(_static(lib, cuda, g, N, seed, tiles, ptype),
                       _with_workspace(lib, cuda, g, N, seed, tiles, ptype))
    _lib.device_status(cuda.index)


def test_static_scratch_many_rows_accumulate_and_scale(cuda):
    """More rows than one pass takes (the array is reused pass after pass inside the call), fp32 input,
    alpha != 1 and accumulation into an existing result; also checked against the CPU oracle."""
    from oracle import jl_oracle as o
    from trak_b200 import _lib
    lib = _lib.lib()
    B, F, N, seed, tiles, alpha = 300, 3001, 512, 21, 37, 0.25
    assert lib.tb_project_workspace_bytes(2, B, F, N, tiles) <= STATIC_BYTES
    g = _grads(cuda, B, F, torch.float32)
    base = torch.randn(B, N, device=cuda, generator=torch.Generator(device=cuda).manual_seed(1))
    for ptype in (0, 1):
        got = _static(lib, cuda, g, N, seed, tiles, ptype, alpha=alpha, out=base.clone())
        want = _with_workspace(lib, cuda, g, N, seed, tiles, ptype, alpha=alpha, out=base.clone())
        assert torch.equal(got, want)
        # the kernels round fp32 gradients to fp16 on the way in (fast_jl/data_loading.cuh:10)
        ref = alpha * o.project(ptype, g.half().cpu().numpy(), N, seed, tiles) + base.double().cpu().numpy()
        err = np.linalg.norm(got.double().cpu().numpy() - ref, axis=1) / np.linalg.norm(ref, axis=1)
        assert err.max() <= TOL
    _lib.device_status(cuda.index)


def test_static_scratch_call_leaves_free_device_memory_unchanged(cuda):
    from trak_b200 import _lib
    lib = _lib.lib()
    B, F, N = 16, 50021, 1024
    g = _grads(cuda, B, F, torch.float16)
    out = torch.empty(B, N, device=cuda, dtype=torch.float32)
    stream = torch.cuda.current_stream(cuda).cuda_stream

    def call():
        rc = lib.tb_project_static(cuda.index, stream, g.data_ptr(), 0, B, F, F, out.data_ptr(), N, N, 17, 148, 0,
                                   1.0, 0)
        assert rc == 0, lib.tb_strerror(rc)
        torch.cuda.synchronize(cuda)

    call()  # the one-time set-up of this device (address look-up, kernel loading) happens here
    free_before, _ = torch.cuda.mem_get_info(cuda)
    for _ in range(3):
        call()
    free_after, _ = torch.cuda.mem_get_info(cuda)
    assert free_after == free_before


def test_static_scratch_refuses_shapes_beyond_its_limit(cuda):
    from trak_b200 import _lib
    lib = _lib.lib()
    B, F, N = 128, 2_000_000, 4096
    assert lib.tb_project_workspace_bytes(0, B, F, N, 148) > STATIC_BYTES
    g = torch.zeros(4, device=cuda)  # never read: the call is refused on the host
    rc = lib.tb_project_static(cuda.index, None, g.data_ptr(), 0, B, F, F, g.data_ptr(), N, N, 0, 148, 0, 1.0, 0)
    assert rc == 9
    assert b"scratch" in lib.tb_strerror(rc)
