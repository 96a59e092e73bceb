"""tb_project_static: the projection for hosts that cannot allocate device memory (their
memory belongs to another component's pool, or they must avoid the device-wide
synchronisation of cudaMalloc / cudaFree).  Its scratch is a fixed array inside the library.

The test drives the C ABI directly with ctypes: the workspace-free entry point must give
what tb_project gives with a caller-provided workspace, on two calls in a row (the second
reuses the array with the first call's bytes still in it), and must refuse shapes whose
scratch does not fit.  This file sorts last so that a run stopping at the first failure
has already run every other test.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 1e-3  # per row ||a - b|| / ||b||, the tolerance of the other projection tests
STATIC_BYTES = 32 * 1024 * 1024


def _rel_rows(a, b):
    a = a.double().cpu().numpy()
    b = b.double().cpu().numpy()
    return float((np.linalg.norm(a - b, axis=1) / np.maximum(np.linalg.norm(b, axis=1), 1e-30)).max())


def _with_workspace(lib, dev, g, N, seed, tiles, ptype):
    B, F = g.shape
    out = torch.empty(B, N, device=dev, dtype=torch.float32)
    nbytes = lib.tb_project_workspace_bytes(0, B, F, N, tiles)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    rc = lib.tb_project(dev.index, stream, g.data_ptr(), 0, B, F, g.stride(0), out.data_ptr(), N, N, seed,
                        tiles, ptype, 1.0, 0, ws.data_ptr(), ws.numel())
    assert rc == 0, lib.tb_strerror(rc)
    torch.cuda.synchronize(dev)
    return out


def _static(lib, dev, g, N, seed, tiles, ptype):
    B, F = g.shape
    out = torch.empty(B, N, device=dev, dtype=torch.float32)
    stream = torch.cuda.current_stream(dev).cuda_stream
    rc = lib.tb_project_static(dev.index, stream, g.data_ptr(), 0, B, F, g.stride(0), out.data_ptr(), N, N,
                               seed, tiles, ptype, 1.0, 0)
    assert rc == 0, lib.tb_strerror(rc)
    torch.cuda.synchronize(dev)
    return out


def test_static_scratch_projection_matches_workspace_projection(cuda):
    from trak_b200 import _lib
    lib = _lib.lib()
    # two calls in a row with different shapes, seeds and projection types
    cases = [(16, 50021, 1024, 17, 148, 0), (5, 9000, 512, 3, 108, 1)]
    for B, F, N, seed, tiles, ptype in cases:
        assert lib.tb_project_workspace_bytes(0, B, F, N, tiles) <= STATIC_BYTES
        g = (torch.randn(B, F, device=cuda, generator=torch.Generator(device=cuda).manual_seed(F)) * 1e-2).half()
        got = _static(lib, cuda, g, N, seed, tiles, ptype)
        want = _with_workspace(lib, cuda, g, N, seed, tiles, ptype)
        assert _rel_rows(got, want) <= TOL
    # and the first shape once more, now over the second call's leftovers
    B, F, N, seed, tiles, ptype = cases[0]
    g = (torch.randn(B, F, device=cuda, generator=torch.Generator(device=cuda).manual_seed(F)) * 1e-2).half()
    assert _rel_rows(_static(lib, cuda, g, N, seed, tiles, ptype),
                     _with_workspace(lib, cuda, g, N, seed, tiles, ptype)) <= TOL
    _lib.device_status(cuda.index)


def test_static_scratch_refuses_shapes_beyond_its_limit(cuda):
    from trak_b200 import _lib
    lib = _lib.lib()
    B, F, N = 128, 2_000_000, 4096
    assert lib.tb_project_workspace_bytes(0, B, F, N, 148) > STATIC_BYTES
    g = torch.zeros(1, device=cuda)  # never read: the call is refused on the host
    rc = lib.tb_project_static(cuda.index, None, g.data_ptr(), 0, B, F, F, g.data_ptr(), N, N, 0, 148, 0, 1.0, 0)
    assert rc == 9
    assert b"scratch" in lib.tb_strerror(rc)
