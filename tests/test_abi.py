"""The C-ABI library loads without a GPU, exports every symbol the header declares,
and rejects bad arguments with the documented codes before touching a device."""
import ctypes
import os
import re

import pytest

from trak_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "trak_b200.h")


def _declared():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(tb_[a-z0-9_]+)\s*\(", src)))


def test_header_symbols_are_exported_and_bound():
    lib = _lib.lib()
    names = _declared()
    assert "tb_project" in names and "tb_version" in names
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/trak_b200.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature in trak_b200/_lib.py"
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_error_text():
    lib = _lib.lib()
    assert lib.tb_version() >= 100
    assert lib.tb_strerror(0) == b"ok"
    assert b"multiple of 512" in lib.tb_strerror(_lib.TB_ERR_BAD_PROJ_DIM)
    assert lib.tb_strerror(12345) == b"unknown error code"


def test_project_workspace_query():
    lib = _lib.lib()
    assert lib.tb_project_workspace_bytes(0, 0, 10, 512, 148) == 0
    small = lib.tb_project_workspace_bytes(0, 8, 1000, 512, 148)
    big = lib.tb_project_workspace_bytes(0, 128, 11173962, 4096, 148)
    assert 0 < small < big
    # staged copy (128 rows x 148 tiles x 75520 padded features x 2 B) + partials
    assert big >= 128 * 148 * 75520 * 2
    # batches are walked at most 512 rows at a time: the workspace stops growing there
    big256 = lib.tb_project_workspace_bytes(0, 256, 11173962, 4096, 148)
    big512 = lib.tb_project_workspace_bytes(0, 512, 11173962, 4096, 148)
    assert big < big256 <= 2 * big and big256 < big512 <= 2 * big256
    assert lib.tb_project_workspace_bytes(0, 1024, 11173962, 4096, 148) == big512
    # passes of more than 256 rows are padded to a multiple of 32 rows, smaller ones to 16
    assert lib.tb_project_workspace_bytes(0, 257, 11173962, 4096, 148) >= 288 * 148 * 75520 * 2


def _call(**kw):
    lib = _lib.lib()
    a = dict(device=0, stream=None, grads=0x1000, dtype=0, B=8, F=1000, ld=1000, out=0x2000, ld_out=512,
             N=512, seed=0, tiles=148, ptype=0, alpha=1.0, acc=0, ws=0x10000, ws_bytes=1 << 40)
    a.update(kw)
    return lib.tb_project(a["device"], a["stream"], a["grads"], a["dtype"], a["B"], a["F"], a["ld"],
                          a["out"], a["ld_out"], a["N"], a["seed"], a["tiles"], a["ptype"], a["alpha"],
                          a["acc"], a["ws"], a["ws_bytes"])


@pytest.mark.parametrize("kw,code", [
    (dict(dtype=7), 1),
    (dict(B=0), 2), (dict(F=0), 2), (dict(ld=999), 2), (dict(ld_out=100), 2), (dict(tiles=0), 2),
    (dict(N=500), 3), (dict(N=0), 3), (dict(N=256), 3),
    (dict(grads=None), 4), (dict(out=None), 4), (dict(ptype=2), 4), (dict(out=0x2004), 4),
    (dict(ws=None), 5), (dict(ws=0x10010), 5), (dict(ws_bytes=16), 5),
])
def test_project_argument_validation(kw, code):
    # all of these are rejected on the host, before any CUDA call
    assert _call(**kw) == code


@pytest.mark.parametrize("kw,code", [
    (dict(dtype=7), 1), (dict(B=0), 2), (dict(ld=999), 2), (dict(N=500), 3), (dict(N=500, F=10 ** 9, ld=10 ** 9), 3),
    (dict(grads=None), 4), (dict(out=0x2004), 4), (dict(ptype=2), 4),
    (dict(B=128, F=2_000_000, ld=2_000_000, N=4096, ld_out=4096), 9),
])
def test_static_entry_validates_like_tb_project_before_touching_a_device(kw, code):
    # same codes as tb_project for bad arguments, then the scratch limit; all on the host
    lib = _lib.lib()
    a = dict(device=0, stream=None, grads=0x1000, dtype=0, B=8, F=1000, ld=1000, out=0x2000, ld_out=512,
             N=512, seed=0, tiles=148, ptype=0, alpha=1.0, acc=0)
    a.update(kw)
    assert lib.tb_project_static(a["device"], a["stream"], a["grads"], a["dtype"], a["B"], a["F"], a["ld"], a["out"],
                                 a["ld_out"], a["N"], a["seed"], a["tiles"], a["ptype"], a["alpha"], a["acc"]) == code


def test_check_maps_codes_to_reference_exception_types():
    with pytest.raises(ValueError, match="multiple of 512"):
        _lib.check(3)
    with pytest.raises(RuntimeError):
        _lib.check(2)
    with pytest.raises(_lib.DeviceTimeout):
        _lib.check(7)
    _lib.check(0)


def test_scoring_workspace_queries_and_validation():
    lib = _lib.lib()
    assert lib.tb_gram_workspace_bytes(2, 0, 10) == 0
    # packed X^T: k rows x n, bf16 hi + lo planes = 4 bytes per element (rounded up to 128 x 32 tiles)
    assert lib.tb_gram_workspace_bytes(2, 65536, 8192) >= 65536 * 8192 * 4
    assert lib.tb_gram_workspace_bytes(0, 65536, 8192) >= 65536 * 8192 * 2
    assert lib.tb_gemm_nt_workspace_bytes(2, 1000, 500, 64) >= (1024 + 512) * 64 * 4
    assert lib.tb_spd_inverse_workspace_bytes(8192) >= 8192 * 8192 * 4
    big = 1 << 40
    # rejected on the host, before any CUDA call
    assert lib.tb_gram(0, None, 0x1000, 9, 10, 10, 10, 0x2000, 10, 0, 0x10000, big) == 1     # dtype
    assert lib.tb_gram(0, None, 0x1000, 2, 10, 10, 5, 0x2000, 10, 0, 0x10000, big) == 2      # ld < k
    assert lib.tb_gram(0, None, None, 2, 10, 10, 10, 0x2000, 10, 0, 0x10000, big) == 4       # null input
    assert lib.tb_gram(0, None, 0x1000, 2, 10, 10, 10, 0x2000, 10, 0, None, big) == 5        # no workspace
    assert lib.tb_spd_inverse(0, None, 0x1000, 0, 10, 0.0, 1, None, 0x10000, big) == 2
    assert lib.tb_spd_inverse(0, None, None, 10, 10, 0.0, 1, None, 0x10000, big) == 4
    assert lib.tb_spd_inverse(0, None, 0x1000, 10, 10, 0.0, 1, None, 0x10000, 16) == 5
    assert lib.tb_gemm_nt(0, None, 0x1000, 8, 0x2000, 8, 2, 4, 4, 8, 0x3000, 2, None, 1.0, 0, 0x10000, big) == 2  # ldc < N
    assert lib.tb_gemm_nt(0, None, 0x1000, 8, None, 8, 2, 4, 4, 8, 0x3000, 4, None, 1.0, 0, 0x10000, big) == 4


def test_segment_table_validation():
    lib = _lib.lib()
    segs = (_lib.Segment * 2)()
    segs[0].ptr, segs[0].numel, segs[0].row_stride = 0x1000, 10, 10
    segs[1].ptr, segs[1].numel, segs[1].row_stride = 0x2000, 5, 4          # stride < numel
    big = 1 << 40
    assert lib.tb_project_segments(0, None, segs, 2, 0, 4, 0x3000, 512, 512, 0, 148, 0, 1.0, 0, 0x10000, big) == 2
    segs[1].row_stride = 5
    assert lib.tb_project_segments(0, None, segs, 0, 0, 4, 0x3000, 512, 512, 0, 148, 0, 1.0, 0, 0x10000, big) == 4
    assert lib.tb_project_segments(0, None, segs, 2, 0, 4, 0x3000, 512, 500, 0, 148, 0, 1.0, 0, 0x10000, big) == 3
    assert lib.tb_project_segments_workspace_bytes(0, 4, 15, 512, 148, 2) > lib.tb_project_workspace_bytes(0, 4, 15, 512, 148)
