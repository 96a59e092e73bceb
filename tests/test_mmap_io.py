"""Row-range I/O on the reference's on-disk stores: files written here must be byte-identical to
what the unmodified MmapSaver writes (fixtures from tests/golden/make_mmapsaver_golden.py), and
files written by the reference must read back exactly."""
import os

import numpy as np
import pytest
import torch

from trak_b200 import mmap_io

N, K, M = 6, 8, 3


def _values(shape, dtype, offset=0.0):
    return (np.arange(np.prod(shape), dtype=np.float64).reshape(shape) / 8.0 - 2.0 + offset).astype(dtype)


CASES = [("grads", (N, K), 0.0), ("features", (N, K), 0.5), ("out_to_loss", (N, 1), 1.0), ("scores", (N, M), 0.25)]


@pytest.mark.parametrize("tag,tdt,ndt", [("f16", torch.float16, np.float16), ("f32", torch.float32, np.float32)])
@pytest.mark.parametrize("name,shape,offset", CASES)
def test_files_are_byte_identical_to_the_reference_saver(tmp_path, golden_dir, tag, tdt, ndt, name, shape, offset):
    want = open(os.path.join(golden_dir, f"mmapsaver_{name}_{tag}.mmap"), "rb").read()
    path = tmp_path / "0" / f"{name}.mmap"
    store = mmap_io.create_store(path, shape, tdt)
    vals = torch.from_numpy(_values(shape, ndt, offset))
    # written as two row ranges, out of order, through a 2-row staging buffer
    stager = mmap_io.PinnedStager(shape[1], tdt, chunk_rows=2)
    mmap_io.write_rows(store, 4, vals[4:], stager)
    mmap_io.write_rows(store, 0, vals[:4].double(), stager)   # cast to the file's dtype on the way
    store.flush()
    del store
    assert open(path, "rb").read() == want


@pytest.mark.parametrize("tag,ndt", [("f16", np.float16), ("f32", np.float32)])
def test_reads_reference_files(golden_dir, tag, ndt):
    store = mmap_io.open_store(os.path.join(golden_dir, f"mmapsaver_grads_{tag}.mmap"), mode="r")
    assert store.shape == (N, K) and store.dtype == ndt
    full = _values((N, K), ndt)
    got = mmap_io.read_rows(store, 1, 5, "cpu", mmap_io.PinnedStager(K, torch.float16 if tag == "f16" else torch.float32, 3))
    assert np.array_equal(got.numpy(), full[1:5])
    assert mmap_io.read_rows(store, 2, 2, "cpu").shape == (0, K)
    with pytest.raises(ValueError):
        mmap_io.read_rows(store, 0, N + 1, "cpu")


def test_write_rejects_mismatched_rows(tmp_path):
    store = mmap_io.create_store(tmp_path / "x.mmap", (4, 3), torch.float32)
    with pytest.raises(ValueError):
        mmap_io.write_rows(store, 3, torch.zeros(2, 3))
    with pytest.raises(ValueError):
        mmap_io.write_rows(store, 0, torch.zeros(2, 4))


@pytest.mark.gpu
def test_row_ranges_through_the_gpu(cuda, tmp_path):
    n, k = 5000, 96
    x = torch.randn(n, k, generator=torch.Generator().manual_seed(0)).half()
    store = mmap_io.create_store(tmp_path / "0" / "grads.mmap", (n, k), torch.float16)
    mmap_io.write_rows(store, 0, x.to(cuda), mmap_io.PinnedStager(k, torch.float16, 700))
    store.flush()
    again = mmap_io.open_store(tmp_path / "0" / "grads.mmap", mode="r")
    part = mmap_io.read_rows(again, 1234, 4321, cuda, mmap_io.PinnedStager(k, torch.float16, 999))
    assert part.device.type == "cuda" and torch.equal(part.cpu(), x[1234:4321])
    # per-shard Gram straight from the store
    g = mmap_io.gram_of_store(again, 1000, 3000, cuda, block_rows=512)
    ref = x[1000:3000].double().T @ x[1000:3000].double()
    assert float((g.double().cpu() - ref).norm() / ref.norm()) < 1e-4
