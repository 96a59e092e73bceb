"""Row-range I/O between the reference's on-disk stores and a GPU.

``MmapSaver`` (trak/savers.py:363-442) keeps every array of a checkpoint in a numpy
``.npy`` memmap created with ``numpy.lib.format.open_memmap`` -- ``grads.mmap``,
``features.mmap``, ``out_to_loss.mmap``, ``<exp>_grads.mmap`` under
``save_dir/<model_id>/`` and ``scores/<exp>.mmap`` -- fp16 or fp32, row-major, one row per
example.  ``TRAKer`` moves whole arrays at once (``ch.as_tensor(memmap, device=...)``,
trak/traker.py:480-486,662-665) and writes results back through a pageable ``.cpu()``.

The helpers here read and write *row ranges* of those same files, so a rank that owns the
train rows ``[lo, hi)`` touches only its part, and they go through a reusable pair of pinned
staging buffers in chunks, the host side of one chunk overlapping the device copy of the next.  The files stay byte-compatible with the reference: they are opened with
the same numpy call, nothing else is written.
"""
import os

import numpy as np
import torch
from numpy.lib.format import open_memmap

_NP = {torch.float16: np.float16, torch.float32: np.float32, torch.int32: np.int32}
_TORCH = {np.dtype(v): k for k, v in _NP.items()}


def create_store(path, shape, dtype=torch.float16) -> np.memmap:
    """A new, zero-filled store with the reference's layout (mode ``w+``)."""
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    return open_memmap(filename=str(path), mode="w+", shape=tuple(shape), dtype=_NP[dtype])


def open_store(path, mode="r+") -> np.memmap:
    """An existing store; shape and dtype come from its npy header."""
    return open_memmap(filename=str(path), mode=mode)


class PinnedStager:
    """Two pinned host buffers of ``chunk_rows`` rows each, reused for every transfer of one store.
    While the GPU copies chunk i out of (or into) one buffer, the host fills (or drains) the other:
    each buffer carries the CUDA event of its last device-side use, and only that event is waited
    for, never the whole stream."""

    def __init__(self, row_len: int, dtype: torch.dtype, chunk_rows: int = 16384):
        self.chunk_rows = max(1, chunk_rows)
        pin = torch.cuda.is_available()
        self.bufs = [torch.empty((self.chunk_rows, row_len), dtype=dtype) for _ in range(2)]
        if pin:
            self.bufs = [b.pin_memory() for b in self.bufs]
        self.events = [None, None]
        self.turn = 0

    @property
    def buf(self):  # first buffer (kept for callers that stage by hand)
        return self.bufs[0]

    def acquire(self):
        """The next buffer, once the device is done with what was last staged in it."""
        i = self.turn
        self.turn ^= 1
        if self.events[i] is not None:
            self.events[i].synchronize()
            self.events[i] = None
        return i, self.bufs[i]

    def mark(self, i, device):
        """Records that the copy just enqueued on ``device``'s current stream uses buffer i."""
        dev = torch.device(device)
        if dev.type == "cuda":
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(dev))
            self.events[i] = ev


def read_rows(store: np.memmap, lo: int, hi: int, device, stager: PinnedStager = None) -> torch.Tensor:
    """Rows ``[lo, hi)`` of a 2-D store as a tensor on ``device`` (dtype of the file).  The host-side
    read of one chunk overlaps the host-to-device copy of the previous one."""
    if store.ndim != 2 or not (0 <= lo <= hi <= store.shape[0]):
        raise ValueError("row range outside the store")
    dtype = _TORCH[store.dtype]
    out = torch.empty((hi - lo, store.shape[1]), dtype=dtype, device=device)
    if stager is None:
        stager = PinnedStager(store.shape[1], dtype, min(16384, max(1, hi - lo)))
    for r0 in range(lo, hi, stager.chunk_rows):
        r1 = min(hi, r0 + stager.chunk_rows)
        i, buf = stager.acquire()
        host = buf[: r1 - r0]
        host.numpy()[...] = store[r0:r1]
        out[r0 - lo:r1 - lo].copy_(host, non_blocking=True)
        stager.mark(i, device)
    return out


def write_rows(store: np.memmap, lo: int, values: torch.Tensor, stager: PinnedStager = None) -> None:
    """Writes ``values`` (any device; cast to the file's dtype) to rows ``[lo, lo + len)``.  The
    device-to-host copy of one chunk overlaps the host-side write of the previous one."""
    n = values.shape[0]
    if store.ndim != 2 or values.dim() != 2 or values.shape[1] != store.shape[1] or lo < 0 \
            or lo + n > store.shape[0]:
        raise ValueError("row range or row length does not match the store")
    dtype = _TORCH[store.dtype]
    if stager is None:
        stager = PinnedStager(store.shape[1], dtype, min(16384, max(1, n)))
    pending = None  # (buffer index, first row, rows) whose copy has been enqueued but not yet written out

    def drain(item):
        i, r0, rows = item
        if stager.events[i] is not None:
            stager.events[i].synchronize()
            stager.events[i] = None
        store[lo + r0:lo + r0 + rows] = stager.bufs[i][:rows].numpy()

    for r0 in range(0, n, stager.chunk_rows):
        r1 = min(n, r0 + stager.chunk_rows)
        i, buf = stager.acquire()
        buf[: r1 - r0].copy_(values[r0:r1], non_blocking=True)  # casts to the file's dtype on the way
        stager.mark(i, values.device)
        if pending is not None:
            drain(pending)
        pending = (i, r0, r1 - r0)
    if pending is not None:
        drain(pending)


def gram_of_store(store: np.memmap, lo: int, hi: int, device, block_rows: int = 65536) -> torch.Tensor:
    """fp32 ``X[lo:hi]^T X[lo:hi]`` of a ``grads.mmap``, streamed block by block through the GPU
    (the per-rank part of ``get_xtx`` when the train rows are sharded)."""
    from . import score_computers as sc
    acc = None
    stager = PinnedStager(store.shape[1], _TORCH[store.dtype], min(block_rows, 16384))
    for r0 in range(lo, hi, block_rows):
        blk = read_rows(store, r0, min(hi, r0 + block_rows), device, stager)
        acc = sc.gram(blk, out=acc, accumulate=acc is not None)
    return acc
