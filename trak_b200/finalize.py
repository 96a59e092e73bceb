"""``finalize_scores`` for any number of checkpoints, with the accumulation and the epilogue on the GPU.

The reference (trak/traker.py:632-684) keeps a host accumulator ``[n_train, n_targets]`` (40 GB for
a million train examples and ten thousand targets), adds every checkpoint's
``features @ target_grads.T`` into it with a host ``+=`` per GPU block
(trak/score_computers.py:179-189), sums the checkpoints' out-to-loss weights, and finally runs
``(sum_scores / M) * (sum_out_to_loss / M)`` with numpy over the whole array before writing it to
``scores/<exp>.mmap`` (trak/savers.py:434-451).

Here the loop is turned inside out: train rows are walked in blocks, and for one block

* every checkpoint's product is accumulated in ONE device buffer (``tb_gemm_nt`` with
  ``accumulate``), the checkpoints' feature rows arriving from their stores through pinned staging;
* the checkpoints' out-to-loss weights of the block are summed on the device;
* ``tb_finalize_scores`` applies ``(sum / M) * (sum_w / M)`` and casts to the store's dtype;
* the finished block leaves the GPU once, through one of two pinned buffers, and the host writes it
  into the memmap while the GPU works on the next block.

No host array of the full size exists, every score crosses PCIe once, finished, and the host does
one ``memcpy`` per block.  A rank that owns the train rows ``[lo, hi)`` finalizes only those.
"""
import numpy as np
import torch

from . import _lib, mmap_io
from . import score_computers as sc

_CODE = {torch.float16: _lib.TB_F16, torch.float32: _lib.TB_F32}


def finalize_scores_block(score_sum: torch.Tensor, out_to_loss_sum: torch.Tensor, num_models: int,
                          out: torch.Tensor = None, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """``(score_sum / M) * (out_to_loss_sum / M)[:, None]`` on the GPU for one row block
    (trak/traker.py:676-678).  ``score_sum`` fp32 CUDA ``[n, m]``, ``out_to_loss_sum`` ``[n]`` or ``[n, 1]``;
    the result is fp32 or fp16."""
    if not score_sum.is_cuda or score_sum.dtype != torch.float32 or score_sum.dim() != 2 or score_sum.stride(1) != 1:
        raise RuntimeError("score_sum must be a CUDA fp32 matrix with unit column stride")
    n, m = score_sum.shape
    dev = score_sum.device
    w = out_to_loss_sum.to(dev, torch.float32).reshape(-1).contiguous()
    if w.numel() != n:
        raise RuntimeError("out_to_loss_sum must have one entry per row of score_sum")
    if out is None:
        out = torch.empty((n, m), dtype=dtype, device=dev)
    if out.dtype not in _CODE or out.device != dev or tuple(out.shape) != (n, m) or out.stride(1) != 1:
        raise RuntimeError("out must be an fp16 or fp32 [n, m] tensor on score_sum's device")
    if n == 0 or m == 0:
        return out
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        _lib.check(_lib.lib().tb_finalize_scores(dev.index, stream, score_sum.data_ptr(), score_sum.stride(0),
                                                 w.data_ptr(), n, m, float(num_models), out.data_ptr(),
                                                 _CODE[out.dtype], out.stride(0)))
    return out


def _rows_to_device(src, lo, hi, device, stager):
    """Rows [lo, hi) of a feature store (numpy memmap / array, CPU or CUDA tensor) as a CUDA matrix."""
    if isinstance(src, torch.Tensor):
        return sc._as_device_matrix(src[lo:hi], device)
    return sc._as_device_matrix(mmap_io.read_rows(src, lo, hi, device, stager), device)


def _whole_to_device(src, device):
    if isinstance(src, torch.Tensor):
        return sc._as_device_matrix(src, device)
    return sc._as_device_matrix(torch.from_numpy(np.array(src)), device)   # a copy: the store may be read-only


class ScoreFinalizer:
    """Streams ``finalize_scores`` through one GPU.

    ``features``      one ``[n_train, k]`` store per checkpoint (``features.mmap`` opened with
                      ``mmap_io.open_store``, a numpy array, or a CPU / CUDA tensor)
    ``target_grads``  one ``[n_targets, k]`` store per checkpoint (``<exp>_grads.mmap``)
    ``out_to_loss``   one ``[n_train, 1]`` store per checkpoint (``out_to_loss.mmap``)

    ``run(scores_store, rows=(lo, hi))`` writes the finished rows into ``scores_store`` (the
    ``scores/<exp>.mmap`` memmap, fp16 or fp32, or a CPU tensor) and returns it.
    """

    STAGE_BYTES = 256 << 20  # each of the two pinned buffers the finished blocks leave through

    def __init__(self, features, target_grads, out_to_loss, device, row_block: int = 65_536):
        if not (len(features) == len(target_grads) == len(out_to_loss)) or len(features) == 0:
            raise ValueError("one feature store, one target-gradient store and one out-to-loss store per checkpoint")
        device = torch.device(device)
        if device.type != "cuda":
            raise ValueError("ScoreFinalizer only works on a CUDA device")
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self.device = device
        self.features, self.out_to_loss = list(features), list(out_to_loss)
        self.num_models = len(features)
        self.n_train = int(features[0].shape[0])
        # the targets are small ([m, k] per checkpoint): resident for the whole run
        self.targets = [_whole_to_device(t, device) for t in target_grads]
        self.n_targets = int(self.targets[0].shape[0])
        for f, t, w in zip(self.features, self.targets, self.out_to_loss):
            if f.shape[0] != self.n_train or w.shape[0] != self.n_train or t.shape[0] != self.n_targets \
                    or f.shape[1] != t.shape[1]:
                raise ValueError("stores of the checkpoints do not agree in shape")
        self.row_block = max(256, row_block)
        _lib.lib()

    def run(self, scores_store, rows=None):
        lo, hi = (0, self.n_train) if rows is None else rows
        if not (0 <= lo <= hi <= self.n_train):
            raise ValueError("row range outside the train set")
        if tuple(scores_store.shape) != (self.n_train, self.n_targets):
            raise ValueError("scores store must be [n_train, n_targets]")
        is_tensor = isinstance(scores_store, torch.Tensor)
        out_dtype = scores_store.dtype if is_tensor else mmap_io._TORCH[scores_store.dtype]
        if out_dtype not in _CODE:
            raise ValueError("scores store must be fp16 or fp32")
        dev, m, M = self.device, self.n_targets, self.num_models
        esize = 2 if out_dtype == torch.float16 else 4
        step = max(256, min(self.row_block, self.STAGE_BYTES // (esize * m) // 256 * 256))
        step = min(step, max(1, hi - lo))
        with torch.cuda.device(dev):
            acc = torch.empty(step, m, dtype=torch.float32, device=dev)
            done = torch.empty(step, m, dtype=out_dtype, device=dev)
            stage = [torch.empty(step, m, dtype=out_dtype).pin_memory() for _ in range(2)]
            stagers = {}
            pending = None

            def flush(item):
                r0, nrows, buf, event = item
                event.synchronize()
                if is_tensor:
                    scores_store[r0:r0 + nrows] = buf[:nrows]
                else:
                    scores_store[r0:r0 + nrows] = buf[:nrows].numpy()

            for i, r0 in enumerate(range(lo, hi, step)):
                r1 = min(hi, r0 + step)
                nrows = r1 - r0
                w_sum = torch.zeros(nrows, dtype=torch.float32, device=dev)
                for j in range(M):
                    src = self.features[j]
                    stager = None
                    if not isinstance(src, torch.Tensor):
                        key = (src.dtype, src.shape[1])
                        if key not in stagers:
                            stagers[key] = mmap_io.PinnedStager(src.shape[1], mmap_io._TORCH[np.dtype(src.dtype)],
                                                                min(16384, step))
                        stager = stagers[key]
                    blk = _rows_to_device(src, r0, r1, dev, stager)
                    tg = self.targets[j]
                    if tg.dtype != blk.dtype:
                        wide = torch.promote_types(tg.dtype, blk.dtype)
                        blk, tg = blk.to(wide), tg.to(wide)
                    sc.gemm_nt(blk, tg, out=acc[:nrows], accumulate=j > 0)
                    wj = self.out_to_loss[j]
                    wj = wj[r0:r1] if isinstance(wj, torch.Tensor) else torch.from_numpy(np.array(wj[r0:r1]))
                    w_sum += wj.to(dev, torch.float32, non_blocking=True).reshape(-1)
                finalize_scores_block(acc[:nrows], w_sum, M, out=done[:nrows])
                # buffer i % 2 was last read by the flush of block i - 2, which has returned
                buf = stage[i % 2]
                buf[:nrows].copy_(done[:nrows], non_blocking=True)
                event = torch.cuda.Event()
                event.record(torch.cuda.current_stream(dev))
                if pending is not None:
                    flush(pending)
                pending = (r0, nrows, buf, event)
            if pending is not None:
                flush(pending)
            _lib.device_status(dev.index)
        if not is_tensor and hasattr(scores_store, "flush"):
            scores_store.flush()
        return scores_store
