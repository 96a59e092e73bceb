"""Score computer with the reference's interface, running on the sm_100a kernels.

Mirrors ``BasicScoreComputer`` (trak/score_computers.py:114-189): same constructor
arguments, same three methods, same shapes and dtypes of the results, so it can be
passed to an unmodified ``TRAKer(score_computer=B200ScoreComputer)``
(trak/traker.py:186-193).  Differences:

* products run on the tensor cores (fp32 inputs as row-scaled fp16 hi + lo planes, three
  passes; the Gram is accumulated 64 rows at a time, so it is as accurate as an fp32 GEMM);
* the regularised inverse goes through Cholesky in fp32 instead of LU and raises
  ``NotPositiveDefinite`` where the matrix is not positive definite;
* Gram blocks are accumulated in fp32 whatever ``dtype`` is (the reference adds
  them in ``dtype``) and cast once at the end;
* with a ``process_group`` the Gram of this rank's rows is summed over the group
  (one all-reduce of k x k fp32) -- rows sharded across GPUs, everything else
  local: the inverse is replicated, features and scores stay row-sharded;
* ``get_scores`` takes an optional ``row_scale`` (the out-to-loss weights) that is
  applied inside the GEMM epilogue, and streams the scores to a host accumulator through
  two pinned buffers while the next block is being multiplied.

There is no CPU path: tensors are moved to ``device`` and the CUDA library must load.
"""
import logging

import torch

from . import _lib

_DTYPES = {torch.float16: _lib.TB_F16, torch.bfloat16: _lib.TB_BF16, torch.float32: _lib.TB_F32}
_workspaces = {}
_MAX_CACHED_WORKSPACES = 8  # per process; streams come and go, their workspaces should not pile up


def _workspace(device, stream, nbytes):
    key = (device.index, stream)
    ws = _workspaces.pop(key, None)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)
    _workspaces[key] = ws  # most recently used last
    while len(_workspaces) > _MAX_CACHED_WORKSPACES:
        _workspaces.pop(next(iter(_workspaces)))
    return ws


def free_workspaces():
    _workspaces.clear()


class StreamPair:
    """Two side streams that row blocks alternate between.  Every product here is a memory-bound packing pass
    (row maxima, fp16 hi / lo planes) followed by a tensor-core GEMM; on one stream the packing of block i + 1
    waits for the GEMM of block i although the two use different parts of the SM.  With blocks alternating
    between two streams the packing (and any host-to-device copy) of one block runs under the GEMM of the other.
    Inside ``with pair:`` the side streams first wait for the caller's stream, and the caller's stream waits for
    both on exit; ``with pair.stream(i):`` makes stream ``i % 2`` current.  Work that touches the same memory
    from consecutive blocks (an accumulator, a reused buffer) must be given one buffer per stream."""

    def __init__(self, device):
        self.device = torch.device(device)
        self.streams = [torch.cuda.Stream(self.device), torch.cuda.Stream(self.device)]

    def __enter__(self):
        self.main = torch.cuda.current_stream(self.device)
        for s in self.streams:
            s.wait_stream(self.main)
        return self

    def __exit__(self, *exc):
        for s in self.streams:
            self.main.wait_stream(s)
        return False

    def stream(self, i: int):
        return torch.cuda.stream(self.streams[i % 2])


def _as_device_matrix(t: torch.Tensor, device) -> torch.Tensor:
    t = t.to(device, non_blocking=True)
    if t.dtype not in _DTYPES:
        t = t.float()
    if t.dim() != 2:
        raise RuntimeError("expected a 2-D tensor")
    if t.stride(1) != 1 or t.stride(0) < t.shape[1]:
        t = t.contiguous()
    return t


def gram(x: torch.Tensor, out: torch.Tensor = None, accumulate: bool = False) -> torch.Tensor:
    """fp32 [k, k] = x^T x (+ out) for a CUDA matrix x [n, k] (fp16 / bf16 / fp32)."""
    n, k = x.shape
    dev = x.device
    if out is None:
        out = torch.empty((k, k), dtype=torch.float32, device=dev)
        accumulate = False
    lib = _lib.lib()
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        dt = _DTYPES[x.dtype]
        ws = _workspace(dev, stream, lib.tb_gram_workspace_bytes(dt, n, k))
        _lib.check(lib.tb_gram(dev.index, stream, x.data_ptr(), dt, n, k, x.stride(0), out.data_ptr(),
                               out.stride(0), int(accumulate), ws.data_ptr(), ws.numel()))
    return out


def spd_inverse_(a: torch.Tensor, lambda_reg: float = 0.0, rescale: bool = True) -> torch.Tensor:
    """In place: a <- inv(a + lambda I) [/ mean |entry|] for a CUDA fp32 [k, k] matrix."""
    if a.dtype != torch.float32 or a.dim() != 2 or a.shape[0] != a.shape[1] or a.stride(1) != 1:
        raise RuntimeError("expected a square fp32 matrix with unit column stride")
    dev = a.device
    lib = _lib.lib()
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        ws = _workspace(dev, stream, lib.tb_spd_inverse_workspace_bytes(a.shape[0]))
        _lib.check(lib.tb_spd_inverse(dev.index, stream, a.data_ptr(), a.shape[0], a.stride(0),
                                      float(lambda_reg), int(rescale), None, ws.data_ptr(), ws.numel()))
        _lib.device_status(dev.index)  # raises NotPositiveDefinite / DeviceTimeout
    return a


def gemm_nt(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor = None, row_scale: torch.Tensor = None,
            alpha: float = 1.0, accumulate: bool = False) -> torch.Tensor:
    """fp32 [M, N] = alpha * row_scale[:, None] * a @ b.T (+ out) for CUDA a [M, K], b [N, K]."""
    if a.dtype != b.dtype:
        a, b = a.float(), b.float()
    M, K = a.shape
    N = b.shape[0]
    if b.shape[1] != K:
        raise RuntimeError("inner dimensions differ")
    dev = a.device
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=dev)
        accumulate = False
    if row_scale is not None:
        row_scale = row_scale.to(dev, torch.float32).reshape(-1).contiguous()
        if row_scale.numel() != M:
            raise RuntimeError("row_scale must have one entry per row of a")
    lib = _lib.lib()
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        dt = _DTYPES[a.dtype]
        ws = _workspace(dev, stream, lib.tb_gemm_nt_workspace_bytes(dt, M, N, K))
        _lib.check(lib.tb_gemm_nt(dev.index, stream, a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), dt,
                                  M, N, K, out.data_ptr(), out.stride(0),
                                  row_scale.data_ptr() if row_scale is not None else None, float(alpha),
                                  int(accumulate), ws.data_ptr(), ws.numel()))
    return out


class B200ScoreComputer:
    """Drop-in for ``BasicScoreComputer`` on a B200."""

    def __init__(self, dtype: torch.dtype, device, CUDA_MAX_DIM_SIZE: int = 65_536,
                 logging_level=logging.INFO, lambda_reg: float = 0.0, process_group=None) -> None:
        self.dtype = dtype
        device = torch.device(device)
        if device.type != "cuda":
            raise ValueError("B200ScoreComputer only works on a CUDA device")
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self.device = device
        self.CUDA_MAX_DIM_SIZE = CUDA_MAX_DIM_SIZE  # rows moved to the GPU and multiplied at a time
        self.logger = logging.getLogger("ScoreComputer")
        self.logger.setLevel(logging_level)
        self.lambda_reg = lambda_reg
        self.process_group = process_group
        _lib.lib()

    # -- trak/score_computers.py:145-155
    def get_xtx(self, grads: torch.Tensor) -> torch.Tensor:
        self.proj_dim = grads.shape[1]
        accs = [None, None]   # one partial Gram per stream of the pair (blocks alternate between them)
        with torch.cuda.device(self.device), self._pair() as pair:
            for i, block in enumerate(b for b in torch.split(grads, self.CUDA_MAX_DIM_SIZE, dim=0) if b.shape[0]):
                with pair.stream(i):
                    blk = _as_device_matrix(block, self.device)
                    blk.record_stream(torch.cuda.current_stream(self.device))
                    accs[i % 2] = gram(blk, out=accs[i % 2], accumulate=accs[i % 2] is not None)
        main = torch.cuda.current_stream(self.device)
        for a in accs:   # allocated on a side stream, used on the caller's from here on
            if a is not None:
                a.record_stream(main)
        acc = accs[0]
        if acc is None:
            # a rank whose shard holds no rows still has to reach the all-reduce: it contributes zeros
            acc = torch.zeros(self.proj_dim, self.proj_dim, dtype=torch.float32, device=self.device)
        elif accs[1] is not None:
            acc.add_(accs[1])
        acc = reduce_gram(acc, self.process_group)
        _lib.device_status(self.device.index)
        return acc.to(self.dtype)

    # -- trak/score_computers.py:157-177
    def get_x_xtx_inv(self, grads: torch.Tensor, xtx: torch.Tensor) -> torch.Tensor:
        inv = xtx.to(self.device, torch.float32).clone()
        spd_inverse_(inv, self.lambda_reg, rescale=True)
        inv = inv.to(self.dtype)
        result = torch.empty(grads.shape[0], inv.shape[1], dtype=self.dtype, device=self.device)
        if grads.shape[0]:
            probe = grads[:1]
            in_dtype = probe.dtype if probe.dtype in _DTYPES else torch.float32
            if in_dtype != inv.dtype:  # the narrower operand is promoted, never the inverse demoted
                inv = inv.to(torch.promote_types(in_dtype, inv.dtype))
        start = 0
        with torch.cuda.device(self.device), self._pair() as pair:
            for i, block in enumerate(b for b in torch.split(grads, self.CUDA_MAX_DIM_SIZE, dim=0) if b.shape[0]):
                rows = slice(start, start + block.shape[0])
                start += block.shape[0]
                with pair.stream(i):
                    blk = _as_device_matrix(block, self.device).to(inv.dtype)
                    blk.record_stream(torch.cuda.current_stream(self.device))
                    # the inverse is symmetric, so block @ inv == block @ inv.T
                    if result.dtype == torch.float32:
                        gemm_nt(blk, inv, out=result[rows])
                    else:
                        result[rows] = gemm_nt(blk, inv).to(self.dtype)
        _lib.device_status(self.device.index)
        return result

    def _pair(self) -> StreamPair:
        pair = getattr(self, "_stream_pair", None)
        if pair is None:
            self._stream_pair = pair = StreamPair(self.device)
        return pair

    # -- trak/score_computers.py:179-189
    def get_scores(self, features: torch.Tensor, target_grads: torch.Tensor, accumulator: torch.Tensor,
                   row_scale: torch.Tensor = None) -> None:
        """``accumulator += features @ target_grads.T`` (times ``row_scale`` per train row when given).

        TRAKer keeps the accumulator on the host (trak/traker.py:632): the product then leaves the GPU
        through two pinned staging buffers of at most ``HOST_STAGE_BYTES`` each, the copy of one row block
        overlapping the GEMM of the next and the host-side ``+=`` of the one before, instead of one
        synchronous pageable copy per block."""
        self._accumulate_products(features, _as_device_matrix(target_grads, self.device), accumulator, row_scale)

    def get_scores_from_grads(self, grads: torch.Tensor, xtx: torch.Tensor, target_grads: torch.Tensor,
                              accumulator: torch.Tensor, row_scale: torch.Tensor = None) -> None:
        """The same scores without materialising the features:
        ``accumulator += grads @ (inv @ target_grads.T)`` with ``inv`` the regularised, rescaled inverse of
        ``xtx`` exactly as ``get_x_xtx_inv`` forms it (trak/score_computers.py:157-168).  One product over
        the train rows instead of two: ``2 k^2 m`` flop for ``inv @ target_grads.T`` replace the ``2 n k^2``
        of the features.  For callers that do not need the features themselves (TRAKer stores them)."""
        inv = xtx.to(self.device, torch.float32).clone()
        spd_inverse_(inv, self.lambda_reg, rescale=True)
        targets = _as_device_matrix(target_grads, self.device)
        solved = gemm_nt(targets.float(), inv)  # [m, k] = target_grads @ inv  (inv is symmetric)
        self._accumulate_products(grads, solved, accumulator, row_scale)

    def _accumulate_products(self, features, targets, accumulator, row_scale):
        m = targets.shape[0]
        on_host = accumulator.device.type == "cpu"
        step = self.CUDA_MAX_DIM_SIZE
        if on_host:
            step = max(256, min(step, self.HOST_STAGE_BYTES // (4 * m) // 256 * 256))
            stage = self._host_stage(min(step, features.shape[0]), m)
        pending = None

        def flush(item):
            rows, buf, event = item
            event.synchronize()
            accumulator[rows] += buf.to(accumulator.dtype)

        start = 0
        with torch.cuda.device(self.device), self._pair() as pair:
            for i, block in enumerate(b for b in torch.split(features, step, dim=0) if b.shape[0]):
                rows = slice(start, start + block.shape[0])
                start += block.shape[0]
                with pair.stream(i):
                    cur = torch.cuda.current_stream(self.device)
                    blk = _as_device_matrix(block, self.device)
                    blk.record_stream(cur)
                    rs = None if row_scale is None else row_scale.reshape(-1)[rows]
                    part = gemm_nt(blk, targets, row_scale=rs)
                    if not on_host:
                        if accumulator.device == part.device:
                            accumulator[rows] += part.to(accumulator.dtype)
                        else:
                            accumulator[rows] += part.to(accumulator.dtype).to(accumulator.device)
                        continue
                    # buffer i % 2 was last read by the flush of block i - 2, which has returned; the copy runs
                    # on this block's stream, so the GEMM of the next block (other stream) overlaps it
                    buf = stage[i % 2][:blk.shape[0]]
                    buf.copy_(part, non_blocking=True)
                    event = torch.cuda.Event()
                    event.record(cur)
                if pending is not None:
                    flush(pending)
                pending = (rows, buf, event)
        if pending is not None:
            flush(pending)
        _lib.device_status(self.device.index)

    HOST_STAGE_BYTES = 256 << 20  # each of the two pinned buffers get_scores copies through

    def _host_stage(self, rows: int, m: int):
        """Two pinned fp32 buffers [rows, m], kept between calls (pinning is slow) and regrown when too small."""
        stage = getattr(self, "_stage", None)
        if stage is None or stage[0].shape[0] < rows or stage[0].shape[1] != m:
            self._stage = stage = [torch.empty(rows, m, dtype=torch.float32).pin_memory() for _ in range(2)]
        return stage


def reduce_gram(local_gram: torch.Tensor, process_group=None) -> torch.Tensor:
    """Sums the per-rank Gram matrices when the train rows are sharded over a process group
    (the only exchange of the scoring path); a no-op for a single process."""
    import torch.distributed as dist
    if process_group is None:
        return local_gram
    if not (dist.is_available() and dist.is_initialized()):
        raise RuntimeError("process_group given but torch.distributed is not initialised")
    dist.all_reduce(local_gram, op=dist.ReduceOp.SUM, group=process_group)
    return local_gram


def shard_rows(n: int, rank: int, world: int):
    """Contiguous row range [lo, hi) of rank `rank` when n rows are split over `world` ranks."""
    base, rem = divmod(n, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)
