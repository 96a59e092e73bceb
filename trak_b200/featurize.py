"""The store side of ``TRAKer.featurize`` without a synchronisation per batch.

The reference projects a batch, divides by ``sqrt(num_params)``, casts, and writes into the
``grads.mmap`` rows with ``grads.to(dtype).cpu()`` -- a blocking device-to-host copy per batch, and
the same again for the out-to-loss weights (trak/traker.py:424-437).  ``FeatureWriter`` does the
same arithmetic with

* ``1 / normalize_factor`` folded into the projection (``alpha`` of ``tb_project``),
* a small ring of device buffers the projection writes into and pinned host buffers the cast
  result is copied to asynchronously,
* the host-side write into the memmap rows deferred until that copy's event has completed, i.e.
  while the GPU is already computing the gradients of a later batch,
* optionally the features of the whole shard kept on the device (``keep_on_device``), so that
  ``finalize_features`` can form the Gram without reading them back from the store.

Files stay byte-compatible with the reference's ``MmapSaver``: rows are written through the same
numpy memmaps (``mmap_io.open_store``).
"""
import numpy as np
import torch

from . import mmap_io
from .projectors import CudaProjector


class FeatureWriter:
    def __init__(self, projector, normalize_factor: float, dtype: torch.dtype, device, max_batch: int,
                 grads_store=None, out_to_loss_store=None, slots: int = 4, keep_on_device: bool = False,
                 n_rows: int = None):
        device = torch.device(device)
        if device.type != "cuda":
            raise ValueError("FeatureWriter only works on a CUDA device")
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self.projector, self.device, self.dtype = projector, device, dtype
        self.alpha = 1.0 / float(normalize_factor)
        self.grads_store, self.out_to_loss_store = grads_store, out_to_loss_store
        self.max_batch, self.k = max_batch, projector.proj_dim
        self.slots = max(2, slots)
        self.dev = [torch.empty(max_batch, self.k, dtype=torch.float32, device=device) for _ in range(self.slots)]
        self.host = [torch.empty(max_batch, self.k, dtype=dtype).pin_memory() for _ in range(self.slots)]
        self.host_w = [torch.empty(max_batch, 1, dtype=dtype).pin_memory() for _ in range(self.slots)]
        self.pending = [None] * self.slots   # (event, inds, rows, has_weights)
        self.turn = 0
        self.features_device = None
        if keep_on_device:
            if n_rows is None:
                n_rows = grads_store.shape[0]
            self.features_device = torch.zeros(n_rows, self.k, dtype=dtype, device=device)

    def _drain(self, slot):
        item = self.pending[slot]
        if item is None:
            return
        event, inds, rows, has_w = item
        event.synchronize()
        if self.grads_store is not None:
            self.grads_store[inds] = self.host[slot][:rows].numpy()
        if has_w and self.out_to_loss_store is not None:
            self.out_to_loss_store[inds] = self.host_w[slot][:rows].numpy()
        self.pending[slot] = None

    def add(self, grads, inds, model_id: int = 0, loss_grads: torch.Tensor = None) -> torch.Tensor:
        """Projects one batch of per-sample gradients (dict of tensors or ``[B, D]`` matrix), scales by
        ``1 / normalize_factor`` and queues the rows ``inds`` of the stores.  Returns the fp32 device
        features of the batch (valid until ``slots`` more batches have been added)."""
        if isinstance(inds, torch.Tensor):
            inds = inds.detach().cpu().numpy()
        inds = np.asarray(inds).reshape(-1)
        rows = len(inds)
        if rows > self.max_batch:
            raise RuntimeError(f"batch of {rows} exceeds max_batch={self.max_batch}")
        slot = self.turn
        self.turn = (self.turn + 1) % self.slots
        self._drain(slot)  # the copy that last used this slot finished long ago; its rows go to the store now
        out = self.dev[slot][:rows]
        if isinstance(self.projector, CudaProjector):
            self.projector.project(grads, model_id, alpha=self.alpha, out=out)
        else:  # any projector with the reference's signature
            out.copy_(self.projector.project(grads, model_id=model_id).to(torch.float32) * self.alpha)
        with torch.cuda.device(self.device):
            self.host[slot][:rows].copy_(out, non_blocking=True)      # casts to the store dtype on the way
            if loss_grads is not None:
                self.host_w[slot][:rows].copy_(loss_grads.reshape(rows, 1), non_blocking=True)
            if self.features_device is not None:
                self.features_device[torch.as_tensor(inds, device=self.device)] = out.to(self.dtype)
            event = torch.cuda.Event()
            event.record(torch.cuda.current_stream(self.device))
        self.pending[slot] = (event, inds, rows, loss_grads is not None)
        return out

    def flush(self):
        """Writes every queued batch into the stores (waits for their copies) and flushes the memmaps."""
        for s in range(self.slots):
            self._drain((self.turn + s) % self.slots)
        for st in (self.grads_store, self.out_to_loss_store):
            if st is not None and hasattr(st, "flush"):
                st.flush()
