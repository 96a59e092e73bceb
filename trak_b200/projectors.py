"""Projector classes with the reference's constructor and ``project`` signatures,
running on the sm_100a kernels.

Mirrors ``ProjectionType`` (trak/projectors.py:25-27), ``CudaProjector``
(trak/projectors.py:317-427) and ``ChunkedCudaProjector``
(trak/projectors.py:430-516).  They can be handed to an unmodified ``TRAKer``
through its ``projector=`` argument, or picked up implicitly by registering
``trak_b200.fast_jl`` as the ``fast_jl`` module.
"""
from enum import Enum
from typing import Union

import torch

from . import fast_jl as _fast_jl
from . import _lib


class ProjectionType(str, Enum):
    normal: str = "normal"
    rademacher: str = "rademacher"


_PTYPE_CODE = {"rademacher": _lib.TB_RADEMACHER, "normal": _lib.TB_NORMAL}


def _ptype_code(proj_type) -> int:
    name = proj_type.value if isinstance(proj_type, Enum) else str(proj_type)
    try:
        return _PTYPE_CODE[name]
    except KeyError:
        raise KeyError(f"Projection type {proj_type} not recognized.")


def vectorize(g: dict, device="cuda") -> torch.Tensor:
    """Flattens a dict of per-sample gradients ``{name: [B, *shape]}`` into ``[B, D]`` in
    dict order; a tensor with fewer than two dimensions contributes one column
    (trak/utils.py:80-110)."""
    vals = list(g.values())
    B = vals[0].shape[0]
    widths = [1 if v.dim() < 2 else v[0].numel() for v in vals]
    out = torch.empty((B, sum(widths)), dtype=vals[0].dtype, device=device)
    ptr = 0
    for v, w in zip(vals, widths):
        if v.shape[0] != B:
            raise AssertionError("all gradients must share the batch dimension")
        out[:, ptr:ptr + w] = v.data.reshape(B, w).to(device)
        ptr += w
    return out


def _segmentable(vals, device) -> bool:
    if not vals:
        return False
    d = torch.device(device)
    return all(v.is_cuda and v.device == d and v.dtype == vals[0].dtype for v in vals) and \
        vals[0].dtype in (torch.float16, torch.bfloat16, torch.float32)


class CudaProjector:
    """JL projection on a B200.  ``max_batch_size`` is accepted for signature
    compatibility; the kernels take any batch and ignore it."""

    def __init__(self, grad_dim: int, proj_dim: int, seed: int, proj_type: ProjectionType, device,
                 max_batch_size: int = 32, *args, store_matrix: bool = False, **kwargs) -> None:
        # store_matrix: keep the projection matrix of the current (seed, model_id) in device memory
        # (2 * proj_dim bytes per feature: 91.6 GB for a CIFAR ResNet-18 and proj_dim 4096) and read it
        # instead of regenerating it in every call -- about three times faster for the Gaussian matrix
        # when the same projector serves many batches, as TRAKer.featurize does.  Same matrix, same results
        # up to the order of the fp32 sums.
        self.store_matrix = bool(store_matrix)
        self._matrix = None
        self.grad_dim = grad_dim
        self.proj_dim = proj_dim
        self.seed = seed
        self.proj_type = proj_type
        self.max_batch_size = max_batch_size
        if isinstance(device, str):
            device = torch.device(device)
        if device.type != "cuda":
            raise ValueError("CudaProjector only works on a CUDA device; Either switch to a CUDA "
                             "device, or use the BasicProjector")
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self.device = device
        self._ptype = _ptype_code(proj_type)
        # the SM count is part of the matrix definition (trak/projectors.py:370,409)
        self.num_sms = torch.cuda.get_device_properties(device.index).multi_processor_count
        try:
            _lib.lib()
        except ImportError as e:
            raise ModuleNotFoundError(str(e))
        # same init-time launch as the reference, on this projector's device
        _fast_jl.project_rademacher_8(torch.zeros(8, 1_000, device=device), 512, 0, self.num_sms)

    def project(self, grads: Union[dict, torch.Tensor], model_id: int, *, alpha: float = 1.0,
                out: torch.Tensor = None, accumulate: bool = False) -> torch.Tensor:
        # the kernel's seed is an unsigned 32-bit integer: a value outside that range raises TypeError,
        # as the reference's pybind signature does (fast_jl/fast_jl.cu:81-110)
        seed = self.seed + int(1e4) * model_id
        if isinstance(grads, dict):
            vals = list(grads.values())
            if _segmentable(vals, self.device):
                # straight from the per-parameter tensors: no [B, D] copy (trak/utils.py:80-110)
                width = sum(1 if v.dim() < 2 else v[0].numel() for v in vals)
                return _fast_jl.project_segments(vals, self.proj_dim, seed, self.num_sms, self._ptype,
                                                 alpha=alpha, out=out, accumulate=accumulate,
                                                 matrix=self._stored(seed, width, vals[0].dtype))
            grads = vectorize(grads, device=self.device)
        return _fast_jl.project(grads, self.proj_dim, seed,
                                self.num_sms, self._ptype, alpha=alpha, out=out,
                                accumulate=accumulate, allow_strided=True,
                                matrix=self._stored(seed, grads.shape[1], grads.dtype))

    def _stored(self, seed, width, dtype):
        """The stored matrix for this seed and gradient format, generated on first use (one at a time: a new
        model_id or dtype replaces it); None when store_matrix is off."""
        if not self.store_matrix:
            return None
        elem = _lib.TB_BF16 if dtype == torch.bfloat16 else _lib.TB_F16
        m = self._matrix
        if m is None or (m.seed, m.F, m.elem) != (seed, width, elem):
            self._matrix = m = None   # drop every reference to the old one before the new one is allocated
            self._matrix = m = _fast_jl.StoredMatrix(width, self.proj_dim, seed, self.num_sms, self._ptype,
                                                     dtype=dtype, device=self.device)
        return m

    def free_memory(self):
        """Drops the cached kernel workspaces and the stored matrix."""
        self._matrix = None
        _fast_jl.free_workspaces()


class ChunkedCudaProjector:
    """Projects models whose gradient does not fit one call: parameters are packed,
    whole, into chunks of at most ``max_chunk_size`` features, each chunk has its own
    projector (own seed), and the chunk projections are summed.

    Differences from the reference that do not change the result beyond fp32
    round-off: chunks are summed in fp32 inside the kernel's epilogue instead of
    ``add_`` in the storage dtype, and only the rows of the current batch are
    projected."""

    def __init__(self, projector_per_chunk: list, max_chunk_size: int, params_per_chunk: list,
                 feat_bs: int, device: torch.device, dtype: torch.dtype):
        self.projector_per_chunk = projector_per_chunk
        self.proj_dim = self.projector_per_chunk[0].proj_dim
        self.proj_type = self.projector_per_chunk[0].proj_type
        self.params_per_chunk = params_per_chunk
        self.max_chunk_size = max_chunk_size
        self.feat_bs = feat_bs
        self.device = device
        self.dtype = dtype
        self.input_allocated = False

    def allocate_input(self):
        if self.input_allocated:
            return
        width = max(int(c) for c in self.params_per_chunk)
        self.ch_input = torch.zeros((self.feat_bs, width), device=self.device, dtype=self.dtype)
        self.input_allocated = True

    def free_memory(self):
        if not self.input_allocated:
            return
        del self.ch_input
        self.input_allocated = False

    def _project_direct(self, vals, rows, model_id, out):
        """Same chunking rule, but every chunk is projected straight from its parameters' tensors
        (no packing into ch_input) and accumulated into `out` by the kernel."""
        chunk, width, index = [], 0, 0
        for p in vals:
            w = 1 if p.dim() < 2 else p[0].numel()
            if width + w > self.max_chunk_size:
                self._check_chunk(index, width)
                self.projector_per_chunk[index].project(dict(enumerate(chunk)), model_id, out=out,
                                                        accumulate=index > 0)
                chunk, width, index = [], 0, index + 1
            chunk.append(p[:rows])
            width += w
        self._check_chunk(index, width)
        self.projector_per_chunk[index].project(dict(enumerate(chunk)), model_id, out=out, accumulate=index > 0)
        return out.to(self.dtype)

    def _check_chunk(self, index, width):
        """A chunk must hold at least one whole parameter.  ``get_parameter_chunk_sizes`` emits a leading
        chunk of width 0 when the first parameter alone exceeds the cap (trak/utils.py:321-326); such a
        chunk cannot be projected, so the cap has to be raised to admit the largest parameter."""
        if width == 0:
            raise ValueError(f"parameter chunk {index} is empty: a single parameter is larger than "
                             f"max_chunk_size={self.max_chunk_size}; raise the chunk size to at least the largest "
                             "parameter")
        assert width == self.params_per_chunk[index], "params_per_chunk does not match grads"

    def _flush(self, index, rows, pointer, model_id, out, first):
        self._check_chunk(index, pointer)
        proj = self.projector_per_chunk[index]
        chunk = self.ch_input[:rows, :pointer]
        if isinstance(proj, CudaProjector):
            # row-strided view goes to the kernel as is (leading dimension = buffer width)
            proj.project(chunk, model_id=model_id, out=out, accumulate=not first)
        else:  # any other projector object with the reference's project(grads, model_id)
            res = proj.project(chunk.contiguous(), model_id=model_id).to(torch.float32)
            out.copy_(res) if first else out.add_(res)

    def project(self, grads, model_id):
        vals = list(grads.values())
        rows = vals[0].shape[0]
        if rows > self.feat_bs:
            # the reference fails here on the shape mismatch of its copy into ch_input (trak/projectors.py:501-502)
            raise RuntimeError(f"batch of {rows} gradients exceeds feat_bs={self.feat_bs} of this projector")
        out = torch.empty((rows, self.proj_dim), device=self.device, dtype=torch.float32)
        if all(isinstance(p, CudaProjector) for p in self.projector_per_chunk) and \
                _segmentable(vals, self.device):
            return self._project_direct(vals, rows, model_id, out)
        self.allocate_input()
        pointer, index, first = 0, 0, True
        for p in vals:
            flat = p.data.unsqueeze(-1) if p.dim() < 2 else p.data.flatten(start_dim=1)
            width = flat.size(1)
            if pointer + width > self.max_chunk_size:
                self._flush(index, rows, pointer, model_id, out, first)
                pointer, index, first = 0, index + 1, False
            # same consistency requirement as the reference's asserts on params_per_chunk
            assert pointer + width <= self.ch_input.size(1), "params_per_chunk does not match grads"
            self.ch_input[:rows, pointer:pointer + width].copy_(flat[:rows])
            pointer += width
        self._flush(index, rows, pointer, model_id, out, first)
        return out.to(self.dtype)


def get_parameter_chunk_sizes(model_or_widths, batch_size: int = None, max_chunk_size: int = None):
    """``(max_chunk_size, params_per_chunk)`` as the reference computes them (trak/utils.py:297-331): the
    parameters, in order, are grouped whole into chunks, a new chunk starting when the running width would
    reach ``max_chunk_size``.  The reference's cap is ``uint32 max // batch_size`` (its kernel indexes the
    batch with 32 bits); these kernels have no such limit, so any ``max_chunk_size`` may be given instead.
    ``model_or_widths`` is a module or the list of parameter widths.  A parameter wider than the cap leaves an
    empty leading chunk, exactly as in the reference -- raise the cap to at least the widest parameter."""
    import numpy as np
    if isinstance(model_or_widths, torch.nn.Module):
        widths = [p.numel() for p in model_or_widths.parameters()]
    else:
        widths = [int(w) for w in model_or_widths]
    if max_chunk_size is None:
        if not batch_size:
            raise ValueError("give batch_size (the reference's rule) or max_chunk_size")
        max_chunk_size = int(np.iinfo(np.uint32).max // batch_size)
    chunk_sum, params_per_chunk = 0, []
    for w in widths:
        if chunk_sum + w >= max_chunk_size:
            params_per_chunk.append(chunk_sum)
            chunk_sum = 0
        chunk_sum += w
    rest = sum(widths) - sum(params_per_chunk)
    if rest > 0:
        params_per_chunk.append(rest)
    return max_chunk_size, params_per_chunk


def make_chunked_projector(model_or_widths, proj_dim: int, proj_seed: int, feat_bs: int, device, dtype,
                           max_chunk_size: int = None) -> ChunkedCudaProjector:
    """The ``ChunkedCudaProjector`` that ``TRAKer.init_projector`` builds (trak/traker.py:284-320): one
    Rademacher ``CudaProjector`` per chunk with seeds ``default_rng(proj_seed).integers(0, 500, n_chunks)``."""
    import numpy as np
    cap, sizes = get_parameter_chunk_sizes(model_or_widths, batch_size=feat_bs, max_chunk_size=max_chunk_size)
    seeds = np.random.default_rng(proj_seed).integers(low=0, high=500, size=len(sizes))
    projs = [CudaProjector(grad_dim=int(s), proj_dim=proj_dim, seed=int(sd), proj_type=ProjectionType.rademacher,
                           device=device, max_batch_size=feat_bs) for s, sd in zip(sizes, seeds) if s > 0]
    if len(projs) != len(sizes):
        raise ValueError(f"a parameter is wider than max_chunk_size={cap}; raise it to at least the widest parameter")
    return ChunkedCudaProjector(projs, cap, sizes, feat_bs, torch.device(device), dtype)
