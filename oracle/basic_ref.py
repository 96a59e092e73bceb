"""TEST INFRASTRUCTURE ONLY -- CPU restatement (torch, fp32) of the reference's
own CPU implementations of the two hot paths.  Only tests, the smoke check and
the benchmark's CPU legs may import it; the product never does.

* ``basic_project``   follows BasicProjector (trak/projectors.py:209-314): the
  matrix is drawn 100 columns at a time from a torch CPU generator seeded
  ``seed + 1000*block + 100000*model_id`` (trak/projectors.py:258-266), normal
  or ``2*bernoulli(0.5) - 1`` (trak/projectors.py:276-287), and each block is
  multiplied into its slice of the sketch (trak/projectors.py:303-313).
  Its matrix is NOT the fast_jl matrix; it is the statistical reference and
  the CPU timing baseline for the projection.
* ``xtx`` / ``x_xtx_inv`` / ``scores`` follow BasicScoreComputer
  (trak/score_computers.py:145-155, 157-177, 179-189) with the
  ``features @ target_grads.T`` product of trak/utils.py:128-133.
* ``finalize_scores_epilogue`` follows the host arithmetic at
  trak/traker.py:676-678.

Pins: ``tests/golden/basic_*.npz`` were produced by the unmodified reference
classes (tests/golden/make_reference_golden.py) and are compared bit for bit
(projection) or to fp32 round-off (scoring) in tests/test_oracle_basic.py.
"""
import math

import torch


def basic_project(grads: torch.Tensor, proj_dim: int, seed: int, proj_type: str,
                  block_size: int = 100, model_id: int = 0, blocks=None) -> torch.Tensor:
    """Sketch [B, proj_dim] of fp32 ``grads`` [B, D] on the CPU.

    ``blocks`` (an iterable of block indices) restricts the work to some column
    blocks -- the other columns stay zero -- which the benchmark uses to time a
    bounded sample.
    """
    g = grads.to(torch.float32)
    D = g.shape[1]
    bs = min(proj_dim, block_size)
    nblocks = math.ceil(proj_dim / bs)
    out = torch.zeros(g.shape[0], proj_dim, dtype=torch.float32)
    gen = torch.Generator(device="cpu")
    P = torch.empty(D, bs, dtype=torch.float32)
    for i in (range(nblocks) if blocks is None else blocks):
        gen.manual_seed(seed + 1000 * i + 100000 * model_id)
        if proj_type == "normal":
            P.normal_(generator=gen)
        elif proj_type == "rademacher":
            P.bernoulli_(p=0.5, generator=gen)
            P.mul_(2.0).sub_(1.0)
        else:
            raise KeyError(proj_type)
        lo, hi = i * bs, min((i + 1) * bs, proj_dim)
        out[:, lo:hi] = g @ P[:, : hi - lo]
    return out


def xtx(grads: torch.Tensor, block_rows: int = 20_000) -> torch.Tensor:
    k = grads.shape[1]
    acc = torch.zeros(k, k, dtype=grads.dtype)
    for blk in torch.split(grads, block_rows, dim=0):
        acc += blk.T @ blk
    return acc


def xtx_inverse(gram: torch.Tensor, lambda_reg: float) -> torch.Tensor:
    """Regularised inverse with the reference's global rescale by mean |entry|."""
    reg = gram + lambda_reg * torch.eye(gram.shape[0], dtype=gram.dtype)
    inv = torch.linalg.inv(reg.to(torch.float32))
    inv /= inv.abs().mean()
    return inv


def x_xtx_inv(grads: torch.Tensor, gram: torch.Tensor, lambda_reg: float,
              block_rows: int = 20_000) -> torch.Tensor:
    inv = xtx_inverse(gram, lambda_reg).to(grads.dtype)
    out = torch.empty(grads.shape[0], inv.shape[1], dtype=grads.dtype)
    for i, blk in enumerate(torch.split(grads, block_rows, dim=0)):
        out[i * block_rows: i * block_rows + blk.shape[0]] = blk @ inv
    return out


def scores(features: torch.Tensor, target_grads: torch.Tensor, accumulator: torch.Tensor) -> None:
    accumulator += features @ target_grads.T


def finalize_scores_epilogue(score_sum: torch.Tensor, out_to_loss_sum: torch.Tensor,
                             num_models: int) -> torch.Tensor:
    """(sum of per-checkpoint scores / M) * (sum of per-checkpoint out-to-loss / M),
    the latter [n, 1] broadcast over targets."""
    return (score_sum / num_models) * (out_to_loss_sum / num_models)
