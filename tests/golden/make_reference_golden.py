"""Generates ``basic_*.npz``: outputs of the UNMODIFIED reference CPU classes
(BasicProjector, BasicScoreComputer) on small seeded inputs.

Run where the reference checkout is importable:

    python tests/golden/make_reference_golden.py --reference /path/to/trak

The fixtures pin the CPU restatement in ``oracle/basic_ref.py`` and serve as
the expected values of the scoring parity tests.  Inputs are regenerated from
the seeds stored in each file, so only outputs (and small inputs) are saved.
"""
import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of MadryLab/trak")
    a = ap.parse_args()
    sys.path.insert(0, a.reference)
    from trak.projectors import BasicProjector
    from trak.score_computers import BasicScoreComputer

    torch.set_num_threads(1)  # fixed summation order inside the CPU matmuls

    # ---- projection: two proj types, proj_dim not a multiple of the block size
    for ptype in ("rademacher", "normal"):
        B, D, k, seed, model_id = 5, 777, 250, 42, 1
        g = torch.randn(B, D, generator=torch.Generator().manual_seed(7))
        proj = BasicProjector(grad_dim=D, proj_dim=k, seed=seed, proj_type=ptype, device="cpu",
                              model_id=model_id)
        out = proj.project(g, model_id=model_id)
        np.savez_compressed(os.path.join(HERE, f"basic_project_{ptype}.npz"), B=B, D=D, k=k,
                            seed=seed, model_id=model_id, input_seed=7, out=out.numpy())

    # ---- scoring: n > k, two row blocks (block size forced small), lambda > 0
    n, k, m, lam = 700, 96, 33, 1e-3
    X = torch.randn(n, k, generator=torch.Generator().manual_seed(11)) / k ** 0.5
    T = torch.randn(m, k, generator=torch.Generator().manual_seed(12)) / k ** 0.5
    sc = BasicScoreComputer(dtype=torch.float32, device="cpu", CUDA_MAX_DIM_SIZE=512, lambda_reg=lam)
    gram = sc.get_xtx(X)
    feats = sc.get_x_xtx_inv(X, gram)
    acc = torch.zeros(n, m)
    sc.get_scores(feats, T, accumulator=acc)
    np.savez_compressed(os.path.join(HERE, "basic_scoring.npz"), n=n, k=k, m=m, lam=lam,
                        x_seed=11, t_seed=12, block_rows=512, gram=gram.numpy(),
                        features=feats.numpy(), scores=acc.numpy())
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))


if __name__ == "__main__":
    main()
