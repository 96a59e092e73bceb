"""Generates ``fastjl_golden.npz`` with the reference's own compiled CUDA kernel.

Needs a GPU and the witness module built by ``oracle/build_ref.py``
(``oracle/_ref/fast_jl.so``, compiled from the reference checkout):

    python tests/golden/make_fastjl_golden.py [--out tests/golden/fastjl_golden.npz]

Two kinds of records, for both projection types:

* ``rows_*``  -- rows P[f, :] of the virtual projection matrix, read out by
  projecting one-hot inputs (fp16 values are exact: +-1, or fp16 normals);
* ``proj_*``  -- projections of seeded random fp16 / fp32 inputs
  (``torch.randn`` on the CPU generator, so the inputs can be rebuilt anywhere).

The file pins the CPU oracle's element map (CPU tests) and the new kernels
(GPU tests) to what the reference kernel actually computes.
"""
import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))

# (F, N, seed, num_feature_tiles); the third entry is the shape / seed / tile
# count of the reference's cross-GPU test (tests/test_jl_gpu_compatibility)
ROW_CASES = [(1000, 512, 0, 148), (5000, 1024, 123, 108), (100000, 4096, 123, 108),
             (75533, 512, 17, 148)]
PROJ_CASES = [(8, 1000, 512, 0, 148), (16, 33333, 1024, 5, 148), (32, 100000, 512, 123, 108)]


def row_features(F, T):
    fts = (F - 1) // min(F, T) + 1
    cand = [0, 1, 15, 16, 17, fts - 1, fts, fts + 1, F // 2, F - 1]
    return sorted(set(f for f in cand if 0 <= f < F))[:8]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(HERE, "fastjl_golden.npz"))
    a = ap.parse_args()
    sys.path.insert(0, ROOT)
    from oracle import build_ref
    w = build_ref.load()
    if w is None:
        raise SystemExit("oracle/_ref/fast_jl.so missing: run oracle/build_ref.py first")
    rec = {}
    for ci, (F, N, seed, T) in enumerate(ROW_CASES):
        feats = row_features(F, T)
        g = torch.zeros(8, F, dtype=torch.float16, device="cuda")
        for i, f in enumerate(feats):
            g[i, f] = 1.0
        rec[f"rows_{ci}_meta"] = np.array([F, N, seed, T], np.int64)
        rec[f"rows_{ci}_feats"] = np.array(feats, np.int64)
        for name in ("rademacher", "normal"):
            out = getattr(w, f"project_{name}_8")(g, N, seed, T)[:len(feats)].cpu().numpy()
            assert np.array_equal(out, out.astype(np.float16).astype(np.float32))
            rec[f"rows_{ci}_{name}"] = out.astype(np.float16)
    for ci, (B, F, N, seed, T) in enumerate(PROJ_CASES):
        rec[f"proj_{ci}_meta"] = np.array([B, F, N, seed, T, 100 + ci], np.int64)
        base = torch.randn(B, F, generator=torch.Generator().manual_seed(100 + ci))
        for dt, dn in ((torch.float16, "f16"), (torch.float32, "f32")):
            g = base.to(dt).cuda()
            for name in ("rademacher", "normal"):
                out = getattr(w, f"project_{name}_32")(g, N, seed, T).cpu().numpy()
                rec[f"proj_{ci}_{dn}_{name}"] = out.astype(np.float32)
    np.savez_compressed(a.out, **rec)
    print("wrote", a.out, os.path.getsize(a.out), "bytes")


if __name__ == "__main__":
    main()
