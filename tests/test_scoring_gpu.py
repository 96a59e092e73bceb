"""Parity of the sm_100a scoring path (through the C ABI) with the reference's CPU
BasicScoreComputer: against fixtures produced by the unmodified reference and against
its CPU port on seeded inputs.

Tolerance: Frobenius-relative 1e-3 for Gram, features and scores; the three-pass fp16-split
GEMMs land around 1e-5.
"""
import os

import numpy as np
import pytest
import torch

from oracle import basic_ref as br

pytestmark = pytest.mark.gpu
TOL = 1e-3


def rel(a, b):
    a = torch.as_tensor(a).double().cpu()
    b = torch.as_tensor(b).double().cpu()
    return float((a - b).norm() / b.norm())


def test_pipeline_matches_reference_fixture(cuda, golden_dir):
    from trak_b200.score_computers import B200ScoreComputer
    d = np.load(os.path.join(golden_dir, "basic_scoring.npz"))
    n, k, m, lam = int(d["n"]), int(d["k"]), int(d["m"]), float(d["lam"])
    X = torch.randn(n, k, generator=torch.Generator().manual_seed(int(d["x_seed"]))) / k ** 0.5
    T = torch.randn(m, k, generator=torch.Generator().manual_seed(int(d["t_seed"]))) / k ** 0.5
    sc = B200ScoreComputer(dtype=torch.float32, device=cuda, CUDA_MAX_DIM_SIZE=int(d["block_rows"]), lambda_reg=lam)
    gram = sc.get_xtx(X)                      # CPU input, like TRAKer's memmaps
    feats = sc.get_x_xtx_inv(X, gram)
    acc = torch.zeros(n, m)                   # CPU accumulator, as in trak/traker.py:632
    sc.get_scores(feats, T, acc)
    assert gram.shape == (k, k) and feats.shape == (n, k) and gram.dtype == torch.float32
    assert rel(gram, d["gram"]) <= TOL
    assert rel(feats, d["features"]) <= TOL
    assert rel(acc, d["scores"]) <= TOL
    sc.get_scores(feats, T, acc)              # accumulates
    assert rel(acc, 2 * d["scores"]) <= TOL


@pytest.mark.parametrize("n,k,m,lam,dtype", [
    (3000, 256, 100, 1e-3, torch.float32),
    (2500, 333, 77, 1e-2, torch.float32),      # nothing a multiple of the tile sizes
    (4000, 512, 1000, 1e-3, torch.float16),    # TRAKer's default storage dtype
    (300, 64, 5, 0.5, torch.float32),
])
def test_pipeline_matches_cpu_port(cuda, n, k, m, lam, dtype):
    from trak_b200.score_computers import B200ScoreComputer
    X = (torch.randn(n, k, generator=torch.Generator().manual_seed(n)) / k ** 0.5).to(dtype)
    T = (torch.randn(m, k, generator=torch.Generator().manual_seed(m)) / k ** 0.5).to(dtype)
    sc = B200ScoreComputer(dtype=dtype, device=cuda, CUDA_MAX_DIM_SIZE=1024, lambda_reg=lam)
    gram = sc.get_xtx(X.to(cuda))
    feats = sc.get_x_xtx_inv(X.to(cuda), gram)
    acc = torch.zeros(n, m)
    sc.get_scores(feats, T.to(cuda), acc)
    assert gram.dtype == dtype and feats.dtype == dtype
    Xf, Tf = X.float(), T.float()
    g_ref = br.xtx(Xf)
    f_ref = br.x_xtx_inv(Xf, g_ref, lam)
    s_ref = torch.zeros(n, m)
    br.scores(f_ref, Tf, s_ref)
    tol = TOL if dtype == torch.float32 else 3e-3   # fp16 storage of the Gram and the features
    assert rel(gram, g_ref) <= tol
    assert rel(feats, f_ref) <= tol
    assert rel(acc, s_ref) <= tol


def test_primitives_against_fp64(cuda):
    from trak_b200 import score_computers as sc
    torch.manual_seed(0)
    a = torch.randn(257, 70, device=cuda)
    b = torch.randn(513, 70, device=cuda)
    assert rel(sc.gemm_nt(a, b), a.double() @ b.double().T) <= 1e-4
    w = torch.rand(257, device=cuda)
    out = torch.ones(257, 513, device=cuda)
    sc.gemm_nt(a, b, out=out, row_scale=w, alpha=0.5, accumulate=True)
    assert rel(out, 1.0 + 0.5 * w.double()[:, None] * (a.double() @ b.double().T)) <= 1e-4
    x = torch.randn(1000, 130, device=cuda)
    g = sc.gram(x)
    assert torch.equal(g, g.T)                # stored twice from the same accumulator
    assert rel(g, x.double().T @ x.double()) <= 1e-4
    for k in (1, 63, 64, 65, 200):
        y = torch.randn(4 * k + 3, k, device=cuda, dtype=torch.float64)
        A = (y.T @ y / k).float()
        inv = sc.spd_inverse_(A.clone(), 1e-2, rescale=False)
        ref = torch.linalg.inv(A.double() + 1e-2 * torch.eye(k, device=cuda, dtype=torch.float64))
        assert rel(inv, ref) <= 1e-4
        inv2 = sc.spd_inverse_(A.clone(), 1e-2, rescale=True)
        assert rel(inv2, ref / ref.abs().mean()) <= 1e-4


def test_fused_out_to_loss_weighting(cuda):
    # the host epilogue of trak/traker.py:676-678 with one checkpoint, fused as a row scale
    from trak_b200.score_computers import B200ScoreComputer
    n, k, m = 900, 128, 40
    F = torch.randn(n, k, generator=torch.Generator().manual_seed(1))
    T = torch.randn(m, k, generator=torch.Generator().manual_seed(2))
    w = torch.rand(n, 1, generator=torch.Generator().manual_seed(3))
    sc = B200ScoreComputer(dtype=torch.float32, device=cuda, CUDA_MAX_DIM_SIZE=400)
    acc = torch.zeros(n, m)
    sc.get_scores(F, T, acc, row_scale=w)
    plain = torch.zeros(n, m)
    br.scores(F, T, plain)
    assert rel(acc, br.finalize_scores_epilogue(plain, w, 1)) <= TOL


def test_not_positive_definite_is_reported(cuda):
    from trak_b200 import _lib, score_computers as sc
    with pytest.raises(_lib.NotPositiveDefinite):
        sc.spd_inverse_(-torch.eye(100, device=cuda), 0.0)
    _lib.device_status(cuda.index)            # the status word was cleared


def test_larger_shape_properties(cuda):
    # k = 2048: symmetry, inverse times matrix = identity, agreement with an fp64 solve
    from trak_b200 import score_computers as sc
    k, n = 2048, 16384
    x = torch.randn(n, k, device=cuda) / k ** 0.5
    g = sc.gram(x)
    assert torch.equal(g, g.T)
    inv = sc.spd_inverse_(g.clone(), 1e-3, rescale=False)
    eye = (g.double() + 1e-3 * torch.eye(k, device=cuda, dtype=torch.float64)) @ inv.double()
    assert float((eye - torch.eye(k, device=cuda, dtype=torch.float64)).abs().max()) < 1e-3


def test_fp32_products_are_fp32_grade(cuda):
    """fp32 operands travel as two fp16 planes of the row-scaled value (22-23 mantissa bits, the lo*lo term
    dropped), and the row scales must absorb any spread of magnitudes between rows.  The Gram, whose error
    the inverse amplifies, is accumulated 64 k at a time and must sit within a small factor of plain fp32
    arithmetic; the other products keep one long tensor-core accumulation (truncating: about 1e-5)."""
    from trak_b200 import score_computers as sc
    g = torch.Generator(device=cuda).manual_seed(5)
    a = torch.randn(700, 3000, device=cuda, generator=g)
    b = torch.randn(900, 3000, device=cuda, generator=g)
    exact = a.double() @ b.double().T
    assert rel(sc.gemm_nt(a, b), exact) <= 3e-5
    x = torch.randn(5000, 600, device=cuda, generator=g)
    exact_gram = x.double().T @ x.double()
    err = rel(sc.gram(x), exact_gram)
    print(f"Gram 5000 x 600: {err:.2e} (torch fp32 matmul: {rel(x.T @ x, exact_gram):.2e})")
    assert err <= 5e-7, err
    # rows spread over twenty orders of magnitude each (and some all-zero): row-wise relative error
    sa = 10.0 ** (torch.rand(700, 1, device=cuda, generator=g) * 20 - 18)
    sb = 10.0 ** (torch.rand(900, 1, device=cuda, generator=g) * 20 - 2)
    a2, b2 = a * sa, b * sb
    a2[17] = 0
    b2[5] = 0
    got = sc.gemm_nt(a2, b2).double()
    want = a2.double() @ b2.double().T
    assert torch.isfinite(got).all()
    assert float(got[17].abs().max()) == 0.0 and float(got[:, 5].abs().max()) == 0.0
    keep = torch.ones(700, dtype=torch.bool, device=cuda)
    keep[17] = False
    rows = (got - want).norm(dim=1)[keep] / want.norm(dim=1)[keep]
    assert float(rows.max()) <= 3e-5
    # columns of the transposed operand (the Gram's scales) spread as well
    x2 = x * 10.0 ** (torch.rand(1, 600, device=cuda, generator=g) * 30 - 15)
    g2 = sc.gram(x2).double()
    w2 = x2.double().T @ x2.double()
    d = w2.diagonal().sqrt()
    assert float(((g2 - w2) / (d[:, None] * d[None, :])).abs().max()) <= 1e-6


def test_ill_conditioned_gram_keeps_the_scores_accurate(cuda):
    """Features with a fast-decaying spectrum (what real gradient features look like): the inverse amplifies
    any error of the Gram by its condition number (here about 3000), so the products have to be fp32-grade
    for the scores to stay within the 1e-3 bar."""
    from trak_b200.score_computers import B200ScoreComputer
    n, k, m = 4000, 512, 64
    g = torch.Generator().manual_seed(11)
    u = torch.linalg.qr(torch.randn(n, k, generator=g, dtype=torch.float64))[0]
    v = torch.linalg.qr(torch.randn(k, k, generator=g, dtype=torch.float64))[0]
    sv = torch.logspace(0, -2, k, dtype=torch.float64)            # singular values 1 ... 1e-2
    X = ((u * sv) @ v.T).float()
    T = (torch.randn(m, k, generator=g, dtype=torch.float64) @ (v * sv) @ v.T).float()
    lam = float(sv[-1] ** 2 * 2.5)                                 # cond(G + lam I) about 2900
    sc = B200ScoreComputer(dtype=torch.float32, device=cuda, CUDA_MAX_DIM_SIZE=1500, lambda_reg=lam)
    feats = sc.get_x_xtx_inv(X, sc.get_xtx(X))
    acc = torch.zeros(n, m)
    sc.get_scores(feats, T, acc)
    Xd, Td = X.double(), T.double()
    inv = torch.linalg.inv(Xd.T @ Xd + lam * torch.eye(k, dtype=torch.float64))
    inv /= inv.abs().mean()
    err = rel(acc, Xd @ inv @ Td.T)
    assert err <= 2e-4, err


@pytest.mark.parametrize("k", [511, 513, 1000, 1025, 1537, 2049, 3000])
def test_inverse_at_sizes_around_the_block_boundaries(cuda, k):
    """Sizes on both sides of the 512-wide block columns of the Cholesky and of the 1024 threshold from which the
    triangular merges run on the tensor cores, with ragged last blocks: inverse against an fp64 solve."""
    from trak_b200 import score_computers as sc
    g = torch.Generator(device=cuda).manual_seed(k)
    y = torch.randn(3 * k, k, device=cuda, generator=g, dtype=torch.float64)
    A = (y.T @ y / k).float()
    lam = 1e-2
    ref = torch.linalg.inv(A.double() + lam * torch.eye(k, device=cuda, dtype=torch.float64))
    inv = sc.spd_inverse_(A.clone(), lam, rescale=False)
    assert torch.equal(inv, inv.T)
    assert rel(inv, ref) <= 2e-5, rel(inv, ref)
    inv2 = sc.spd_inverse_(A.clone(), lam, rescale=True)
    assert rel(inv2, ref / ref.abs().mean()) <= 2e-5


@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (129, 257, 33), (300, 700, 95), (128, 256, 64), (513, 100, 4097)])
def test_gram_and_gemm_at_ragged_sizes(cuda, M, N, K):
    """Tile, chunk (64 k) and slot (32 k) boundaries of both GEMM kernels, with accumulation into existing output."""
    from trak_b200 import score_computers as sc
    g = torch.Generator(device=cuda).manual_seed(M + N + K)
    a = torch.randn(M, K, device=cuda, generator=g)
    b = torch.randn(N, K, device=cuda, generator=g)
    out = torch.full((M, N), 2.0, device=cuda)
    sc.gemm_nt(a, b, out=out, accumulate=True, alpha=-0.5)
    assert rel(out, 2.0 - 0.5 * (a.double() @ b.double().T)) <= 3e-5   # one long tensor-core accumulation
    x = torch.randn(K, N, device=cuda, generator=g)          # Gram over K rows: the chunked kernel
    gram = torch.ones(N, N, device=cuda)
    sc.gram(x, out=gram, accumulate=True)
    want = 1.0 + x.double().T @ x.double()
    assert torch.equal(gram, gram.T)
    assert rel(gram, want) <= 1e-6


def test_scores_stream_to_a_host_accumulator_in_several_blocks(cuda):
    """The host accumulator path: more row blocks than staging buffers, a ragged last block, two calls
    accumulating (two checkpoints), fp32 and fp16 accumulators."""
    from trak_b200.score_computers import B200ScoreComputer
    n, k, m = 3000, 256, 70
    F = torch.randn(n, k, generator=torch.Generator().manual_seed(1))
    T = torch.randn(m, k, generator=torch.Generator().manual_seed(2))
    sc = B200ScoreComputer(dtype=torch.float32, device=cuda)
    sc.HOST_STAGE_BYTES = 256 * m * 4 * 3            # 768 rows per block: four blocks, the last one ragged
    want = F.double() @ T.double().T
    for dt, tol in ((torch.float32, 1e-5), (torch.float16, 2e-3)):
        acc = torch.zeros(n, m, dtype=dt)
        sc.get_scores(F, T, acc)
        assert rel(acc, want) <= tol
        sc.get_scores(F.to(cuda), T.to(cuda), acc)
        assert rel(acc, 2 * want) <= tol


def test_scores_without_forming_the_features(cuda):
    """get_scores_from_grads (targets through the inverse first, one product over the train rows) against
    get_x_xtx_inv + get_scores and against the CPU port of the reference."""
    from trak_b200.score_computers import B200ScoreComputer
    n, k, m, lam = 2500, 333, 77, 1e-2
    X = torch.randn(n, k, generator=torch.Generator().manual_seed(4)) / k ** 0.5
    T = torch.randn(m, k, generator=torch.Generator().manual_seed(5)) / k ** 0.5
    w = torch.rand(n, 1, generator=torch.Generator().manual_seed(6))
    sc = B200ScoreComputer(dtype=torch.float32, device=cuda, CUDA_MAX_DIM_SIZE=1024, lambda_reg=lam)
    gram = sc.get_xtx(X)
    two_step = torch.zeros(n, m)
    sc.get_scores(sc.get_x_xtx_inv(X, gram), T, two_step, row_scale=w)
    direct = torch.zeros(n, m)
    sc.get_scores_from_grads(X, gram, T, direct, row_scale=w)
    assert rel(direct, two_step) <= 1e-4
    s_ref = torch.zeros(n, m)
    br.scores(br.x_xtx_inv(X, br.xtx(X), lam), T, s_ref)
    assert rel(direct, br.finalize_scores_epilogue(s_ref, w, 1)) <= TOL


def test_pipeline_at_the_benchmark_projection_dim(cuda):
    """k = 8192, the size the scoring benchmark runs at (X ~ N(0, 1/k), lambda = 1e-3): Gram, rescaled inverse,
    features and scores of get_xtx -> get_x_xtx_inv -> get_scores (and of get_scores_from_grads) against the CPU
    port of BasicScoreComputer on the same inputs, each within 1e-3 Frobenius-relative.  At this size the
    inverse runs 16 block columns of the two-level Cholesky, the tensor-core merge levels 1024, 2048 and 4096
    and the 1056-tile symmetric W^T W."""
    from trak_b200.score_computers import B200ScoreComputer
    n, k, m, lam = 16_384, 8192, 512, 1e-3
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    X = torch.randn(n, k, generator=torch.Generator().manual_seed(2000)) / k ** 0.5
    T = torch.randn(m, k, generator=torch.Generator().manual_seed(3000)) / k ** 0.5
    w = torch.rand(n, 1, generator=torch.Generator().manual_seed(4000))
    sc = B200ScoreComputer(dtype=torch.float32, device=cuda, lambda_reg=lam)
    gram = sc.get_xtx(X)
    feats = sc.get_x_xtx_inv(X, gram)
    acc = torch.zeros(n, m)
    sc.get_scores(feats, T, acc)
    direct = torch.zeros(n, m)
    sc.get_scores_from_grads(X, gram, T, direct, row_scale=w)

    g_ref = br.xtx(X)
    inv_ref = br.xtx_inverse(g_ref, lam)
    f_ref = br.x_xtx_inv(X, g_ref, lam)
    s_ref = torch.zeros(n, m)
    br.scores(f_ref, T, s_ref)
    from trak_b200 import score_computers as scm
    inv = scm.spd_inverse_(gram.to(cuda).float().clone(), lam, rescale=True)
    errs = {"gram": rel(gram, g_ref), "inverse": rel(inv, inv_ref), "features": rel(feats, f_ref),
            "scores": rel(acc, s_ref), "scores_from_grads": rel(direct, br.finalize_scores_epilogue(s_ref, w, 1))}
    print("k = 8192 against the CPU port:", {a: f"{b:.2e}" for a, b in errs.items()})
    for name, e in errs.items():
        assert e <= TOL, (name, errs)


def test_inverse_at_8192_against_an_fp64_inverse(cuda):
    from trak_b200 import score_computers as sc
    k, lam = 8192, 1e-3
    g = torch.Generator(device=cuda).manual_seed(8192)
    A = torch.zeros(k, k, device=cuda, dtype=torch.float64)
    for _ in range(3):   # Gram of 3k rows of N(0, 1/k), formed block-wise in fp64
        y = torch.randn(k, k, device=cuda, generator=g, dtype=torch.float64) / k ** 0.5
        A += y.T @ y
    A32 = A.float()
    ref = torch.linalg.inv(A32.double() + lam * torch.eye(k, device=cuda, dtype=torch.float64))
    inv = sc.spd_inverse_(A32.clone(), lam, rescale=False)
    assert torch.equal(inv, inv.T)
    err = rel(inv, ref)
    assert err <= 2e-5, err
    inv2 = sc.spd_inverse_(A32.clone(), lam, rescale=True)
    assert rel(inv2, ref / ref.abs().mean()) <= 2e-5


def test_empty_row_block_contributes_a_zero_gram(cuda):
    """A rank whose shard holds no train rows (fewer rows than ranks) must still return a Gram, so that it
    reaches the all-reduce its peers are waiting in."""
    from trak_b200.score_computers import B200ScoreComputer
    sc = B200ScoreComputer(dtype=torch.float32, device=cuda, lambda_reg=1.0)
    g = sc.get_xtx(torch.zeros(0, 64))
    assert g.shape == (64, 64) and float(g.abs().sum()) == 0.0
    f = sc.get_x_xtx_inv(torch.zeros(0, 64), torch.eye(64))
    assert f.shape == (0, 64)
    # 16-bit gradients with an fp32 score computer: the block is promoted, the inverse keeps its precision
    X = torch.randn(500, 64, generator=torch.Generator().manual_seed(0)).half()
    gram = sc.get_xtx(X)
    feats = sc.get_x_xtx_inv(X, gram)
    ref = br.x_xtx_inv(X.float(), br.xtx(X.float()), 1.0)
    assert feats.dtype == torch.float32 and rel(feats, ref) <= 1e-4
