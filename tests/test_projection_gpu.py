"""Parity of the sm_100a projection (called through the C ABI via the fast_jl shim)
with the CPU oracle, with golden vectors from the reference's compiled kernel, and
with that kernel itself when its build is present.

Tolerance (floating point): per row, ||out - ref||_2 / ||ref||_2 <= 1e-3 against an
fp64 host matmul with the identical matrix.  Matrix entries themselves (one-hot
rows) must be bit-exact.
"""
import os

import numpy as np
import pytest
import torch

from oracle import jl_oracle as o
from oracle import build_ref

pytestmark = pytest.mark.gpu

TOL = 1e-3
RAD, NOR = 0, 1
DT = {"f16": torch.float16, "f32": torch.float32, "bf16": torch.bfloat16}


def rel_rows(out, ref):
    out = np.asarray(out, np.float64)
    ref = np.asarray(ref, np.float64)
    num = np.linalg.norm(out - ref, axis=1)
    den = np.maximum(np.linalg.norm(ref, axis=1), 1e-30)
    return float((num / den).max())


def as_numpy_input(t):
    return t.view(torch.uint16).numpy() if t.dtype == torch.bfloat16 else t.numpy()


def ours(g, N, seed, T, p, **kw):
    from trak_b200 import fast_jl
    return fast_jl.project(g, N, seed, T, p, **kw)


def one_hot(B, F, feats, dtype, device):
    g = torch.zeros(B, F, dtype=dtype, device=device)
    for i, f in enumerate(feats):
        g[i, f] = 1.0
    return g


SHAPES = [  # B, F, N, seed, tiles
    (8, 1000, 512, 0, 148),
    (31, 20000, 1024, 123, 108),
    (130, 5000, 512, 17, 7),      # more rows than one pass holds
    (1, 70001, 512, 5, 148),
    (5, 16, 512, 9, 148),         # fewer features than tiles
    (3, 1, 512, 2, 1),            # a single feature
    (16, 4096, 1536, 4, 4),       # tile size a multiple of 64
]


@pytest.mark.parametrize("p", [RAD, NOR])
@pytest.mark.parametrize("dt", ["f16", "f32", "bf16"])
@pytest.mark.parametrize("B,F,N,seed,T", SHAPES)
def test_parity_with_oracle(cuda, p, dt, B, F, N, seed, T):
    g_cpu = torch.randn(B, F, generator=torch.Generator().manual_seed(B * 1000 + F)).to(DT[dt])
    out = ours(g_cpu.to(cuda), N, seed, T, p).cpu().numpy()
    assert out.shape == (B, N) and out.dtype == np.float32
    if dt == "bf16" and p == NOR:
        # bf16 gradients meet the fp16-valued matrix rounded once more to bf16
        P = torch.from_numpy(o.matrix(NOR, F, N, seed, T)).to(torch.bfloat16).double().numpy()
        ref = g_cpu.double().numpy() @ P
    else:
        ref = o.project(p, as_numpy_input(g_cpu), N, seed, T, round_f16=(dt == "f32"))
    assert rel_rows(out, ref) <= TOL
    if dt == "f32":
        # still within tolerance of the fp64 product of the un-rounded fp32 gradients
        assert rel_rows(out, o.project(p, g_cpu.numpy(), N, seed, T)) <= TOL


@pytest.mark.parametrize("dt", ["f16", "f32", "bf16"])
@pytest.mark.parametrize("F,N,seed,T", [(1000, 512, 0, 148), (5000, 1024, 123, 108), (70000, 512, 7, 148)])
def test_rademacher_matrix_rows_bit_exact_vs_oracle(cuda, dt, F, N, seed, T):
    fts = o.feature_tile_size(F, T)
    feats = sorted({0, 1, 15, 16, 17, 63, 64, fts - 1, fts, fts + 1, F // 2, F - 1})
    out = ours(one_hot(len(feats), F, feats, DT[dt], cuda), N, seed, T, RAD).cpu().numpy()
    assert np.array_equal(out, o.matrix_rows(RAD, F, N, seed, T, feats))


def _golden(golden_dir):
    path = os.path.join(golden_dir, "fastjl_golden.npz")
    if not os.path.exists(path):
        pytest.fail("tests/golden/fastjl_golden.npz is missing")
    return np.load(path)


@pytest.mark.parametrize("case", [0, 1, 2, 3])
@pytest.mark.parametrize("name,p", [("rademacher", RAD), ("normal", NOR)])
def test_matrix_rows_bit_exact_vs_reference_kernel_golden(cuda, golden_dir, case, name, p):
    d = _golden(golden_dir)
    F, N, seed, T = (int(v) for v in d[f"rows_{case}_meta"])
    feats = d[f"rows_{case}_feats"].tolist()
    want = d[f"rows_{case}_{name}"].astype(np.float32)
    for dt in (torch.float16, torch.float32):
        out = ours(one_hot(8, F, feats, dt, cuda), N, seed, T, p).cpu().numpy()[:len(feats)]
        assert np.array_equal(out, want), f"{name} rows differ from the reference kernel ({dt})"


@pytest.mark.parametrize("case", [0, 1, 2])
def test_projection_vs_reference_kernel_golden(cuda, golden_dir, case):
    d = _golden(golden_dir)
    B, F, N, seed, T, in_seed = (int(v) for v in d[f"proj_{case}_meta"])
    base = torch.randn(B, F, generator=torch.Generator().manual_seed(in_seed))
    for dn, dt in (("f16", torch.float16), ("f32", torch.float32)):
        for name, p in (("rademacher", RAD), ("normal", NOR)):
            out = ours(base.to(dt).to(cuda), N, seed, T, p).cpu().numpy()
            assert rel_rows(out, d[f"proj_{case}_{dn}_{name}"]) <= TOL


def test_reference_known_answers_even_odd(cuda):
    # tests/test_rademacher.py:65-108 of the reference
    for F, parity in ((10240, 0), (10241, 1)):
        out = ours(torch.ones(8, F, dtype=torch.float16, device=cuda), 1024, 0, 148, RAD).cpu().numpy()
        assert np.all(np.mod(out, 2) == parity)


@pytest.mark.parametrize("F", [1024, 2048])
@pytest.mark.parametrize("N", [512, 1024, 2048])
def test_shape_all_entry_points(cuda, F, N):
    from trak_b200 import fast_jl
    g = torch.randn(8, F, device=cuda)
    for t in ("rademacher", "normal"):
        for b in (8, 16, 32):
            out = getattr(fast_jl, f"project_{t}_{b}")(g, N, 1, 148)
            assert out.shape == (8, N) and out.dtype == torch.float32 and out.device == g.device


def test_run_to_run_bit_identical(cuda):
    from trak_b200 import fast_jl
    g = torch.randn(32, 123457, device=cuda).half()
    for p in (RAD, NOR):
        a = ours(g, 2048, 123, 148, p)
        fast_jl.free_workspaces()
        b = ours(g, 2048, 123, 148, p)
        assert torch.equal(a, b)
        assert torch.equal(a[:7], ours(g[:7].contiguous(), 2048, 123, 148, p))  # rows independent


def test_alpha_accumulate_and_strided_rows(cuda):
    g = torch.randn(12, 3000, device=cuda).half()
    base = ours(g, 512, 3, 148, RAD)
    out = torch.full((12, 512), 2.0, device=cuda)
    ours(g, 512, 3, 148, RAD, alpha=0.5, out=out, accumulate=True)
    torch.testing.assert_close(out, 2.0 + 0.5 * base, rtol=1e-6, atol=1e-5)
    wide = torch.randn(12, 5000, device=cuda).half()
    wide[:, :3000] = g
    assert torch.equal(ours(wide[:, :3000], 512, 3, 148, RAD, allow_strided=True), base)
    odd = wide[:, 1:3000]  # rows start on odd (2-byte aligned) addresses
    assert torch.equal(ours(odd, 512, 3, 148, RAD, allow_strided=True),
                       ours(odd.contiguous(), 512, 3, 148, RAD))


def test_argument_errors_on_device(cuda):
    from trak_b200 import fast_jl
    g = torch.randn(8, 1000, device=cuda)
    with pytest.raises(ValueError, match="multiple of 512"):
        fast_jl.project_rademacher_8(g, 500, 0, 148)
    with pytest.raises(RuntimeError):
        fast_jl.project_rademacher_8(g.long(), 512, 0, 148)
    with pytest.raises(RuntimeError):
        fast_jl.project_rademacher_8(g.t(), 512, 0, 148)
    with pytest.raises(RuntimeError):
        fast_jl.project_rademacher_8(g[0], 512, 0, 148)
    with pytest.raises(TypeError):
        fast_jl.project_rademacher_8(g, 512, -1, 148)


def test_norm_and_inner_product_preservation(cuda):
    # statistical JL property (tests/test_jl.py:159-282 of the reference), at 1/sqrt(k) scale
    k = 4096
    g = torch.randn(16, 200000, device=cuda)
    for p in (RAD, NOR):
        y = ours(g, k, 11, 148, p).double() / k ** 0.5
        gd = g.double()
        ratio = (y.norm(dim=1) / gd.norm(dim=1)).cpu().numpy()
        assert np.all(np.abs(ratio - 1) < 0.1)
        ip = (y @ y.T - gd @ gd.T).abs().max().item() / (gd.norm(dim=1).max().item() ** 2)
        assert ip < 0.1


def test_projector_classes(cuda):
    from trak_b200 import projectors as pj
    torch.manual_seed(0)
    grads = {"w1": torch.randn(6, 40, 50, device=cuda), "b1": torch.randn(6, device=cuda),
             "w2": torch.randn(6, 3000, device=cuda)}
    D = 2000 + 1 + 3000
    proj = pj.CudaProjector(D, 1024, 5, pj.ProjectionType.rademacher, cuda, 32)
    flat = pj.vectorize(grads, device=cuda)
    a = proj.project(grads, model_id=2)
    ref = o.project(RAD, flat.cpu().numpy(), 1024, 5 + 20000, proj.num_sms, round_f16=True)
    assert rel_rows(a.cpu().numpy(), ref) <= TOL
    # chunked: [w1, b1] and [w2] with their own seeds, summed
    p0 = pj.CudaProjector(2001, 1024, 7, pj.ProjectionType.rademacher, cuda, 32)
    p1 = pj.CudaProjector(3000, 1024, 9, pj.ProjectionType.rademacher, cuda, 32)
    cp = pj.ChunkedCudaProjector([p0, p1], 3500, [2001, 3000], 8, cuda, torch.float32)
    got = cp.project(grads, model_id=0)
    want = p0.project(flat[:, :2001].contiguous(), 0) + p1.project(flat[:, 2001:].contiguous(), 0)
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-3)
    assert got.shape == (6, 1024)


def _chunked_like_the_reference_suite(g, proj_dim, seed, proj_type, dtype, cuda, n_chunks):
    """The projector set-up of the reference's tests/test_jl.py:394-443: the gradient split into column chunks
    (a dict, one entry per chunk), one CudaProjector per chunk with seeds from default_rng(seed), summed by
    ChunkedCudaProjector."""
    from trak_b200.projectors import CudaProjector, ChunkedCudaProjector
    chunks = dict(enumerate(torch.chunk(g, n_chunks, dim=1)))
    seeds = np.random.default_rng(seed).integers(low=0, high=500, size=len(chunks))
    sizes = [v.size(1) for v in chunks.values()]
    per_chunk = [CudaProjector(grad_dim=sz, proj_dim=proj_dim, seed=int(seeds[i]), proj_type=proj_type,
                               max_batch_size=32, dtype=dtype, device=cuda) for i, sz in enumerate(sizes)]
    return ChunkedCudaProjector(per_chunk, max(sizes), sizes, g.shape[0], cuda, dtype), chunks


@pytest.mark.parametrize("ptype", ["rademacher", "normal"])
@pytest.mark.parametrize("dt", [torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(1, 25), (8, 10_000), (16, 10_002), (9, 10_002), (45, 1049)])
def test_properties_of_the_reference_suite(cuda, ptype, dt, shape):
    """The property tests of the reference's own suite, on its shapes (tests/test_jl.py:46-56), through the same
    classes: equal rows give equal projections (test_same_features), every output depends on every feature
    (test_single_nonzero_feature), orthogonal rows stay nearly orthogonal (test_orthogonality), the same seed gives
    the same projection and another seed another one (test_seed_consistency)."""
    from trak_b200.projectors import CudaProjector, ProjectionType
    pt = ProjectionType(ptype)
    B, F = shape
    gen = torch.Generator(device=cuda).manual_seed(F + B)
    for proj_dim in (1024, 4096):
        g = (torch.rand(B, F, device=cuda, generator=gen) * 2 - 1).to(dt)
        g[-1] = g[0]
        proj, chunks = _chunked_like_the_reference_suite(g, proj_dim, 10 ** 8, pt, dt, cuda, n_chunks=min(3, F))
        p = proj.project(chunks, model_id=0)
        assert p.shape == (B, proj_dim) and torch.equal(p[0], p[-1])
        # one non-zero feature per row, anywhere: no output stays zero
        z = torch.zeros(B, F, device=cuda, dtype=dt)
        cols = torch.randint(0, F, (B,), generator=torch.Generator().manual_seed(B))
        z[torch.arange(B), cols] = torch.randn(B, generator=torch.Generator().manual_seed(F)).to(dt).to(cuda) + 2.0
        single = CudaProjector(grad_dim=F, proj_dim=proj_dim, seed=1, proj_type=pt, device=cuda, max_batch_size=32)
        q = single.project(z, model_id=0)
        assert bool((q != 0).all())
        assert torch.equal(q, single.project(z, model_id=0))
        other = CudaProjector(grad_dim=F, proj_dim=proj_dim, seed=2, proj_type=pt, device=cuda, max_batch_size=32)
        assert not torch.equal(q, other.project(z, model_id=0))
        # (the Rademacher bits of a stream's first draws are the same for seeds 10^4 apart -- a property of the
        # reference's seeding that the oracle reproduces -- so another model_id is compared on dense rows)
        if F >= 1000:
            assert not torch.equal(single.project(g, model_id=0), single.project(g, model_id=1))
        if B > 1 and F >= 1000:
            # the reference's criterion (tests/test_jl.py:451-497) is that of ten orthogonal pairs more than a
            # third project to an inner product below 1e-3; here the cosine itself is bounded.  Gaussian matrix
            # only: with feature tiles of a few 16-feature chunks (F / 148 features per tile) the Rademacher
            # matrix consists of the first draws of XORWOW streams whose seeds are in arithmetic progression,
            # which are strongly correlated -- cosines of 0.3 to 0.4 at these sizes, with the oracle's matrix as
            # with this kernel's: a property of the matrix definition, which large models (thousands of chunks
            # per tile) do not show (test_norm_and_inner_product_preservation)
            if pt != ProjectionType.normal:
                continue
            wins, worst = 0, 0.0
            for _ in range(10):
                a = torch.rand(B, F, device=cuda, generator=gen) * 2 - 1
                a[-1] -= (a[0] @ a[-1]) / a[0].norm() ** 2 * a[0]
                r = single.project(a.to(dt), model_id=0)
                wins += int(float(r[0] @ r[-1]) < 1e-3)
                worst = max(worst, abs(float(r[0] @ r[-1] / (r[0].norm() * r[-1].norm()))))
            assert wins > 0.33 * 10 and worst < 6.0 / proj_dim ** 0.5, (wins, worst)


@pytest.mark.parametrize("dt", ["f16", "f32", "bf16"])
@pytest.mark.parametrize("B", [5, 140])
def test_segments_equal_concatenation(cuda, dt, B):
    """Projecting straight from per-parameter tensors gives the bits of projecting their concatenation."""
    from trak_b200 import fast_jl
    torch.manual_seed(B)
    shapes = [(64, 3, 3, 3), (), (17,), (129, 31), (1,), (300, 7, 2), (5,)]   # () and (n,) as vectorize sees them
    tensors = [torch.randn((B,) + sh, device=cuda).to(DT[dt]) for sh in shapes]
    flat = torch.cat([t.reshape(B, 1) if t.dim() < 2 else t.flatten(start_dim=1) for t in tensors], dim=1)
    for p in (RAD, NOR):
        a = fast_jl.project_segments(tensors, 1024, 21, 148, p)
        b = fast_jl.project(flat.contiguous(), 1024, 21, 148, p)
        assert torch.equal(a, b)
    out = torch.ones(B, 512, device=cuda)
    fast_jl.project_segments(tensors, 512, 3, 148, RAD, alpha=2.0, out=out, accumulate=True)
    torch.testing.assert_close(out, 1.0 + 2.0 * fast_jl.project(flat.contiguous(), 512, 3, 148, RAD),
                               rtol=1e-6, atol=1e-4)


def test_full_size_properties(cuda):
    """The benchmark's shape (128 x 11,173,962 fp16 -> 4096, 148 tiles): matrix rows at the far end
    of the feature range against the oracle, linearity and run-to-run identity."""
    B, F, N, seed, T = 128, 11_173_962, 4096, 17, 148
    fts = o.feature_tile_size(F, T)
    assert fts == 75500
    feats = [0, fts - 1, fts * 147, F - 1]
    g = torch.zeros(B, F, dtype=torch.float16, device=cuda)
    for i, f in enumerate(feats):
        g[i, f] = 1.0
    g[4:] = (torch.randn(B - 4, F, device=cuda) * 1e-2).half()
    rad = ours(g, N, seed, T, RAD)
    assert np.array_equal(rad[:4].cpu().numpy(), o.matrix_rows(RAD, F, N, seed, T, feats))
    nor = ours(g, N, seed, T, NOR)
    want = o.matrix_rows(NOR, F, N, seed, T, feats[:2] + feats[3:])
    got = nor[[0, 1, 3]].cpu().numpy()
    # host libm vs device logf / __sincosf (absolute error ~1e-6 before the fp16 rounding):
    # equal except for a last-place difference on a small fraction of entries
    assert (got != want).mean() < 0.01
    np.testing.assert_allclose(got, want, rtol=2 ** -10, atol=4e-6)
    assert torch.equal(nor, ours(g, N, seed, T, NOR))
    # linearity on exactly representable combinations: P(a) + P(b) == P(a + b) for one-hot a, b
    s = torch.zeros(8, F, dtype=torch.float16, device=cuda)
    s[0, feats[0]] = 1.0
    s[0, feats[3]] = 1.0
    both = ours(s, N, seed, T, RAD)[0]
    assert torch.equal(both, rad[0] + rad[3])
    # norms: E||Pg||^2 = k ||g||^2
    ratio = (rad[4:].double().norm(dim=1) / (g[4:].double().norm(dim=1) * N ** 0.5)).cpu().numpy()
    assert np.all(np.abs(ratio - 1) < 0.05)


def test_randomised_shapes_against_oracle_rows_and_projection(cuda):
    """Forty seeded random shapes (feature counts around tile and stage boundaries, tile counts that leave the
    generator groups uneven work, batches on both sides of the 64 / 128 / 256-row shape switches): matrix rows
    bit-exact (Rademacher), projections within tolerance (both types)."""
    rng = np.random.default_rng(2024)
    for case in range(40):
        T = int(rng.choice([1, 2, 3, 5, 7, 37, 108, 148, 149, 1000]))
        F = int(rng.choice([1, 15, 16, 17, 63, 64, 65, 1000, 4097, 9472, 9473, 75_531, 200_003]))
        N = int(rng.choice([512, 1024, 2560]))
        B = int(rng.choice([1, 7, 16, 17, 64, 65, 128, 129, 200, 257, 300]))
        if B * F > 20_000_000:
            B = max(1, 20_000_000 // F)
        seed = int(rng.integers(0, 2 ** 32))
        dt = ["f16", "f32", "bf16"][case % 3]
        g_cpu = torch.randn(B, F, generator=torch.Generator().manual_seed(case)).to(DT[dt])
        # the first rows are one-hot at boundary features
        fts = o.feature_tile_size(F, T)
        feats = sorted({0, F - 1, min(F - 1, fts), max(0, fts - 1), F // 2})[:B]
        for i, f in enumerate(feats):
            g_cpu[i].zero_()
            g_cpu[i, f] = 1.0
        g = g_cpu.to(cuda)
        rad = ours(g, N, seed, T, RAD).cpu().numpy()
        assert np.array_equal(rad[:len(feats)], o.matrix_rows(RAD, F, N, seed, T, feats)), (case, T, F, N, B, dt)
        if B * F * N <= 3e11:
            ref = o.project(RAD, as_numpy_input(g_cpu), N, seed, T, round_f16=(dt == "f32"))
            assert rel_rows(rad, ref) <= TOL, (case, T, F, N, B, dt)
            if dt != "bf16":
                nor = ours(g, N, seed, T, NOR).cpu().numpy()
                refn = o.project(NOR, as_numpy_input(g_cpu), N, seed, T, round_f16=(dt == "f32"))
                assert rel_rows(nor, refn) <= TOL, (case, T, F, N, B, dt)


_big_rows = {}   # oracle rows of the large shapes (20 s of host time), shared by the cases below


@pytest.mark.parametrize("B,F", [(8, 180_645_096), (32, 180_645_096), (2, 780_645_096)])
def test_large_feature_count_and_projection_dim(cuda, B, F):
    """The shapes of the reference's overflow tests (tests/test_jl.py:59-73: fp32, k = 15,360, seed 123): 8 rows of
    180,645,096 features, which the reference handles, and 32 rows of them and 2 rows of 780,645,096, which it
    marks as failing (its row offsets are 32-bit, fast_jl/data_loading.cuh:37-41).  64-bit addressing in the
    restaging pass, matrix rows deep inside feature tiles of 1.2 and 5.3 million features (20 and 80 accumulation
    chains per tile): one-hot rows bit for bit against the oracle's matrix, an exactly representable combination
    of them in the last row, zeros elsewhere."""
    N, seed, T = 15_360, 123, 148
    need = B * F * 4 + o.feature_tile_size(F, T) * T * 16 * 2 * 2 + (8 << 30)
    if torch.cuda.mem_get_info(cuda)[0] < need:
        pytest.skip("not enough free device memory for this shape")
    fts = o.feature_tile_size(F, T)
    # the oracle walks a stream draw by draw, so the one feature of the two-row case sits early in the last tile
    feats = [0, fts - 1, 5 * fts + 12_345, F - 1][:B - 1] if B > 2 else [147 * fts + 100_003]
    coef = [0.5, -2.0, 3.0, -0.25][:len(feats)]
    g = torch.zeros(B, F, dtype=torch.float32, device=cuda)
    for i, f in enumerate(feats):
        g[i, f] = 1.0
        g[B - 1, f] = coef[i]
    out = ours(g, N, seed, T, RAD)
    del g
    from trak_b200 import fast_jl
    fast_jl.free_workspaces()       # tens of GB of staging for these shapes: not kept for the tests that follow
    torch.cuda.empty_cache()
    key = (F, tuple(feats))
    if key not in _big_rows:
        _big_rows[key] = o.matrix_rows(RAD, F, N, seed, T, feats)
    rows = _big_rows[key]
    assert np.array_equal(out[:len(feats)].cpu().numpy(), rows)
    want = sum(np.float32(c) * r for c, r in zip(coef, rows))        # +-c_i: every partial sum is exact in fp32
    assert np.array_equal(out[B - 1].cpu().numpy(), want)
    if B - 1 > len(feats):
        assert float(out[len(feats):B - 1].abs().max()) == 0.0


# ---- against the compiled reference kernel itself, when it travelled with the repo ----

def _witness():
    w = build_ref.load()
    if w is None:
        pytest.skip("oracle/_ref/fast_jl.so not built (run oracle/build_ref.py where the reference is)")
    return w


@pytest.mark.parametrize("B,F,N,seed,T", [(8, 1000, 512, 0, 148), (32, 100000, 4096, 123, 108),
                                          (16, 33333, 1024, 5, 148)])
def test_bit_exact_matrix_and_parity_vs_reference_kernel(cuda, B, F, N, seed, T):
    w = _witness()
    fts = o.feature_tile_size(F, T)
    feats = [0, 1, 15, 16, fts - 1, fts, F // 2, F - 1][:B]
    for dt in (torch.float16, torch.float32):
        g1 = one_hot(B, F, feats, dt, cuda)
        g = torch.randn(B, F, device=cuda).to(dt)
        for name, p in (("rademacher", RAD), ("normal", NOR)):
            ref_fn = getattr(w, f"project_{name}_32")
            assert torch.equal(ours(g1, N, seed, T, p), ref_fn(g1, N, seed, T))
            assert rel_rows(ours(g, N, seed, T, p).cpu().numpy(), ref_fn(g, N, seed, T).cpu().numpy()) <= TOL


def test_full_benchmark_shape_all_rows_against_the_reference_kernel(cuda):
    """The benchmark's own launch (fp16 [128 x 11,173,962] -> 4096, seed 17, 148 tiles), every row, both
    matrix types, against the reference's compiled kernel on the same input: one-hot rows (matrix entries at
    the ends of the feature range and of a tile) bit for bit, the 120 random rows within tolerance."""
    w = _witness()
    B, F, N, seed, T = 128, 11_173_962, 4096, 17, 148
    fts = o.feature_tile_size(F, T)
    feats = [0, 1, 15, 16, fts - 1, fts, 73 * fts + 40_001, F - 1]
    g = (torch.randn(B, F, device=cuda, generator=torch.Generator(device=cuda).manual_seed(1000)) * 1e-2).half()
    for i, f in enumerate(feats):
        g[i].zero_()
        g[i, f] = 1.0
    rows, groups = [8, 9, 64, 127], [0, 77]
    cols = np.concatenate([np.arange(32 * c, 32 * c + 32) for c in groups])
    g_rows = g[rows].cpu().numpy()
    for name, p in (("rademacher", RAD), ("normal", NOR)):
        got = ours(g, N, seed, T, p)
        ref = getattr(w, f"project_{name}_32")(g, N, seed, T)
        assert torch.equal(got[:len(feats)], ref[:len(feats)]), name
        # four random rows on 64 columns against the fp64 product with the identical matrix: what the long
        # tensor-core accumulations (302,000 features per CTA, truncating fp32 adds) cost at this size
        exact = o.project_column_groups(p, g_rows, seed, T, groups)
        mine = got[rows][:, cols].double().cpu().numpy()
        theirs = ref[rows][:, cols].double().cpu().numpy()
        e_mine = (np.linalg.norm(mine - exact, axis=1) / np.linalg.norm(exact, axis=1)).max()
        e_ref = (np.linalg.norm(theirs - exact, axis=1) / np.linalg.norm(exact, axis=1)).max()
        print(f"{name}: against the fp64 oracle on 64 columns: this library {e_mine:.2e}, reference kernel {e_ref:.2e}")
        assert e_mine <= TOL, (name, e_mine)
        err = ((got - ref).double().norm(dim=1) / ref.double().norm(dim=1))[len(feats):].max().item()
        print(f"{name}: 120 random rows against the reference kernel, worst row {err:.2e}")
        assert err <= TOL, (name, err)
        del got, ref
        # the same launch timed on both (CUDA events on the current stream, 3 calls after a warm-up each; the
        # reference kernel runs on the legacy default stream, which the current stream synchronises with)
        ms = {}
        for who, fn in (("ours", lambda: ours(g, N, seed, T, p, strict=False)),
                        ("reference", lambda: getattr(w, f"project_{name}_32")(g, N, seed, T))):
            fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(3):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms[who] = e0.elapsed_time(e1) / 3
        print(f"{name}, 128 x 11,173,962 -> 4096: reference fast_jl kernel {ms['reference']:.1f} ms, "
              f"this library {ms['ours']:.1f} ms ({ms['reference'] / ms['ours']:.1f}x)")
        assert ms["reference"] >= 3.0 * ms["ours"], ms


WIDE_SHAPES = [  # B, F, N, seed, tiles, dtype: batches that take the 512-row Gaussian kernel
    (512, 20011, 1024, 17, 148, "f16"),
    (300, 75_531, 512, 5, 37, "bf16"),
    (257, 9473, 512, 99, 7, "f32"),     # fewer tiles than generator groups
    (600, 3001, 512, 3, 148, "f16"),    # 512 rows, then 88 through the narrow kernel
    (384, 4096, 1536, 4, 4, "f16"),     # tile size a multiple of 64
    (290, 130, 512, 8, 148, "f32"),     # fewer features than tiles
]


@pytest.mark.parametrize("B,F,N,seed,T,dt", WIDE_SHAPES)
def test_wide_gaussian_batches(cuda, B, F, N, seed, T, dt):
    """More than 256 rows of a Gaussian projection go through one generation of the matrix (operand staged
    in shared memory).  One-hot rows must give the very bits the narrow kernel gives (which the tests above
    tie to the reference kernel); random rows are checked against the fp64 oracle."""
    g_cpu = (torch.randn(B, F, generator=torch.Generator().manual_seed(B + F)) * 1e-1).to(DT[dt])
    fts = o.feature_tile_size(F, T)
    feats = sorted({0, 1, min(F - 1, 15), min(F - 1, 16), min(F - 1, fts - 1), min(F - 1, fts), F // 2, F - 1})
    hot_rows = [0, 1, 2, 100, 255, 256, B - 2, B - 1][:len(feats)]   # spread over both halves of the batch
    for r, f in zip(hot_rows, feats):
        g_cpu[r].zero_()
        g_cpu[r, f] = 1.0
    g = g_cpu.to(cuda)
    wide = ours(g, N, seed, T, NOR)
    narrow = torch.cat([ours(g[i:i + 200].contiguous(), N, seed, T, NOR) for i in range(0, B, 200)])
    assert torch.equal(wide[hot_rows], narrow[hot_rows])
    # both kernels accumulate in the tensor core's truncating fp32, in different orders: about 1e-5 apart
    assert rel_rows(wide.cpu().numpy(), narrow.cpu().numpy()) <= 1e-4
    assert torch.equal(wide, ours(g, N, seed, T, NOR))            # run-to-run identical
    if B * F * N <= 6e12:
        ref = o.project(NOR, as_numpy_input(g_cpu), N, seed, T, round_f16=(dt == "f32"))
        keep = [r for r in range(B) if r not in hot_rows]
        # for bf16 gradients the kernel rounds the fp16-valued matrix once more to bf16 (about 2^-9 per entry,
        # unbiased): the rows are still within tolerance of the oracle's fp16-valued matrix
        assert rel_rows(wide.cpu().numpy()[keep], ref[keep]) <= (TOL if dt != "bf16" else 4e-3)
    # alpha and accumulation through the wide path
    out = torch.full((B, N), 0.5, device=cuda)
    ours(g, N, seed, T, NOR, alpha=0.25, out=out, accumulate=True)
    torch.testing.assert_close(out, 0.5 + 0.25 * wide, rtol=1e-6, atol=1e-5)


def test_randomised_wide_shapes_against_the_narrow_kernel(cuda):
    """Sixteen seeded random shapes for the 512-row Gaussian kernel (row counts on both sides of a pass, feature
    counts around tile and stage boundaries, tile counts that leave generator groups idle or give ragged last
    bundles): the same input through 200-row calls (narrow kernel) must agree to fp32 summation order (the tensor
    core's accumulation truncates, so two orders differ by about 1e-5), one-hot rows bit for bit."""
    rng = np.random.default_rng(7)
    for case in range(16):
        T = int(rng.choice([1, 2, 6, 7, 8, 13, 37, 108, 148, 149, 500]))
        F = int(rng.choice([1, 31, 32, 33, 63, 64, 65, 1000, 4097, 9473, 30_011]))
        N = int(rng.choice([512, 1024, 2560]))
        B = int(rng.choice([257, 258, 288, 300, 333, 511, 512, 513, 700, 1025]))
        seed = int(rng.integers(0, 2 ** 32))
        dt = ["f16", "f32", "bf16"][case % 3]
        g = (torch.randn(B, F, device=cuda, generator=torch.Generator(device=cuda).manual_seed(case)) * 0.1).to(DT[dt])
        hot = sorted({0, F - 1, F // 2})
        rows = [0, 256, B - 1][:len(hot)]
        for r, f in zip(rows, hot):
            g[r].zero_()
            g[r, f] = 1.0
        wide = ours(g, N, seed, T, NOR)
        narrow = torch.cat([ours(g[i:i + 200].contiguous(), N, seed, T, NOR) for i in range(0, B, 200)])
        assert torch.equal(wide[rows], narrow[rows]), (case, T, F, N, B, dt)
        assert rel_rows(wide.cpu().numpy(), narrow.cpu().numpy()) <= 1e-4, (case, T, F, N, B, dt)


def test_wide_gaussian_from_segments(cuda):
    from trak_b200 import fast_jl
    B = 320
    shapes = [(64, 3, 3, 3), (), (17,), (129, 31), (300, 7, 2)]
    tensors = [torch.randn((B,) + sh, device=cuda) for sh in shapes]
    flat = torch.cat([t.reshape(B, 1) if t.dim() < 2 else t.flatten(start_dim=1) for t in tensors], dim=1)
    a = fast_jl.project_segments(tensors, 1024, 21, 148, NOR)
    assert torch.equal(a, fast_jl.project(flat.contiguous(), 1024, 21, 148, NOR))


CHAIN_SHAPES = [  # B, F, tiles: feature tiles long enough for several accumulation chains per tile
    (128, 98_304, 3),     # 32,768 features per tile: a whole number of chains for every kernel shape; NG > tiles
    (128, 200_003, 5),    # ragged last chain; more tiles than generator groups of the 128-row shapes
    (8, 150_001, 2),      # small batch: the generator-bound shape for both matrix types
    (256, 120_007, 3),    # the 256-row shapes
    (300, 98_304, 3),     # Gaussian: the 512-row kernel (32-feature stages), then nothing left
    (300, 131_075, 9),    # Gaussian: 512-row kernel with more tiles than its seven groups
]


@pytest.mark.parametrize("p", [RAD, NOR])
@pytest.mark.parametrize("B,F,T", CHAIN_SHAPES)
def test_accumulation_chains(cuda, p, B, F, T):
    """The accumulators are read out and restarted every 2048 / 4096 MMA steps of a feature tile and at its end.
    Feature tiles of 15,000 to 75,000 features make every kernel shape run several chains per tile, with chain ends
    that do and do not coincide with the tile's end, with generator groups that have no tile at all, and with
    groups that finish before the others: results against the fp64 oracle on four 32-column groups, one-hot rows
    bit for bit against the oracle's matrix, the stored-matrix kernel against the regenerating one."""
    from trak_b200 import fast_jl
    N, seed = 1024, 29
    g_cpu = (torch.randn(B, F, generator=torch.Generator().manual_seed(B + F + T)) * 0.1).half()
    fts = o.feature_tile_size(F, T)
    feats = [0, fts - 1, fts, F // 2, F - 1][:B]
    for r, f in enumerate(feats):
        g_cpu[r].zero_()
        g_cpu[r, f] = 1.0
    g = g_cpu.to(cuda)
    out = ours(g, N, seed, T, p)
    assert torch.equal(out, ours(g, N, seed, T, p))                      # run-to-run identical
    groups = [0, 7, 16, 31]
    cols = np.concatenate([np.arange(32 * c, 32 * c + 32) for c in groups])
    ref = o.project_column_groups(p, g_cpu.numpy(), seed, T, groups)
    got = out.cpu().numpy()[:, cols]
    # one-hot rows are single matrix entries: exact whatever the number of chains (the oracle's Gaussian entries
    # come from the host's libm, so that matrix is compared through a small batch of the same rows instead)
    if p == RAD:
        assert np.array_equal(out.cpu().numpy()[:len(feats)], o.matrix_rows(p, F, N, seed, T, feats))
    else:
        assert torch.equal(out[:len(feats)], ours(g[:len(feats)].contiguous(), N, seed, T, p))
    err = rel_rows(got[len(feats):], ref[len(feats):])
    assert err <= 1e-4, err      # short chains: well inside the 1e-3 tolerance of the projection
    m = fast_jl.StoredMatrix(F, N, seed, T, p, dtype=torch.float16, device=cuda)
    stored = ours(g, N, seed, T, p, matrix=m)
    assert torch.equal(stored[:len(feats)], out[:len(feats)])
    assert rel_rows(stored.cpu().numpy()[:, cols][len(feats):], ref[len(feats):]) <= 1e-4


STORED_SHAPES = [  # B, F, N, seed, tiles, dtype
    (16, 20011, 1024, 17, 148, "f16"),
    (130, 9473, 512, 5, 7, "f32"),
    (300, 4097, 512, 99, 37, "bf16"),     # two passes of the stored-matrix kernel
    (5, 16, 512, 9, 148, "f16"),          # fewer features than tiles
    (64, 4096, 1536, 4, 4, "f16"),        # tile size a multiple of 64
]


@pytest.mark.parametrize("p", [RAD, NOR])
@pytest.mark.parametrize("B,F,N,seed,T,dt", STORED_SHAPES)
def test_stored_matrix_projection(cuda, p, B, F, N, seed, T, dt):
    """The matrix materialised once in device memory and read back by a plain two-operand GEMM: one-hot rows
    must give the very bits of the on-the-fly generator, random rows agree to fp32 summation order and with the
    fp64 oracle."""
    from trak_b200 import fast_jl
    g_cpu = (torch.randn(B, F, generator=torch.Generator().manual_seed(B + F)) * 0.1).to(DT[dt])
    fts = o.feature_tile_size(F, T)
    feats = sorted({0, min(F - 1, 15), min(F - 1, 16), min(F - 1, fts - 1), min(F - 1, fts), F - 1})[:B]
    for r, f in enumerate(feats):
        g_cpu[r].zero_()
        g_cpu[r, f] = 1.0
    g = g_cpu.to(cuda)
    m = fast_jl.StoredMatrix(F, N, seed, T, p, dtype=DT[dt], device=cuda)
    assert m.data.numel() == fast_jl.StoredMatrix.nbytes(F, N, T) >= 2 * F * N
    stored = ours(g, N, seed, T, p, matrix=m)
    fly = ours(g, N, seed, T, p)
    assert torch.equal(stored[:len(feats)], fly[:len(feats)])
    assert rel_rows(stored.cpu().numpy(), fly.cpu().numpy()) <= 1e-4
    assert torch.equal(stored, ours(g, N, seed, T, p, matrix=m))          # run-to-run identical
    if dt != "bf16" or p == RAD:
        ref = o.project(p, as_numpy_input(g_cpu), N, seed, T, round_f16=(dt == "f32"))
        assert rel_rows(stored.cpu().numpy(), ref) <= TOL
    out = torch.full((B, N), 0.5, device=cuda)
    ours(g, N, seed, T, p, matrix=m, alpha=0.25, out=out, accumulate=True)
    torch.testing.assert_close(out, 0.5 + 0.25 * stored, rtol=1e-6, atol=1e-5)
    with pytest.raises(RuntimeError):
        ours(g, N, seed + 1, T, p, matrix=m)      # a matrix of another seed is refused


def test_stored_matrix_through_the_projector_and_from_segments(cuda):
    from trak_b200 import fast_jl
    from trak_b200.projectors import CudaProjector, ProjectionType
    B = 40
    shapes = [(64, 3, 3, 3), (), (17,), (129, 31), (300, 7, 2)]
    grads = {i: torch.randn((B,) + sh, device=cuda) for i, sh in enumerate(shapes)}
    D = sum(int(np.prod(sh)) if len(sh) else 1 for sh in shapes)
    plain = CudaProjector(D, 1024, 3, ProjectionType.normal, cuda, 32)
    keep = CudaProjector(D, 1024, 3, ProjectionType.normal, cuda, 32, store_matrix=True)
    for model_id in (0, 1, 0):                      # a new model_id means a new seed: the matrix is replaced
        a, b = plain.project(grads, model_id), keep.project(grads, model_id)
        assert rel_rows(b.cpu().numpy(), a.cpu().numpy()) <= 1e-4
        assert keep._matrix is not None and keep._matrix.seed == 3 + 10_000 * model_id
    flat = torch.cat([t.reshape(B, 1) if t.dim() < 2 else t.flatten(start_dim=1) for t in grads.values()], dim=1)
    assert torch.equal(keep.project(grads, 0), keep.project(flat.contiguous(), 0))   # segments == dense
    keep.free_memory()
    assert keep._matrix is None


def test_stored_matrix_mode_of_the_entry_points(cuda, monkeypatch):
    """``store_matrices(True)`` (env TRAK_B200_STORE_MATRIX=1): the six-function interface the reference's own
    CudaProjector calls keeps the Gaussian matrix of the current (shape, seed) on the device.  Same results, one
    matrix per device, replaced when the seed changes, never used for the Rademacher matrix, skipped when it does
    not fit, argument errors unchanged."""
    from trak_b200 import fast_jl
    F, N, T = 20011, 1024, 148
    g = (torch.randn(40, F, generator=torch.Generator().manual_seed(3)) * 0.1).half()
    g[0].zero_()
    g[0, 777] = 1.0
    g = g.to(cuda)
    plain = fast_jl.project_normal_32(g, N, 5, T)
    fast_jl.store_matrices(True)
    try:
        a = fast_jl.project_normal_32(g, N, 5, T)
        m = fast_jl._stored[cuda.index]
        assert (m.F, m.N, m.seed, m.tiles) == (F, N, 5, T)
        assert torch.equal(a[0], plain[0]) and rel_rows(a.cpu().numpy(), plain.cpu().numpy()) <= 1e-4
        b = fast_jl.project_normal_8(g[:8].contiguous(), N, 5, T)
        assert fast_jl._stored[cuda.index] is m                      # the same matrix serves the next batch
        assert torch.equal(b[0], plain[0]) and rel_rows(b.cpu().numpy(), plain[:8].cpu().numpy()) <= 1e-4
        c = fast_jl.project_normal_16(g, N, 6, T)                    # next checkpoint: the matrix is replaced
        assert fast_jl._stored[cuda.index].seed == 6 and len(fast_jl._stored) == 1
        assert rel_rows(c.cpu().numpy(), ours(g, N, 6, T, NOR).cpu().numpy()) <= 1e-4
        r = fast_jl.project_rademacher_32(g, N, 5, T)
        assert fast_jl._stored[cuda.index].seed == 6                 # untouched by the Rademacher entry points
        assert torch.equal(r, ours(g, N, 5, T, RAD))
        with pytest.raises(ValueError):
            fast_jl.project_normal_32(g, 100, 5, T)
        with pytest.raises(RuntimeError):
            fast_jl.project_normal_32(g.cpu(), N, 5, T)
        # a matrix that would not leave the caller its headroom is not stored; the call regenerates as usual
        monkeypatch.setattr(fast_jl, "_STORE_HEADROOM", 1 << 60)
        d = fast_jl.project_normal_32(g, N, 7, T)
        assert cuda.index not in fast_jl._stored and len(fast_jl._does_not_fit) == 1
        assert torch.equal(d, ours(g, N, 7, T, NOR))
    finally:
        fast_jl.store_matrices(False)
    assert not fast_jl._stored and not fast_jl._does_not_fit


def test_bounded_wait_times_out_and_device_stays_usable(cuda):
    """Failure detection without a fault: a wait that nothing satisfies gives up after its limit, the
    status word reports it, and the next call works."""
    import time
    from trak_b200 import _lib, fast_jl
    lib = _lib.lib()
    _lib.device_status(cuda.index)
    t0 = time.time()
    assert lib.tb_selftest_wait_timeout(cuda.index, None, 100) == 0
    with pytest.raises(_lib.DeviceTimeout):
        _lib.device_status(cuda.index)
    assert 0.09 < time.time() - t0 < 5.0
    _lib.device_status(cuda.index)                      # the word was cleared
    g = torch.ones(8, 1024, dtype=torch.float16, device=cuda)
    assert np.all(np.mod(fast_jl.project_rademacher_8(g, 512, 0, 148).cpu().numpy(), 2) == 0)


def test_generator_square_root_is_exact_on_every_possible_draw(cuda):
    """The Gaussian generator's shortened square root against sqrtf on all 2^32 draws (bit for bit)."""
    from trak_b200 import _lib
    lib = _lib.lib()
    bad = torch.zeros(1, dtype=torch.int64, device=cuda)
    total = 0
    for first in range(0, 1 << 32, 1 << 30):
        assert lib.tb_selftest_sqrt(cuda.index, None, first, 1 << 30, bad.data_ptr()) == 0
        torch.cuda.synchronize()
        total += int(bad.item())
    assert total == 0, f"{total} draws give a different square root"


def test_device_status_clean(cuda):
    from trak_b200 import _lib
    _lib.device_status(cuda.index)
