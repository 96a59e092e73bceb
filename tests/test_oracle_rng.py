"""Pins the RNG core of the CPU oracle: XORWOW seeded like curand_init(seed, 0, 0)
and the Box-Muller pairing of curand_normal, against known answers from NVIDIA's
cuRAND host generator (recorded values, plus a live cross-check when libcurand
can be loaded), and the two independent restatements against each other."""
import ctypes

import numpy as np
import pytest

from oracle import jl_oracle as o

# first four draws of curand_init(seed, 0, 0) XORWOW streams, taken from
# curandGenerate on a host generator (output index i*4096 is draw i of the stream)
KAT = {
    0: [3179217846, 1883133293, 2220552389, 674260989],
    123: [2080129350, 3958764955, 514776033, 3365353227],
    3290526197: [3371806399, 3180219577, 2830466343, 3563060809],
}


def test_xorwow_known_answers():
    for seed, want in KAT.items():
        assert o.xorwow_draws(seed, 4).tolist() == want


def test_box_muller_known_answer():
    # curandGenerateNormal, seed 123: out[0] = s*sin(v), out[1] = s*cos(v) from draws 0, 1
    d = o.xorwow_draws(123, 2)
    got = o.box_muller(int(d[0]), int(d[1]))
    np.testing.assert_allclose(got, [-0.5686642, 1.0614371], rtol=2e-7)


def _curand():
    try:
        return ctypes.CDLL("libcurand.so")
    except OSError:
        try:
            return ctypes.CDLL("/usr/local/cuda/lib64/libcurand.so")
        except OSError:
            return None


@pytest.mark.parametrize("seed", [1, 17, 658105236, 0xFFFFFFFF])
def test_xorwow_against_live_curand_host(seed):
    cr = _curand()
    if cr is None:
        pytest.skip("libcurand not loadable here")
    gen = ctypes.c_void_p()
    assert cr.curandCreateGeneratorHost(ctypes.byref(gen), 101) == 0  # CURAND_RNG_PSEUDO_XORWOW
    try:
        assert cr.curandSetPseudoRandomGeneratorSeed(gen, ctypes.c_ulonglong(seed)) == 0
        n = 6
        buf = np.empty(4096 * n, np.uint32)
        assert cr.curandGenerate(gen, buf.ctypes.data_as(ctypes.c_void_p), ctypes.c_size_t(buf.size)) == 0
        assert o.xorwow_draws(seed, n).tolist() == buf[::4096].tolist()
    finally:
        cr.curandDestroyGenerator(gen)


@pytest.mark.parametrize("ptype", [o.RADEMACHER, o.NORMAL])
@pytest.mark.parametrize("F,N,seed,T", [(1000, 512, 7, 13), (300, 64, 0, 148), (4099, 96, 99, 5)])
def test_structural_and_closed_form_restatements_agree(ptype, F, N, seed, T):
    fts = o.feature_tile_size(F, T)
    feats = sorted({0, 1, 15, 16, 17, fts - 1, fts % F, (fts + 1) % F, F // 2, F - 1})
    a = o.matrix_rows(ptype, F, N, seed, T, feats)
    b = o.matrix_entries_closed_form(ptype, F, N, seed, T, feats)
    if ptype == o.RADEMACHER:
        assert np.array_equal(a, b)
        assert set(np.unique(a)) <= {-1.0, 1.0}
    else:
        # numpy's float32 log/sin/cos may differ from libm in the last place: allow
        # one fp16 unit on a small fraction of entries
        assert (a != b).mean() < 0.01
        np.testing.assert_allclose(a, b, rtol=2 ** -10, atol=1e-7)


def test_feature_tile_rule():
    # tiles clamp to F (fast_jl.cu:42), tile size is the ceiling (fast_jl_kernel.cuh:124)
    assert o.feature_tile_size(1000, 148) == 7
    assert o.feature_tile_size(11173962, 148) == 75500
    assert o.feature_tile_size(5, 148) == 1
    assert o.feature_tile_size(1048576, 148) == 7085


def test_project_matches_explicit_matrix():
    rng = np.random.default_rng(0)
    F, N, seed, T = 777, 64, 3, 10
    for ptype in (o.RADEMACHER, o.NORMAL):
        P = o.matrix(ptype, F, N, seed, T).astype(np.float64)
        g = rng.standard_normal((5, F)).astype(np.float32)
        np.testing.assert_allclose(o.project(ptype, g, N, seed, T), g.astype(np.float64) @ P,
                                   rtol=1e-12, atol=1e-9)
        g16 = g.astype(np.float16)
        np.testing.assert_allclose(o.project(ptype, g16, N, seed, T), g16.astype(np.float64) @ P,
                                   rtol=1e-12, atol=1e-9)
        np.testing.assert_allclose(o.project(ptype, g, N, seed, T, round_f16=True),
                                   g16.astype(np.float64) @ P, rtol=1e-12, atol=1e-9)


def test_all_ones_parity_known_answer():
    # the reference's own known-answer tests (tests/test_rademacher.py:65-108): an all-ones
    # input sums F entries of +-1, so every output has the parity of F
    for F in (10240, 10241):
        out = o.project(o.RADEMACHER, np.ones((2, F), np.float16), 512, 0, 148)
        assert np.all(np.mod(out, 2) == F % 2)
