"""Pins the CPU oracle to what the reference's compiled CUDA kernel computes: golden
vectors made on a B200 by tests/golden/make_fastjl_golden.py.

Rademacher entries are integer work and must match bit for bit.  Gaussian entries
pass through logf / sincos, where the host libm and the GPU (logf, __sincosf with
~1e-6 absolute error) differ in the last place now and then: at most 1 % of the
entries may differ, and then by about one fp16 unit."""
import os

import numpy as np
import pytest
import torch

from oracle import jl_oracle as o


@pytest.fixture(scope="module")
def gold(golden_dir):
    return np.load(os.path.join(golden_dir, "fastjl_golden.npz"))


@pytest.mark.parametrize("case", [0, 1, 2, 3])
def test_rademacher_rows_bit_exact(gold, case):
    F, N, seed, T = (int(v) for v in gold[f"rows_{case}_meta"])
    feats = gold[f"rows_{case}_feats"].tolist()
    assert np.array_equal(o.matrix_rows(o.RADEMACHER, F, N, seed, T, feats),
                          gold[f"rows_{case}_rademacher"].astype(np.float32))


@pytest.mark.parametrize("case", [0, 1, 2, 3])
def test_normal_rows_within_one_fp16_unit(gold, case):
    F, N, seed, T = (int(v) for v in gold[f"rows_{case}_meta"])
    feats = gold[f"rows_{case}_feats"].tolist()
    got = o.matrix_rows(o.NORMAL, F, N, seed, T, feats)
    want = gold[f"rows_{case}_normal"].astype(np.float32)
    assert (got != want).mean() < 0.01
    np.testing.assert_allclose(got, want, rtol=2 ** -10, atol=4e-6)


@pytest.mark.parametrize("case", [0, 1])
def test_projection_of_random_inputs(gold, case):
    B, F, N, seed, T, in_seed = (int(v) for v in gold[f"proj_{case}_meta"])
    base = torch.randn(B, F, generator=torch.Generator().manual_seed(in_seed))
    for dn, dt in (("f16", torch.float16), ("f32", torch.float32)):
        g = base.to(dt).numpy()
        for name, p in (("rademacher", o.RADEMACHER), ("normal", o.NORMAL)):
            ref = o.project(p, g, N, seed, T, round_f16=True)
            want = gold[f"proj_{case}_{dn}_{name}"].astype(np.float64)
            err = (np.linalg.norm(ref - want, axis=1) / np.linalg.norm(want, axis=1)).max()
            assert err < 2e-5, (dn, name, err)


def test_column_group_subset_equals_the_full_oracle_projection():
    """project_column_groups (used where the full oracle would take minutes) gives exactly the columns of the
    full projection, for both matrix types and whatever the projection dimension."""
    import numpy as np
    from oracle import jl_oracle as o
    g = np.random.default_rng(0).standard_normal((3, 5000)).astype(np.float16)
    for p in (o.RADEMACHER, o.NORMAL):
        full = o.project(p, g, 512, 7, 37)
        part = o.project_column_groups(p, g, 7, 37, [0, 5, 15])
        assert np.array_equal(part[:, :32], full[:, :32])
        assert np.array_equal(part[:, 32:64], full[:, 160:192])
        assert np.array_equal(part[:, 64:], full[:, 480:512])
        assert np.array_equal(o.project(p, g, 1024, 7, 37)[:, 160:192], part[:, 32:64])
