"""The CPU port of the reference's BasicProjector / BasicScoreComputer against
fixtures produced by the unmodified reference (tests/golden/make_reference_golden.py)."""
import os

import numpy as np
import pytest
import torch

from oracle import basic_ref as br


@pytest.fixture(autouse=True)
def _one_thread():
    n = torch.get_num_threads()
    torch.set_num_threads(1)  # the fixtures were made with a fixed summation order
    yield
    torch.set_num_threads(n)


@pytest.mark.parametrize("ptype", ["rademacher", "normal"])
def test_basic_project_matches_reference_bits(golden_dir, ptype):
    d = np.load(os.path.join(golden_dir, f"basic_project_{ptype}.npz"))
    g = torch.randn(int(d["B"]), int(d["D"]), generator=torch.Generator().manual_seed(int(d["input_seed"])))
    out = br.basic_project(g, int(d["k"]), int(d["seed"]), ptype, model_id=int(d["model_id"]))
    assert np.array_equal(out.numpy(), d["out"])


def test_basic_project_block_subset():
    g = torch.randn(3, 500, generator=torch.Generator().manual_seed(1))
    full = br.basic_project(g, 250, 5, "rademacher")
    part = br.basic_project(g, 250, 5, "rademacher", blocks=[1])
    assert torch.equal(part[:, 100:200], full[:, 100:200])
    assert part[:, :100].abs().sum() == 0 and part[:, 200:].abs().sum() == 0


def test_scoring_matches_reference(golden_dir):
    d = np.load(os.path.join(golden_dir, "basic_scoring.npz"))
    n, k, m, lam, rows = int(d["n"]), int(d["k"]), int(d["m"]), float(d["lam"]), int(d["block_rows"])
    X = torch.randn(n, k, generator=torch.Generator().manual_seed(int(d["x_seed"]))) / k ** 0.5
    T = torch.randn(m, k, generator=torch.Generator().manual_seed(int(d["t_seed"]))) / k ** 0.5
    gram = br.xtx(X, rows)
    feats = br.x_xtx_inv(X, gram, lam, rows)
    acc = torch.zeros(n, m)
    br.scores(feats, T, acc)
    assert np.array_equal(gram.numpy(), d["gram"])
    np.testing.assert_allclose(feats.numpy(), d["features"], rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(acc.numpy(), d["scores"], rtol=1e-6, atol=1e-6)


def test_finalize_epilogue():
    s = torch.arange(6.0).reshape(3, 2)
    w = torch.tensor([[1.0], [2.0], [4.0]])
    out = br.finalize_scores_epilogue(s, w, 2)
    assert torch.equal(out, (s / 2) * (w / 2))
