"""The reference's own, unmodified ``TRAKer`` driving this library end to end
(trak/traker.py: featurize -> finalize_features -> start_scoring_checkpoint -> score ->
finalize_scores), two ways:

  A. nothing passed in: ``TRAKer`` imports ``fast_jl`` itself (trak/traker.py:254-262) and finds the
     shim module registered under that name, builds the reference's ``CudaProjector`` on it, and scores
     with the reference's ``BasicScoreComputer`` (torch on the GPU);
  B. ``projector=`` this library's ``CudaProjector`` and ``score_computer=`` ``B200ScoreComputer``.

Both must give the same attribution scores within 1e-3 (Frobenius-relative), and A's projected
gradients must equal the CPU oracle's projection of the same per-sample gradients.

The reference package is not part of this repository; ``__graft_entry__.build()`` installs it, where
its checkout exists, into the git-ignored ``baseline/_ref`` directory, and the test is skipped when
that directory is absent.
"""
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

_REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")


@pytest.fixture()
def trak(cuda, monkeypatch):
    if not os.path.isdir(os.path.join(_REF, "trak")):
        pytest.skip("reference package not installed under baseline/_ref")
    import trak_b200.fast_jl as shim
    monkeypatch.setitem(sys.modules, "fast_jl", shim)
    monkeypatch.syspath_prepend(_REF)
    for name in [m for m in sys.modules if m == "trak" or m.startswith("trak.")]:
        monkeypatch.delitem(sys.modules, name)
    import trak
    assert os.path.abspath(trak.__file__).startswith(_REF)
    return trak


def _model_and_data(cuda):
    torch.manual_seed(0)
    model = torch.nn.Sequential(
        torch.nn.Conv2d(3, 8, 3, padding=1), torch.nn.ReLU(), torch.nn.AvgPool2d(2),
        torch.nn.Flatten(), torch.nn.Linear(8 * 4 * 4, 32), torch.nn.ReLU(), torch.nn.Linear(32, 10),
    ).to(cuda).eval()
    g = torch.Generator().manual_seed(1)
    n, m = 1200, 48
    train = (torch.rand(n, 3, 8, 8, generator=g).to(cuda), torch.randint(0, 10, (n,), generator=g).to(cuda))
    targets = (torch.rand(m, 3, 8, 8, generator=g).to(cuda), torch.randint(0, 10, (m,), generator=g).to(cuda))
    return model, train, targets


def _run(trak, model, train, targets, save_dir, half=False, **kw):
    n, m = train[0].shape[0], targets[0].shape[0]
    tr = trak.TRAKer(model=model, task="image_classification", train_set_size=n, save_dir=str(save_dir),
                     device="cuda", proj_dim=1024, use_half_precision=half, lambda_reg=0.0,
                     logging_level=40, **kw)
    ckpt = model.state_dict()
    tr.load_checkpoint(ckpt, model_id=0)
    for i in range(0, n, 200):
        tr.featurize(batch=(train[0][i:i + 200], train[1][i:i + 200]), num_samples=min(200, n - i))
    # ridge term = a tenth of the Gram's mean eigenvalue (gradients of a tiny model have a fast-decaying
    # spectrum), so that the comparison measures the kernels and not round-off amplified by the conditioning
    X = np.array(tr.saver.current_store["grads"], dtype=np.float64)
    tr.score_computer.lambda_reg = 0.1 * float((X ** 2).sum() / X.shape[1])
    tr.finalize_features()
    tr.start_scoring_checkpoint(exp_name="t", checkpoint=ckpt, model_id=0, num_targets=m)
    tr.score(batch=targets, num_samples=m)
    scores = np.array(tr.finalize_scores(exp_name="t"))
    store = tr.saver.current_store
    grads = np.array(store["grads"])
    # the same scoring arithmetic in fp64 on the host, from the projections this run stored
    # (trak/score_computers.py:145-189, trak/traker.py:676-678)
    X, T = grads.astype(np.float64), np.array(store["t_grads"], dtype=np.float64)
    inv = np.linalg.inv(X.T @ X + tr.score_computer.lambda_reg * np.eye(X.shape[1]))
    inv /= np.abs(inv).mean()
    exact = (X @ inv @ T.T) * np.array(store["out_to_loss"], dtype=np.float64)
    return tr, scores, grads, exact


def test_unmodified_traker_runs_on_the_shim_and_on_the_mirrored_classes(trak, cuda, tmp_path):
    from oracle import jl_oracle as o
    from trak_b200.projectors import CudaProjector, ProjectionType
    from trak_b200.score_computers import B200ScoreComputer
    model, train, targets = _model_and_data(cuda)
    D = sum(p.numel() for p in model.parameters())
    tr_a, s_a, g_a, x_a = _run(trak, model, train, targets, tmp_path / "a")
    assert type(tr_a.projector).__module__ == "trak.projectors"
    assert type(tr_a.projector).__name__ == "CudaProjector"
    assert type(tr_a.score_computer).__name__ == "BasicScoreComputer"

    proj = CudaProjector(grad_dim=D, proj_dim=1024, seed=0, proj_type=ProjectionType.rademacher,
                         device=cuda, max_batch_size=32)
    tr_b, s_b, g_b, x_b = _run(trak, model, train, targets, tmp_path / "b",
                          projector=proj, score_computer=B200ScoreComputer)
    assert isinstance(tr_b.score_computer, B200ScoreComputer)

    assert s_a.shape == s_b.shape == (train[0].shape[0], targets[0].shape[0])
    assert np.isfinite(s_a).all() and np.abs(s_a).max() > 0
    # same matrix, same gradients: the stored projections agree to fp32 summation order
    assert np.linalg.norm(g_a - g_b) <= 1e-5 * np.linalg.norm(g_a)
    err_a = np.linalg.norm(s_a - x_a) / np.linalg.norm(x_a)
    err_b = np.linalg.norm(s_b - x_b) / np.linalg.norm(x_b)
    err_ab = np.linalg.norm(s_a - s_b) / np.linalg.norm(s_a)
    print(f"scores vs fp64: reference classes {err_a:.2e}, this library {err_b:.2e}; A vs B {err_ab:.2e}")
    assert err_b <= 1e-3, (err_a, err_b, err_ab)
    assert err_ab <= 1e-3, (err_a, err_b, err_ab)

    # A's stored projections against the CPU oracle on the same per-sample gradients (the first batch as
    # featurize saw it).  The kernel, like the reference's, rounds fp32 gradients to fp16 on the way in;
    # examples whose gradients are tiny sit in fp16's subnormal range, where a last-bit difference of a
    # recomputed gradient moves the rounded value, so the comparison is over the batch, not per row.
    grads = tr_a.gradient_computer.compute_per_sample_grad(batch=(train[0][:200], train[1][:200]))
    flat = trak.utils.vectorize(grads, device="cuda").float().cpu().numpy()
    ref = o.project(o.RADEMACHER, flat, 1024, 0, tr_a.projector.num_sms, round_f16=True) / D ** 0.5
    assert np.linalg.norm(g_a[:200] - ref) <= 1e-3 * np.linalg.norm(ref)


def test_unmodified_traker_in_its_default_half_precision(trak, cuda, tmp_path):
    """TRAKer's default: projections, Gram, features and scores stored and handed over in fp16
    (trak/traker.py:141).  The mirrored classes must take that as they take fp32; against the fp32 run the
    scores differ by what fp16 storage of the features costs."""
    from trak_b200.projectors import CudaProjector, ProjectionType
    from trak_b200.score_computers import B200ScoreComputer
    model, train, targets = _model_and_data(cuda)
    D = sum(p.numel() for p in model.parameters())

    def projector():
        return CudaProjector(grad_dim=D, proj_dim=1024, seed=0, proj_type=ProjectionType.rademacher,
                             device=cuda, max_batch_size=32)

    _, s32, _, _ = _run(trak, model, train, targets, tmp_path / "f32", projector=projector(),
                        score_computer=B200ScoreComputer)
    tr16, s16, g16, _ = _run(trak, model, train, targets, tmp_path / "f16", half=True, projector=projector(),
                             score_computer=B200ScoreComputer)
    assert g16.dtype == np.float16 and tr16.score_computer.dtype == torch.float16
    assert np.isfinite(s16).all()
    err = np.linalg.norm(s16.astype(np.float64) - s32) / np.linalg.norm(s32)
    print(f"half-precision TRAKer against the fp32 run: {err:.2e}")
    assert err <= 5e-2, err


def test_three_checkpoints_finalized_by_the_reference_and_by_the_streamed_finalizer(trak, cuda, tmp_path):
    """Three checkpoints through the unmodified TRAKer (this library's projector and score computer plugged
    in); its own finalize_scores (host accumulator, numpy epilogue, MmapSaver's scores/<exp>.mmap,
    trak/traker.py:632-684) against ScoreFinalizer reading the same save_dir.  Both accumulate the same
    per-checkpoint products with the same fp32 additions in the same order and apply the same three IEEE
    operations at the end, so the two files must be equal byte for byte."""
    from trak_b200 import mmap_io
    from trak_b200.finalize import ScoreFinalizer
    from trak_b200.projectors import CudaProjector, ProjectionType
    from trak_b200.score_computers import B200ScoreComputer
    model, train, targets = _model_and_data(cuda)
    n, m = 600, targets[0].shape[0]
    train = (train[0][:n], train[1][:n])
    D = sum(p.numel() for p in model.parameters())
    proj = CudaProjector(grad_dim=D, proj_dim=512, seed=0, proj_type=ProjectionType.rademacher, device=cuda,
                         max_batch_size=32)
    tr = trak.TRAKer(model=model, task="image_classification", train_set_size=n, save_dir=str(tmp_path / "s"),
                     device="cuda", proj_dim=512, use_half_precision=False, lambda_reg=1.0, logging_level=40,
                     projector=proj, score_computer=B200ScoreComputer)
    ckpts = []
    base = {k: v.clone() for k, v in model.state_dict().items()}
    for j in range(3):
        g = torch.Generator(device=cuda).manual_seed(100 + j)
        ckpts.append({k: v + 0.05 * j * torch.randn(v.shape, device=cuda, generator=g) for k, v in base.items()})
    for j, ck in enumerate(ckpts):
        tr.load_checkpoint(ck, model_id=j)
        for i in range(0, n, 200):
            tr.featurize(batch=(train[0][i:i + 200], train[1][i:i + 200]), num_samples=200)
    tr.finalize_features()
    for j, ck in enumerate(ckpts):
        tr.start_scoring_checkpoint(exp_name="t", checkpoint=ck, model_id=j, num_targets=m)
        tr.score(batch=targets, num_samples=m)
    ref_scores = np.array(tr.finalize_scores(exp_name="t"))
    assert ref_scores.shape == (n, m) and np.isfinite(ref_scores).all() and np.abs(ref_scores).max() > 0
    ref_file = tmp_path / "s" / "scores" / "t.mmap"

    stores = lambda name: [mmap_io.open_store(tmp_path / "s" / str(j) / name, mode="r") for j in range(3)]  # noqa: E731
    mine = mmap_io.create_store(tmp_path / "mine" / "t.mmap", (n, m), torch.float32)
    ScoreFinalizer(stores("features.mmap"), stores("t_grads.mmap"), stores("out_to_loss.mmap"), cuda,
                   row_block=256).run(mine)
    del mine
    assert open(tmp_path / "mine" / "t.mmap", "rb").read() == open(ref_file, "rb").read()
    # and the weighting is the product of the sums, not the sum of the products
    S = sum(np.array(a, dtype=np.float64) @ np.array(b, dtype=np.float64).T
            for a, b in zip(stores("features.mmap"), stores("t_grads.mmap")))
    w = sum(np.array(x, dtype=np.float64) for x in stores("out_to_loss.mmap"))
    exact = (S / 3) * (w / 3)
    assert np.linalg.norm(ref_scores - exact) <= 1e-3 * np.linalg.norm(exact)
