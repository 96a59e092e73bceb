"""finalize_scores with several checkpoints on the GPU (trak/traker.py:632-684): the epilogue kernel
against the CPU port of the reference's host arithmetic, and the streamed ScoreFinalizer (row blocks,
device accumulation over checkpoints, finished blocks into a ``scores/<exp>.mmap`` memmap) against the CPU
port of BasicScoreComputer.get_scores + that epilogue.

Tolerance: the epilogue itself is three IEEE fp32 operations and must match bit for bit; the streamed
scores are held to the 1e-3 Frobenius-relative bar of the scoring tests.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 1e-3


@pytest.mark.parametrize("n,m,M", [(1000, 37, 3), (257, 128, 1), (64, 5, 7)])
def test_epilogue_is_bit_identical_to_the_host_arithmetic(cuda, n, m, M):
    from oracle import basic_ref as br
    from trak_b200.finalize import finalize_scores_block
    g = torch.Generator().manual_seed(n + m)
    S = torch.randn(n, m, generator=g) * 3.0
    w = torch.rand(n, 1, generator=g) * M
    want = br.finalize_scores_epilogue(S, w, M)
    got = finalize_scores_block(S.to(cuda), w.to(cuda), M)
    assert torch.equal(got.cpu(), want)
    got16 = finalize_scores_block(S.to(cuda), w.to(cuda), M, dtype=torch.float16)
    assert torch.equal(got16.cpu(), want.half())
    # a row-strided accumulator (a block inside a wider buffer) and an output with a leading dimension
    wide = torch.zeros(n, m + 3, device=cuda)
    wide[:, :m] = S.to(cuda)
    out = torch.zeros(n, m + 5, device=cuda)
    finalize_scores_block(wide[:, :m], w.reshape(-1).to(cuda), M, out=out[:, :m])
    assert torch.equal(out[:, :m].cpu(), want) and float(out[:, m:].abs().sum()) == 0.0


def _checkpoints(M, n, k, m, seed):
    g = torch.Generator().manual_seed(seed)
    feats = [torch.randn(n, k, generator=g) / k ** 0.5 for _ in range(M)]
    targs = [torch.randn(m, k, generator=g) / k ** 0.5 for _ in range(M)]
    o2l = [torch.rand(n, 1, generator=g) for _ in range(M)]
    return feats, targs, o2l


def _oracle_scores(feats, targs, o2l):
    from oracle import basic_ref as br
    n, m = feats[0].shape[0], targs[0].shape[0]
    acc = torch.zeros(n, m)
    wsum = torch.zeros(n, 1)
    for f, t, w in zip(feats, targs, o2l):
        br.scores(f, t, acc)
        wsum += w
    return br.finalize_scores_epilogue(acc, wsum, len(feats))


@pytest.mark.parametrize("store_dtype", [torch.float32, torch.float16])
def test_three_checkpoints_streamed_into_a_scores_store(cuda, tmp_path, store_dtype):
    from trak_b200 import mmap_io
    from trak_b200.finalize import ScoreFinalizer
    M, n, k, m = 3, 3001, 256, 70
    feats, targs, o2l = _checkpoints(M, n, k, m, 11)
    # the stores as MmapSaver lays them out: save_dir/<model_id>/{features,out_to_loss,<exp>_grads}.mmap
    f_st, t_st, w_st = [], [], []
    for j in range(M):
        for name, src, lst in (("features", feats[j], f_st), ("exp_grads", targs[j], t_st), ("out_to_loss", o2l[j], w_st)):
            st = mmap_io.create_store(tmp_path / str(j) / f"{name}.mmap", src.shape, torch.float32)
            st[:] = src.numpy()
            st.flush()
            lst.append(mmap_io.open_store(tmp_path / str(j) / f"{name}.mmap", mode="r"))
    scores = mmap_io.create_store(tmp_path / "scores" / "exp.mmap", (n, m), store_dtype)
    fin = ScoreFinalizer(f_st, t_st, w_st, cuda, row_block=1024)   # ragged last block
    # two ranks' row ranges, one after the other, into the same store
    fin.run(scores, rows=(0, 1500))
    fin.run(scores, rows=(1500, n))
    del scores
    got = torch.from_numpy(np.array(mmap_io.open_store(tmp_path / "scores" / "exp.mmap", mode="r"))).double()
    want = _oracle_scores(feats, targs, o2l).double()
    err = float((got - want).norm() / want.norm())
    assert err <= (TOL if store_dtype == torch.float32 else 2e-3), err
    assert err <= 1e-4 or store_dtype == torch.float16, err


def test_finalizer_takes_device_tensors_and_returns_a_host_tensor(cuda):
    from trak_b200.finalize import ScoreFinalizer
    M, n, k, m = 2, 700, 128, 33
    feats, targs, o2l = _checkpoints(M, n, k, m, 5)
    out = torch.zeros(n, m)
    ScoreFinalizer([f.to(cuda) for f in feats], targs, [w.to(cuda) for w in o2l], cuda).run(out)
    want = _oracle_scores(feats, targs, o2l)
    assert float((out - want).norm() / want.norm()) <= 1e-4
    # one checkpoint: the fused row_scale epilogue of the score computer gives the same weighting
    from trak_b200.score_computers import B200ScoreComputer
    sc = B200ScoreComputer(torch.float32, cuda)
    acc = torch.zeros(n, m)
    sc.get_scores(feats[0].to(cuda), targs[0], acc, row_scale=o2l[0])
    one = torch.zeros(n, m)
    ScoreFinalizer(feats[:1], targs[:1], o2l[:1], cuda).run(one)
    assert float((acc - one).norm() / one.norm()) <= 1e-5


def test_shapes_are_checked(cuda):
    from trak_b200.finalize import ScoreFinalizer
    feats, targs, o2l = _checkpoints(2, 50, 64, 8, 1)
    with pytest.raises(ValueError):
        ScoreFinalizer(feats, targs[:1], o2l, cuda)
    with pytest.raises(ValueError):
        ScoreFinalizer(feats, targs, [o2l[0], o2l[1][:10]], cuda)
    fin = ScoreFinalizer(feats, targs, o2l, cuda)
    with pytest.raises(ValueError):
        fin.run(torch.zeros(50, 9))
    with pytest.raises(ValueError):
        fin.run(torch.zeros(50, 8), rows=(10, 60))


def test_half_precision_stores_as_traker_writes_them_by_default(cuda, tmp_path):
    """TRAKer's default dtype is fp16: features.mmap, <exp>_grads.mmap, out_to_loss.mmap and the scores store
    are all fp16 (trak/traker.py:141, trak/savers.py:363-442).  The finalizer takes them as they are (one-plane
    tensor-core products, fp32 accumulation over the checkpoints) and writes fp16 scores."""
    from trak_b200 import mmap_io
    from trak_b200.finalize import ScoreFinalizer
    M, n, k, m = 2, 1500, 192, 40
    feats, targs, o2l = _checkpoints(M, n, k, m, 23)
    feats, targs, o2l = [f.half() for f in feats], [t.half() for t in targs], [w.half() for w in o2l]
    f_st, t_st, w_st = [], [], []
    for j in range(M):
        for name, src, lst in (("features", feats[j], f_st), ("exp_grads", targs[j], t_st), ("out_to_loss", o2l[j], w_st)):
            st = mmap_io.create_store(tmp_path / str(j) / f"{name}.mmap", src.shape, torch.float16)
            st[:] = src.numpy()
            st.flush()
            lst.append(mmap_io.open_store(tmp_path / str(j) / f"{name}.mmap", mode="r"))
    scores = mmap_io.create_store(tmp_path / "scores" / "exp.mmap", (n, m), torch.float16)
    ScoreFinalizer(f_st, t_st, w_st, cuda, row_block=512).run(scores)
    got = torch.from_numpy(np.array(scores)).double()
    S = sum(f.double() @ t.double().T for f, t in zip(feats, targs))
    w = sum(x.double() for x in o2l)
    want = (S / M) * (w / M)
    err = float((got - want).norm() / want.norm())
    assert err <= 1e-3, err        # fp16 rounding of the stored scores (2^-11 per entry)
