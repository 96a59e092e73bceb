"""The benchmark configurations that are parity cases rather than bench lines, at their full shapes:

* fp32 N(0,1) gradients [32 x 1,048,576] -> 2048, Rademacher, seed 0 (the reference runs this one on the CPU
  through BasicProjector, whose matrix is a different one: what carries over is the statistics, checked
  here next to the exact comparison with the fast_jl matrix);
* a GPT-2-small sized model (148 parameter tensors, 124,439,808 features, the largest tensor 38.6M) in bf16,
  16 rows -> 8192 through ChunkedCudaProjector with parameter groups of at most 32M features.
"""
import numpy as np
import pytest
import torch

from oracle import jl_oracle as o

pytestmark = pytest.mark.gpu


def test_fp32_batch_of_32_by_one_million_to_2048_rademacher_seed_0(cuda):
    from trak_b200 import fast_jl
    B, F, N, seed, T = 32, 1_048_576, 2048, 0, 148
    g_cpu = torch.randn(B, F, generator=torch.Generator().manual_seed(0))
    g = g_cpu.to(cuda)
    out = fast_jl.project_rademacher_32(g, N, seed, T)
    assert out.shape == (B, N) and out.dtype == torch.float32
    # exact matrix: fp64 host product with the fast_jl matrix (fp32 inputs rounded to fp16 as the kernel does)
    ref = o.project(o.RADEMACHER, g_cpu.numpy(), N, seed, T, round_f16=True)
    got = out.cpu().numpy().astype(np.float64)
    rel = np.linalg.norm(got - ref, axis=1) / np.linalg.norm(ref, axis=1)
    assert rel.max() <= 1e-3, rel.max()
    # what the CPU path shares with it: E ||P g||^2 = k ||g||^2 per row, E (Pg)_n^2 = ||g||^2 per column
    gn = g_cpu.double().norm(dim=1).numpy()
    row_ratio = np.linalg.norm(got, axis=1) / (gn * N ** 0.5)
    assert np.abs(row_ratio - 1).max() < 0.06
    col_ratio = np.sqrt((got ** 2).sum(0) / (gn ** 2).sum())
    assert abs(col_ratio.mean() - 1) < 0.02 and np.abs(col_ratio - 1).max() < 0.6
    assert torch.equal(out, fast_jl.project_rademacher_32(g, N, seed, T))  # run-to-run identical


def _gpt2_small_shapes():
    d, layers, vocab, ctx = 768, 12, 50257, 1024
    shapes = [(vocab, d), (ctx, d)]
    for _ in range(layers):
        shapes += [(d,), (d,), (d, 3 * d), (3 * d,), (d, d), (d,), (d,), (d,), (d, 4 * d), (4 * d,), (4 * d, d), (d,)]
    shapes += [(d,), (d,)]
    return shapes


def _chunk_sizes(widths, cap):
    """Whole parameters packed in order into groups of at most `cap` features (the rule of
    trak/utils.py:297-331 as TRAKer applies it)."""
    sizes, cur = [], 0
    for w in widths:
        if cur + w >= cap:
            sizes.append(cur)
            cur = 0
        cur += w
    sizes.append(cur)
    return sizes


def test_gpt2_small_sized_gradients_through_the_chunked_projector(cuda):
    from trak_b200.projectors import ChunkedCudaProjector, CudaProjector, ProjectionType
    shapes = _gpt2_small_shapes()
    widths = [int(np.prod(s)) for s in shapes]
    assert len(shapes) == 148 and sum(widths) == 124_439_808 and max(widths) == 38_597_376
    cap, B, N = 32_000_000, 16, 8192
    sizes = _chunk_sizes(widths, cap)
    assert sizes[0] == 0 and sum(sizes) == sum(widths)      # the first tensor alone exceeds the cap
    # a zero-width leading group cannot be projected; TRAKer would hand it over as is, so the cap that
    # admits the largest tensor is used, as a user of the reference has to
    cap = 40_000_000
    sizes = _chunk_sizes(widths, cap)
    assert min(sizes) > 0 and max(sizes) <= cap
    seeds = np.random.default_rng(0).integers(low=0, high=500, size=len(sizes))   # trak/traker.py:294-299
    projs = [CudaProjector(grad_dim=s, proj_dim=N, seed=int(sd), proj_type=ProjectionType.rademacher,
                           device=cuda, max_batch_size=32) for s, sd in zip(sizes, seeds)]
    chunked = ChunkedCudaProjector(projs, cap, sizes, B, cuda, torch.bfloat16)

    gen = torch.Generator(device=cuda).manual_seed(3)
    grads = {i: (torch.randn((B,) + s, device=cuda, generator=gen) * 1e-2).to(torch.bfloat16)
             for i, s in enumerate(shapes)}
    # rows 0..2: one-hot gradients inside three different parameter groups
    starts = np.concatenate([[0], np.cumsum(widths)])
    group_of, local_of = {}, {}
    acc, gi = 0, 0
    for i, w in enumerate(widths):
        if acc + w >= cap:
            acc, gi = 0, gi + 1
        group_of[i], local_of[i] = gi, acc
        acc += w
    picks = [(0, 12_345_678), (76, 1_000_000), (147, 767)]       # (tensor, flat index inside it)
    for row, (ti, fi) in enumerate(picks):
        for t in grads.values():
            t[row].zero_()
        grads[ti][row].view(-1)[fi] = 1.0
    # row 3 = rows 0 + 1 + 2: the groups' projections add
    for t in grads.values():
        t[3].zero_()
    for ti, fi in picks:
        grads[ti][3].view(-1)[fi] = 1.0

    out = chunked.project(grads, model_id=0)
    assert out.shape == (B, N) and out.dtype == torch.bfloat16
    got = out.float().cpu().numpy()
    rows = []
    for row, (ti, fi) in enumerate(picks):
        gidx = group_of[ti]
        want = o.matrix_rows(o.RADEMACHER, sizes[gidx], N, int(seeds[gidx]), projs[gidx].num_sms,
                             [local_of[ti] + fi])[0]
        assert np.array_equal(got[row], want), (row, ti, fi)
        rows.append(want)
    assert np.array_equal(got[3], rows[0] + rows[1] + rows[2])
    # random rows: norms are preserved (E ||P g||^2 = k ||g||^2), bf16 output included
    gn = torch.sqrt(sum((t[4:].float() ** 2).flatten(1).sum(1) for t in grads.values())).cpu().numpy()
    ratio = np.linalg.norm(got[4:], axis=1) / (gn * N ** 0.5)
    assert np.abs(ratio - 1).max() < 0.05, ratio
    assert starts[-1] == 124_439_808


def test_cifar_resnet18_per_sample_gradients_to_2048_rademacher(cuda):
    """CIFAR ResNet-18 (3x3 stem, 10 classes: 11,173,962 parameters in 62 tensors), per-example margin gradients
    from torch.func in fp32, projected straight from the gradient dict: bit-equal to projecting the flattened
    [B, D] matrix, and within tolerance of the fp64 host product with the fast_jl matrix."""
    torchvision = pytest.importorskip("torchvision")
    from torch.func import functional_call, grad, vmap
    from trak_b200 import fast_jl
    from trak_b200.projectors import CudaProjector, ProjectionType, vectorize
    torch.manual_seed(0)
    model = torchvision.models.resnet18(num_classes=10)
    model.conv1 = torch.nn.Conv2d(3, 64, 3, 1, 1, bias=False)
    model.maxpool = torch.nn.Identity()
    model = model.to(cuda).eval()
    params = {k: v.detach() for k, v in model.named_parameters()}
    buffers = {k: v.detach() for k, v in model.named_buffers()}
    D = sum(p.numel() for p in params.values())
    assert D == 11_173_962 and len(params) == 62
    g = torch.Generator().manual_seed(0)
    B, N, seed = 16, 2048, 0
    xs, ys = torch.rand(B, 3, 32, 32, generator=g).to(cuda), torch.randint(0, 10, (B,), generator=g).to(cuda)

    def margin(p, x, y):   # the image-classification model output of trak/modelout_functions.py:100-152
        logits = functional_call(model, (p, buffers), (x.unsqueeze(0),))[0]
        own = torch.arange(logits.numel(), device=logits.device) == y
        rest = torch.logsumexp(torch.where(own, torch.full_like(logits, -torch.inf), logits), 0)
        return (logits * own).sum() - rest

    grads = vmap(grad(margin), in_dims=(None, 0, 0))(params, xs, ys)
    proj = CudaProjector(D, N, seed, ProjectionType.rademacher, cuda, 32)
    feats = proj.project(grads, model_id=0)
    flat = vectorize(grads, device=cuda)
    assert flat.shape == (B, D) and flat.dtype == torch.float32
    assert torch.equal(feats, fast_jl.project_rademacher_16(flat, N, seed, proj.num_sms))
    rows = [0, B - 1]
    ref = o.project(o.RADEMACHER, flat[rows].cpu().numpy(), N, seed, proj.num_sms, round_f16=True)
    got = feats[rows].cpu().numpy().astype(np.float64)
    rel = np.linalg.norm(got - ref, axis=1) / np.linalg.norm(ref, axis=1)
    assert rel.max() <= 1e-3, rel


def test_gpt2_small_real_gradients_through_the_chunked_projector(cuda):
    """GPT-2-small (random init, bf16, 124,439,808 parameters in 148 tensors), 16 sequences of 512 uniform-random
    tokens, per-sequence gradients of the mean next-token log-probability from torch.func, projected to 8192 by
    the chunked projector straight from the gradient dict.  Two real rows are checked against the fp64 oracle on
    three 32-column groups: the sum over the chunks of each chunk's own projection (own seed)."""
    transformers = pytest.importorskip("transformers")
    from torch.func import functional_call, grad, vmap
    from trak_b200.projectors import make_chunked_projector
    torch.manual_seed(0)
    model = transformers.GPT2LMHeadModel(transformers.GPT2Config(attn_implementation="eager")).to(cuda, torch.bfloat16).eval()
    params = {k: v.detach() for k, v in model.named_parameters()}
    buffers = {k: v.detach() for k, v in model.named_buffers()}
    widths = [p.numel() for p in params.values()]
    assert len(widths) == 148 and sum(widths) == 124_439_808 and max(widths) == 38_597_376
    B, S, N = 16, 512, 8192
    ids = torch.randint(0, 50257, (B, S), generator=torch.Generator().manual_seed(0)).to(cuda)

    def mean_next_token_logprob(p, seq):
        logits = functional_call(model, (p, buffers), (seq.unsqueeze(0),)).logits[0]
        logp = torch.log_softmax(logits[:-1].float(), dim=-1)
        return logp.gather(1, seq[1:, None]).mean()

    grads = vmap(grad(mean_next_token_logprob), in_dims=(None, 0), chunk_size=4)(params, ids)
    assert all(g.dtype == torch.bfloat16 and g.shape[0] == B for g in grads.values())
    # the reference's cap for this batch (2^32 / 16) admits the whole model in one chunk; 40M features per
    # chunk (the smallest round cap that admits the 38.6M-feature embedding) gives four
    chunked = make_chunked_projector(widths, N, 0, B, cuda, torch.float32, max_chunk_size=40_000_000)
    sizes = chunked.params_per_chunk
    assert len(sizes) == 4 and min(sizes) > 0 and sum(sizes) == sum(widths)
    out = chunked.project(grads, model_id=0)
    assert out.shape == (B, N) and out.dtype == torch.float32 and bool(torch.isfinite(out).all())

    rows, groups = [0, 7], [0, 100, 255]
    want = np.zeros((len(rows), 32 * len(groups)))
    vals, at = list(grads.values()), 0
    for size, proj in zip(sizes, chunked.projector_per_chunk):
        part, width = [], 0
        while width < size:
            part.append(vals[at][rows].reshape(len(rows), -1))
            width += part[-1].shape[1]
            at += 1
        assert width == size
        flat = torch.cat(part, dim=1).contiguous().view(torch.uint16).cpu().numpy()    # bf16 bit patterns
        want += o.project_column_groups(o.RADEMACHER, flat, proj.seed, proj.num_sms, groups)
    cols = np.concatenate([np.arange(32 * g, 32 * g + 32) for g in groups])
    got = out[rows][:, cols].double().cpu().numpy()
    rel = np.linalg.norm(got - want, axis=1) / np.linalg.norm(want, axis=1)
    print("GPT-2-small real gradients, rows 0 and 7 on 96 columns against the fp64 oracle:", rel)
    assert rel.max() <= 1e-3, rel


def test_feature_writer_fills_the_stores_like_featurize(cuda, tmp_path):
    """FeatureWriter against the reference's per-batch arithmetic (trak/traker.py:424-437): project, divide by
    sqrt(num_params), cast to the store dtype, write rows `inds`; out-to-loss weights beside them.  Batches in
    shuffled index order, a ragged last batch, more batches than staging slots."""
    from trak_b200 import mmap_io
    from trak_b200.featurize import FeatureWriter
    from trak_b200.projectors import CudaProjector, ProjectionType
    n, D, k, bs = 1000, 5003, 512, 96
    g = torch.Generator(device=cuda).manual_seed(0)
    grads = torch.randn(n, D, device=cuda, generator=g)
    o2l = torch.rand(n, 1, device=cuda, generator=g)
    proj = CudaProjector(D, k, 3, ProjectionType.rademacher, cuda, 32)
    perm = np.random.default_rng(0).permutation(n)
    for dtype in (torch.float16, torch.float32):
        tag = str(dtype).split(".")[-1]
        gs = mmap_io.create_store(tmp_path / tag / "grads.mmap", (n, k), dtype)
        ws = mmap_io.create_store(tmp_path / tag / "out_to_loss.mmap", (n, 1), dtype)
        fw = FeatureWriter(proj, D ** 0.5, dtype, cuda, max_batch=bs, grads_store=gs, out_to_loss_store=ws, slots=3,
                           keep_on_device=True)
        for i in range(0, n, bs):
            inds = perm[i:i + bs]
            idx = torch.as_tensor(inds, device=cuda)
            fw.add(grads[idx], inds, model_id=0, loss_grads=o2l[idx])
        fw.flush()
        want = (proj.project(grads, model_id=0) / D ** 0.5).to(dtype).cpu()
        got = torch.from_numpy(np.array(mmap_io.open_store(tmp_path / tag / "grads.mmap", mode="r")))
        # alpha is applied inside the kernel before the cast, the reference divides afterwards: one rounding apart
        torch.testing.assert_close(got.float(), want.float(), rtol=2e-3 if dtype == torch.float16 else 1e-6, atol=1e-6)
        assert torch.equal(torch.from_numpy(np.array(ws)), o2l.to(dtype).cpu())
        assert torch.equal(fw.features_device.cpu(), got)


def test_cifar_featurize_slice_with_stores_and_out_to_loss(cuda, tmp_path):
    """A slice of the 50,000-image featurize job as bench.py runs it: 64 synthetic images, per-example margin
    gradients of the CIFAR ResNet-18, FeatureWriter (projection with 1/sqrt(D) folded in -> grads.mmap rows,
    margin out-to-loss weights beside them, trak/traker.py:424-437, trak/modelout_functions.py:153-179).
    Every stored row is checked on eight 32-column groups against the fp64 oracle."""
    torchvision = pytest.importorskip("torchvision")
    from torch.func import functional_call, grad, vmap
    from trak_b200 import mmap_io
    from trak_b200.featurize import FeatureWriter
    from trak_b200.projectors import CudaProjector, ProjectionType, vectorize
    torch.manual_seed(0)
    model = torchvision.models.resnet18(num_classes=10)
    model.conv1 = torch.nn.Conv2d(3, 64, 3, 1, 1, bias=False)
    model.maxpool = torch.nn.Identity()
    model = model.to(cuda).eval()
    params = {k: v.detach() for k, v in model.named_parameters()}
    buffers = {k: v.detach() for k, v in model.named_buffers()}
    D = sum(p.numel() for p in params.values())
    n, bs, N = 64, 24, 2048
    g = torch.Generator().manual_seed(3)
    xs, ys = torch.rand(n, 3, 32, 32, generator=g).to(cuda), torch.randint(0, 10, (n,), generator=g).to(cuda)

    def margin(p, x, y):
        logits = functional_call(model, (p, buffers), (x.unsqueeze(0),))[0]
        own = torch.arange(logits.numel(), device=logits.device) == y
        rest = torch.logsumexp(torch.where(own, torch.full_like(logits, -torch.inf), logits), 0)
        return (logits * own).sum() - rest

    per_sample = vmap(grad(margin), in_dims=(None, 0, 0))
    gs = mmap_io.create_store(tmp_path / "0" / "grads.mmap", (n, N), torch.float32)
    ws = mmap_io.create_store(tmp_path / "0" / "out_to_loss.mmap", (n, 1), torch.float32)
    proj = CudaProjector(D, N, 0, ProjectionType.rademacher, cuda, 32)
    fw = FeatureWriter(proj, D ** 0.5, torch.float32, cuda, max_batch=bs, grads_store=gs, out_to_loss_store=ws, slots=2)
    flats, weights = [], []
    for i in range(0, n, bs):          # 24 + 24 + 16 rows
        x, y = xs[i:i + bs], ys[i:i + bs]
        grads = per_sample(params, x, y)
        with torch.no_grad():
            ps = torch.softmax(model(x), dim=-1)[torch.arange(x.shape[0], device=cuda), y]
        fw.add(grads, np.arange(i, i + x.shape[0]), model_id=0, loss_grads=(1.0 - ps).unsqueeze(-1))
        flats.append(vectorize(grads, device=cuda).cpu())
        weights.append((1.0 - ps).cpu())
    fw.flush()
    stored = np.array(mmap_io.open_store(tmp_path / "0" / "grads.mmap", mode="r"), dtype=np.float64)
    flat = torch.cat(flats).numpy()
    groups = [0, 9, 17, 26, 35, 44, 53, 63]
    want = o.project_column_groups(o.RADEMACHER, flat, 0, proj.num_sms, groups, round_f16=True) / D ** 0.5
    cols = np.concatenate([np.arange(32 * c, 32 * c + 32) for c in groups])
    rel = np.linalg.norm(stored[:, cols] - want, axis=1) / np.linalg.norm(want, axis=1)
    print("featurize slice: worst of 64 stored rows on 256 columns against the fp64 oracle:", rel.max())
    assert rel.max() <= 1e-3, rel
    w_stored = np.array(mmap_io.open_store(tmp_path / "0" / "out_to_loss.mmap", mode="r"))
    assert np.array_equal(w_stored[:, 0], torch.cat(weights).numpy())
    assert (w_stored > 0).all() and (w_stored < 1).all()
