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
