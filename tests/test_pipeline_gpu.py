"""The two hot paths chained the way TRAKer chains them (trak/traker.py:424-429, 482-486, 570-578,
662-678): per-sample gradients from torch.func -> projection -> /sqrt(D) -> Gram, inverse,
features -> scores with the out-to-loss weighting.  GPU side: the mirrored projector and score
computer.  Reference side: the CPU oracle's projection with the identical matrix and the CPU port
of BasicScoreComputer.  Bar: scores within 1e-3 (Frobenius-relative)."""
import numpy as np
import pytest
import torch

from oracle import basic_ref as br
from oracle import jl_oracle as o

pytestmark = pytest.mark.gpu


def _per_sample_grads(model, xs, ys):
    from torch.func import functional_call, grad, vmap
    params = {k: v.detach() for k, v in model.named_parameters()}

    def margin(p, x, y):
        logits = functional_call(model, p, (x.unsqueeze(0),))[0]
        own = torch.arange(logits.numel(), device=logits.device) == y
        rest = torch.logsumexp(torch.where(own, torch.full_like(logits, -1e9), logits), 0)
        return (logits * own).sum() - rest

    return vmap(grad(margin), in_dims=(None, 0, 0))(params, xs, ys)


def test_featurize_finalize_score_matches_cpu_reference_path(cuda):
    from trak_b200.projectors import CudaProjector, ProjectionType, vectorize
    from trak_b200.score_computers import B200ScoreComputer
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(20, 48), torch.nn.Tanh(), torch.nn.Linear(48, 10)).to(cuda)
    D = sum(p.numel() for p in model.parameters())
    n, m, k, seed = 3000, 40, 512, 7
    xs, ys = torch.randn(n, 20, device=cuda), torch.randint(0, 10, (n,), device=cuda)
    xt, yt = torch.randn(m, 20, device=cuda), torch.randint(0, 10, (m,), device=cuda)
    proj = CudaProjector(D, k, seed, ProjectionType.rademacher, cuda, 32)

    def featurize(x, y):
        feats, flats = [], []
        for i in range(0, x.shape[0], 500):
            g = _per_sample_grads(model, x[i:i + 500], y[i:i + 500])
            feats.append(proj.project(g, model_id=0, alpha=1.0 / D ** 0.5))   # 1/sqrt(D) folded in
            flats.append(vectorize(g, device=cuda).cpu())
        return torch.cat(feats), torch.cat(flats)

    X, gx = featurize(xs, ys)
    T, gt = featurize(xt, yt)
    w = torch.rand(n, 1, generator=torch.Generator().manual_seed(1))          # stands in for out_to_loss
    # gradients of a tiny model have a fast-decaying spectrum; regularise relative to the mean eigenvalue
    # so that the comparison measures the kernels and not fp32 round-off amplified by the conditioning
    lam = 0.1 * float((X.double() ** 2).sum() / k)
    sc = B200ScoreComputer(torch.float32, cuda, CUDA_MAX_DIM_SIZE=1024, lambda_reg=lam)
    gram = sc.get_xtx(X)
    phi = sc.get_x_xtx_inv(X, gram)
    scores = torch.zeros(n, m)
    sc.get_scores(phi, T, scores, row_scale=w)

    # reference path on the CPU: identical matrix (fp32 gradients rounded to fp16 on the way in, as the
    # reference kernel does), then the port of BasicScoreComputer and the host epilogue
    def cpu_features(flat):
        return torch.from_numpy(o.project(o.RADEMACHER, flat.numpy(), k, seed, proj.num_sms, round_f16=True)
                                / D ** 0.5).float()

    Xr, Tr = cpu_features(gx), cpu_features(gt)
    assert float((X.cpu() - Xr).norm() / Xr.norm()) <= 1e-3
    g_ref = br.xtx(Xr)
    phi_ref = br.x_xtx_inv(Xr, g_ref, lam)
    s_ref = torch.zeros(n, m)
    br.scores(phi_ref, Tr, s_ref)
    s_ref = br.finalize_scores_epilogue(s_ref, w, 1)
    err = float((scores - s_ref).norm() / s_ref.norm())
    assert err <= 1e-3, err
