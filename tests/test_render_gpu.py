"""Volume-rendering accumulation kernels against the float64 CPU restatement, and one whole
ray-marched training step (near/far, sampling, fused query, eikonal gradient-of-gradient, density,
rendering, backward) as the reference's PlainVoxels.forward composes it
(demo/train_scene_recon.py:64-161)."""
import numpy as np
import pytest
import torch

import bench_workloads as bw
from oracle import render as orender

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _packed_samples(n_rays, max_per_ray, seed):
    rng = np.random.default_rng(seed)
    counts = rng.integers(0, max_per_ray + 1, n_rays)
    counts[rng.integers(0, n_rays, n_rays // 10)] = 0          # rays without samples
    counts[0] = max_per_ray                                     # a ray longer than one warp round
    ri = np.repeat(np.arange(n_rays), counts)
    m = len(ri)
    ts = rng.uniform(0, 3, m).astype(np.float32)
    te = (ts + rng.uniform(0.005, 0.1, m)).astype(np.float32)
    sg = rng.uniform(0, 20, m).astype(np.float32)
    sg[rng.integers(0, m, m // 8)] = 0
    return ri, ts, te, sg


@pytest.mark.parametrize("n_rays,max_per_ray", [(500, 130), (64, 7), (3, 300)])
def test_render_weights_and_accumulate_vs_oracle(n_rays, max_per_ray):
    from ash.render import accumulate_along_rays, render_weight_from_density

    ri, ts, te, sg = _packed_samples(n_rays, max_per_ray, seed=n_rays)
    m = len(ri)
    t = lambda a: torch.from_numpy(a).to(DEV)
    sig = t(sg).view(-1, 1).requires_grad_(True)
    w = render_weight_from_density(t(ts).view(-1, 1), t(te).view(-1, 1), sig, t(ri), n_rays)
    assert w.shape == (m, 1)
    w_ref = orender.render_weights(ts, te, sg, ri, n_rays)
    np.testing.assert_allclose(w.detach().cpu().numpy().ravel(), w_ref, rtol=2e-5, atol=1e-7)
    rng = np.random.default_rng(1)
    vals = rng.normal(size=(m, 3)).astype(np.float32)
    v = t(vals).requires_grad_(True)
    rgb = accumulate_along_rays(w, t(ri), v, n_rays)
    opacity = accumulate_along_rays(w, t(ri), None, n_rays)
    assert rgb.shape == (n_rays, 3) and opacity.shape == (n_rays, 1)
    np.testing.assert_allclose(rgb.detach().cpu().numpy(), orender.accumulate(w_ref, ri, vals, n_rays), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(opacity.detach().cpu().numpy(), orender.accumulate(w_ref, ri, None, n_rays), rtol=1e-4, atol=1e-6)
    assert (opacity <= 1 + 1e-5).all()
    # gradients: loss = sum(go_rgb * rgb) + sum(go_op * opacity)
    go_rgb = rng.normal(size=(n_rays, 3)).astype(np.float32)
    go_op = rng.normal(size=(n_rays, 1)).astype(np.float32)
    ((rgb * t(go_rgb)).sum() + (opacity * t(go_op)).sum()).backward()
    g_w = (go_rgb[ri] * vals).sum(1) + go_op[ri, 0]              # d loss / d weights
    gs_ref = orender.render_weights_grad(ts, te, sg, ri, n_rays, g_w)
    np.testing.assert_allclose(sig.grad.cpu().numpy().ravel(), gs_ref, rtol=2e-4, atol=2e-5 * max(1.0, np.abs(gs_ref).max()))
    np.testing.assert_allclose(v.grad.cpu().numpy(), w_ref[:, None] * go_rgb[ri], rtol=2e-5, atol=1e-7)


def test_empty_inputs():
    from ash.render import accumulate_along_rays, render_weight_from_density

    e = torch.empty(0, 1, device=DEV)
    ri = torch.empty(0, dtype=torch.long, device=DEV)
    w = render_weight_from_density(e, e, e, ri, 5)
    assert w.shape == (0, 1)
    out = accumulate_along_rays(w, ri, torch.empty(0, 3, device=DEV), 5)
    assert out.shape == (5, 3) and torch.count_nonzero(out) == 0


def test_ray_marched_training_step():
    """One optimisation step of a sphere SDF stored in a sparse-dense grid: every stage runs on the
    library's kernels, gradients reach the embeddings through both the rendering and the eikonal
    (double-backward) term, and a few steps reduce the loss."""
    import ash
    from ash.render import SDFToDensity, accumulate_along_rays, render_weight_from_density

    G, cell = 8, 0.02
    grid = ash.UnBoundedSparseDenseGrid(3, 4000, 5, G, cell_size=cell, device=DEV)
    gen = torch.Generator(device=DEV).manual_seed(0)
    dirs = torch.nn.functional.normalize(torch.randn(60000, 3, generator=gen, device=DEV), dim=-1)
    grid.spatial_init_(dirs * 0.5, dilation=1, bidirectional=True)       # a shell around the sphere of radius 0.5
    gc, cc, gi, ci = grid.items()
    pos = grid.cell_to_world(gc, cc).view(gi.shape[0], -1, 3)
    with torch.no_grad():
        grid.embeddings[gi.view(-1), :, 0] = pos.norm(dim=-1) - 0.5 + 0.02 * torch.randn(pos.shape[:2], generator=gen, device=DEV)
        grid.embeddings[gi.view(-1), :, 1:4] = 0.5
    grid.construct_grid_neighbor_lut_(1, False)
    to_sigma = SDFToDensity(min_beta=cell, init_beta=2 * cell).to(DEV)
    opt = torch.optim.Adam(list(grid.parameters()) + list(to_sigma.parameters()), lr=1e-3)
    n_rays = 2048
    o = torch.nn.functional.normalize(torch.randn(n_rays, 3, generator=gen, device=DEV), dim=-1) * 0.8
    d = torch.nn.functional.normalize(-o + 0.1 * torch.randn(n_rays, 3, generator=gen, device=DEV), dim=-1)
    target = torch.full((n_rays, 3), 0.8, device=DEV)
    losses = []
    for step in range(4):
        near, far = grid.ray_find_near_far(o, d, 0.05, 2.0, 0.01)
        ri, t0, t1, prefix = grid.ray_sample(o, d, near, far, 64)
        assert ri.numel() > 10 * n_rays // 4 and (prefix[-1] == ri.numel())
        t_mid = 0.5 * (t0 + t1).view(-1, 1)
        x = (o[ri] + t_mid * d[ri]).requires_grad_(True)
        emb, masks = grid(x, interpolation="linear")
        sdf, rgb = emb[:, 0:1].contiguous(), emb[:, 1:4].contiguous()
        (sdf_grad,) = torch.autograd.grad(sdf, x, torch.ones_like(sdf), create_graph=True)
        sigma = to_sigma(sdf) * masks.view(-1, 1).float()
        w = render_weight_from_density(t0.view(-1, 1), t1.view(-1, 1), sigma, ri, n_rays)
        rendered = accumulate_along_rays(w, ri, rgb, n_rays)
        depth = accumulate_along_rays(w, ri, t_mid, n_rays)
        opacity = accumulate_along_rays(w, ri, None, n_rays)
        hit = (opacity > 0.5).float()
        eik = ((sdf_grad.norm(dim=-1) - 1) ** 2).mean()
        loss = ((rendered - target) ** 2 * hit).mean() + 0.1 * eik
        opt.zero_grad(set_to_none=True)
        loss.backward()
        assert torch.isfinite(grid.embeddings.grad).all() and grid.embeddings.grad[..., 0].abs().sum() > 0
        assert grid.embeddings.grad[..., 1:4].abs().sum() > 0 and to_sigma.beta.grad is not None
        opt.step()
        losses.append(float(loss.detach()))
        if step == 0:
            # rays aimed at the sphere see it at about the right depth (|o| - radius = 0.3)
            seen = opacity.view(-1) > 0.9
            assert seen.float().mean() > 0.5
            assert (depth.view(-1)[seen] / opacity.view(-1)[seen] - 0.3).abs().median() < 0.05
    assert losses[-1] < losses[0]
