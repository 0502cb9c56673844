"""Fused ray renderer against the composition it replaces.

The reference's training step (demo/train_scene_recon.py:64-161) chains ray_find_near_far ->
ray_sample -> grid(x) -> autograd.grad(sdf, x) -> normalize -> SDFToDensity -> rendering weights
-> per-ray sums.  Every piece of that chain is checked against the CPU oracle elsewhere
(bit-exact sampler, query forward / backward / double backward, rendering accumulation); here the
one-launch renderer must reproduce the chain's per-ray outputs and its gradients w.r.t. the
embeddings and the density scale.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

import ash  # noqa: E402
from ash.render import SDFToDensity, accumulate_along_rays, render_rays, render_weight_from_density  # noqa: E402

DEV = torch.device("cuda:0")


def make_grid(kind, D, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    if kind == "bounded":
        grid = ash.BoundedSparseDenseGrid(3, 6000, D, grid_dim=8, sparse_grid_dim=16, device=DEV)
        # a thick spherical shell of points inside the [-1, 1]^3 box
        dirs = torch.nn.functional.normalize(torch.randn(60000, 3, device=DEV, generator=g), dim=-1)
        radius = 0.55 + 0.12 * torch.rand(60000, 1, device=DEV, generator=g)
        grid.spatial_init_(dirs * radius, dilation=0)
    else:
        grid = ash.UnBoundedSparseDenseGrid(3, 6000, D, 8, cell_size=0.02, device=DEV)
        dirs = torch.nn.functional.normalize(torch.randn(60000, 3, device=DEV, generator=g), dim=-1)
        radius = 0.9 + 0.2 * torch.rand(60000, 1, device=DEV, generator=g)
        grid.spatial_init_(dirs * radius + torch.tensor([0.3, -0.2, 0.1], device=DEV), dilation=0)
    with torch.no_grad():
        grid.embeddings.normal_(0.0, 1.0, generator=g)
        grid.embeddings[..., 0] *= 0.6 * grid.cell_size      # |grad sdf| of order one
        grid.embeddings[..., 1:4].mul_(0.3).add_(0.5)
    grid.construct_grid_neighbor_lut_(radius=1, bidirectional=False)
    return grid


def make_rays(grid, n, seed, centre):
    g = torch.Generator(device=DEV).manual_seed(seed)
    extent = 0.25 if isinstance(grid, ash.BoundedSparseDenseGrid) else 0.4
    o = centre + (torch.rand(n, 3, device=DEV, generator=g) - 0.5) * extent
    d = torch.nn.functional.normalize(torch.randn(n, 3, device=DEV, generator=g), dim=-1)
    return o.contiguous(), d.contiguous()


def composed(grid, o, d, t_min, t_max, max_samples, to_sigma, interpolation):
    """The chain of demo/train_scene_recon.py:64-161 on this repo's ops."""
    n = o.shape[0]
    nears, fars = grid.ray_find_near_far(o, d, t_min, t_max, 0.01)
    ri, t0, t1, _ = grid.ray_sample(o, d, nears, fars, max_samples)
    t0, t1 = t0.view(-1, 1), t1.view(-1, 1)
    t_mid = 0.5 * (t0 + t1)
    x = (o[ri] + t_mid * d[ri]).requires_grad_(True)
    emb, masks = grid(x, interpolation=interpolation)
    sdf, rgb = emb[:, 0:1].contiguous(), emb[:, 1:4].contiguous()
    (g,) = torch.autograd.grad(sdf, x, torch.ones_like(sdf), create_graph=True)
    normals = torch.nn.functional.normalize(g, dim=-1)
    sigma = to_sigma(sdf) * masks.view(-1, 1).float()
    w = render_weight_from_density(t0, t1, sigma, ri, n)
    r = g.norm(dim=-1, keepdim=True) - 1
    per_ray = lambda v: torch.zeros(n, 1, device=DEV).index_add(0, ri, v)
    return {"rgb": accumulate_along_rays(w, ri, rgb, n), "depth": accumulate_along_rays(w, ri, t_mid, n),
            "normal": accumulate_along_rays(w, ri, normals, n), "weights": accumulate_along_rays(w, ri, None, n),
            "eikonal_l1": per_ray(r.abs()), "eikonal_l2": per_ray(r * r),
            "n_samples": per_ray(torch.ones_like(r)).detach(), "near": nears.view(-1, 1), "far": fars.view(-1, 1)}


def loss_of(res, coef):
    return sum((res[k] * coef[k]).sum() for k in coef)


CASES = [("bounded", 4, "linear"), ("bounded", 5, "linear"), ("unbounded", 4, "smooth_step"), ("unbounded", 8, "linear")]


@pytest.mark.parametrize("parallel", [False, True])
@pytest.mark.parametrize("kind,D,interpolation", CASES)
def test_fused_renderer_matches_the_composed_chain(kind, D, interpolation, parallel):
    grid = make_grid(kind, D, seed=3 + D)
    centre = torch.zeros(3, device=DEV) if kind == "bounded" else torch.tensor([0.3, -0.2, 0.1], device=DEV)
    n = 3000
    o, d = make_rays(grid, n, 11, centre)
    t_min, t_max = (0.05, 2.0) if kind == "bounded" else (0.1, 2.5)
    to_sigma = SDFToDensity(min_beta=0.5 * grid.cell_size, init_beta=2.0 * grid.cell_size).to(DEV)
    g = torch.Generator(device=DEV).manual_seed(5)
    coef = {k: torch.randn(n, c, device=DEV, generator=g) for k, c in
            (("rgb", 3), ("depth", 1), ("normal", 3), ("weights", 1))}
    coef["eikonal_l1"] = torch.full((n, 1), 0.01, device=DEV)
    coef["eikonal_l2"] = torch.full((n, 1), 0.02, device=DEV)

    grid.embeddings.grad = None
    to_sigma.beta.grad = None
    ref = composed(grid, o, d, t_min, t_max, 48, to_sigma, interpolation)
    loss_of(ref, coef).backward()
    ref_ge, ref_gb = grid.embeddings.grad.clone(), to_sigma.beta.grad.clone()

    grid.embeddings.grad = None
    to_sigma.beta.grad = None
    beta = to_sigma.min_beta + to_sigma.beta.abs()
    out = render_rays(grid, o, d, t_min, t_max, 48, beta, interpolation, parallel_samples=parallel)
    loss_of(out, coef).backward()
    ge, gb = grid.embeddings.grad, to_sigma.beta.grad

    assert float(ref["n_samples"].sum()) > 5 * n and float((ref["n_samples"] > 0).float().mean()) > 0.5
    assert torch.equal(out["n_samples"], ref["n_samples"])
    assert torch.equal(out["near"], ref["near"]) and torch.equal(out["far"], ref["far"])
    for k in ("rgb", "depth", "normal", "weights", "eikonal_l1", "eikonal_l2"):
        torch.testing.assert_close(out[k], ref[k], rtol=2e-4, atol=2e-5, msg=lambda m, k=k: f"{k}: {m}")
    scale = float(ref_ge.abs().max())
    assert scale > 0
    torch.testing.assert_close(ge, ref_ge, rtol=1e-3, atol=2e-5 * scale)
    torch.testing.assert_close(gb, ref_gb, rtol=1e-3, atol=1e-4 * float(ref_gb.abs().max()))


def test_rays_without_a_hit_can_be_skipped():
    grid = make_grid("bounded", 4, seed=9)
    o, d = make_rays(grid, 2000, 13, torch.zeros(3, device=DEV))
    o[:500] = torch.tensor([0.95, 0.95, 0.95], device=DEV)       # a corner of the box, looking outwards
    d[:500] = torch.nn.functional.normalize(torch.rand(500, 3, device=DEV) + 0.2, dim=-1)
    beta = torch.tensor([0.02], device=DEV)
    with torch.no_grad():
        full = render_rays(grid, o, d, 0.05, 2.0, 32, beta)
        skip = render_rays(grid, o, d, 0.05, 2.0, 32, beta, skip_rays_without_hit=True)
        listed = render_rays(grid, o, d, 0.05, 2.0, 32, beta, skip_rays_without_hit=True, parallel_samples=True)
    for k in ("n_samples", "near", "far"):
        assert torch.equal(listed[k], skip[k])
    for k in ("rgb", "depth", "normal", "weights"):
        torch.testing.assert_close(listed[k], skip[k], rtol=2e-4, atol=2e-5)
    with torch.no_grad():
        pass
    missed = full["near"].view(-1) < 0
    assert int(missed.sum()) >= 500 and int((~missed).sum()) > 500
    for k in ("rgb", "depth", "normal", "weights", "n_samples"):
        assert torch.equal(skip[k][~missed], full[k][~missed])
        assert float(skip[k][missed].abs().max()) == 0.0


def test_in_place_gradient_mode_and_empty_batch():
    grid = make_grid("bounded", 4, seed=21)
    o, d = make_rays(grid, 1500, 17, torch.zeros(3, device=DEV))
    beta = torch.tensor([0.03], device=DEV, requires_grad=True)
    grid.embeddings.grad = None
    out = render_rays(grid, o, d, 0.05, 2.0, 32, beta)
    (out["rgb"].sum() + out["depth"].sum()).backward()
    dense, gb = grid.embeddings.grad.clone(), beta.grad.clone()
    grid.embeddings.grad, beta.grad = None, None
    grid.grad_mode = "in_place"
    for parallel in (False, True):           # accumulates: two passes give twice the gradient
        out = render_rays(grid, o, d, 0.05, 2.0, 32, beta, parallel_samples=parallel)
        (out["rgb"].sum() + out["depth"].sum()).backward()
    grid.grad_mode = "dense"
    scale = float(dense.abs().max())
    torch.testing.assert_close(grid.embeddings.grad, 2 * dense, rtol=1e-4, atol=1e-5 * scale)
    torch.testing.assert_close(beta.grad, 2 * gb, rtol=1e-4, atol=0)
    empty = render_rays(grid, o[:0], d[:0], 0.05, 2.0, 32, beta.detach())
    assert empty["rgb"].shape == (0, 3) and empty["n_samples"].shape == (0, 1)


def test_embedding_dim_below_four_is_refused():
    grid = ash.BoundedSparseDenseGrid(3, 100, 3, grid_dim=4, sparse_grid_dim=4, device=DEV)
    grid.dense_init_()
    o = torch.zeros(4, 3, device=DEV)
    d = torch.nn.functional.normalize(torch.ones(4, 3, device=DEV), dim=-1)
    with pytest.raises(RuntimeError):
        render_rays(grid, o, d, 0.05, 1.0, 8, torch.tensor([0.1], device=DEV))


@pytest.mark.parametrize("parallel", [False, True])
def test_fused_forward_against_the_cpu_oracle(parallel):
    """Per-ray outputs of the one-launch renderer against the CPU oracle run stage by stage:
    oracle near/far -> oracle sampler -> oracle query forward + d/d offset -> numpy density ->
    oracle rendering quadrature."""
    import numpy as np

    import oracle
    from oracle import render as orender

    f32 = np.float32
    grid = make_grid("bounded", 4, seed=31)
    n = 800
    o, d = make_rays(grid, n, 19, torch.zeros(3, device=DEV))
    t_min, t_max, max_samples, beta = 0.05, 2.0, 40, 0.03
    with torch.no_grad():
        out = render_rays(grid, o, d, t_min, t_max, max_samples, torch.tensor([beta], device=DEV), "linear",
                          parallel_samples=parallel)

    G, cs = grid.grid_dim, grid.cell_size
    keys, idx = grid.engine.items()
    hm = oracle.OracleHashMap(3, grid.engine.capacity)
    hm.load_states(keys.cpu().numpy(), idx.cpu().numpy(), grid.engine._heap.cpu().numpy())
    o_c = grid.transform_world_to_cell(o).cpu().numpy()
    o_w, d_np = o.cpu().numpy(), d.cpu().numpy()
    lo, hi = (grid.transform_world_to_cell(b).cpu().numpy() for b in grid.get_bbox())
    nears_c, fars_c = oracle.ray_find_near_far(hm, o_c, d_np, lo, hi, t_min / cs, t_max / cs, 0.01 / cs, float(G))
    nears_w, fars_w = nears_c * f32(cs), fars_c * f32(cs)
    inv_cs = f32(1.0 / cs)
    ri, t0c, t1c, _ = oracle.ray_sample(hm, o_c, d_np, nears_w * inv_cs, fars_w * inv_cs, lo, hi, max_samples, float(G))
    t0w, t1w = t0c * f32(cs), t1c * f32(cs)
    t_mid = f32(0.5) * (t0w + t1w)
    x = o_w[ri] + t_mid[:, None] * d_np[ri]
    xc = (x - np.asarray(grid._origin, f32)) * inv_cs
    block = np.floor(xc * f32(1.0 / G))
    local = xc - block * f32(G)
    cell = np.floor(local)
    off = (local - cell).astype(f32)
    gi, mk = hm.find(block.astype(np.int32))
    ci = (np.clip(cell.astype(np.int64), 0, G - 1) * np.array([1, G, G * G])).sum(-1)
    luts = [t.cpu().numpy() for t in (grid.lut_grid_nb2grid_idx, grid.lut_cell_nb2cell_idx, grid.lut_cell_nb2grid_nb)]
    emb = grid.embeddings.detach().cpu().numpy()
    y = oracle.query_forward(emb, off, gi, ci, mk, *luts, "linear")
    z = np.zeros_like(y)
    z[:, 0] = 1
    _, grad_off = oracle.query_backward_forward(z, emb, off, gi, ci, mk, *luts, "linear")
    g = grad_off.astype(np.float64) * float(inv_cs)
    gnorm = np.linalg.norm(g, axis=1, keepdims=True)
    normals = g / np.maximum(gnorm, 1e-12)
    sdf = y[:, 0].astype(np.float64)
    sigma = (1 / beta) * (0.5 + 0.5 * np.sign(sdf) * np.expm1(-np.abs(sdf) / beta)) * mk
    w = orender.render_weights(t0w, t1w, sigma, ri, n)
    want = np.concatenate([orender.accumulate(w, ri, y[:, 1:4], n), orender.accumulate(w, ri, t_mid, n),
                           orender.accumulate(w, ri, normals, n), orender.accumulate(w, ri, None, n),
                           orender.accumulate(np.ones_like(w), ri, np.abs(gnorm - 1), n),
                           orender.accumulate(np.ones_like(w), ri, (gnorm - 1) ** 2, n),
                           orender.accumulate(np.ones_like(w), ri, None, n)], axis=1)
    got = torch.cat([out[k] for k in ("rgb", "depth", "normal", "weights", "eikonal_l1", "eikonal_l2", "n_samples")],
                    dim=1).cpu().numpy()
    assert len(ri) > 5 * n
    np.testing.assert_array_equal(got[:, 10], want[:, 10])                     # same samples on every ray
    np.testing.assert_array_equal(out["near"].cpu().numpy().ravel(), nears_w)  # bit-exact first stage
    np.testing.assert_array_equal(out["far"].cpu().numpy().ravel(), fars_w)
    np.testing.assert_allclose(got, want, rtol=2e-4, atol=2e-5)
