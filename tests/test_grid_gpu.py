"""Sparse-dense grid parity on the GPU: the reference's unittests/test_sparsedense_grid.py
replayed on the CUDA library, and forward / backward / double-backward outputs compared with
the CPU oracle.  fp32 results are held to the task's 1e-5 relative / 1e-6 absolute against the
oracle evaluated in float64 on the same inputs, relative to the sum of the magnitudes of the terms
each output adds up (tests/sum_bounds.py) -- the order of the scattered sums changes from run to
run, their bound does not; float64 results are compared directly at 1e-12."""
import numpy as np
import pytest
import torch

import oracle
import sum_bounds as sb

pytestmark = pytest.mark.gpu

DEV = torch.device("cuda:0")
RTOL, ATOL = 1e-5, 1e-6


def _cube_grid(G, D, bound, num_embeddings=1000, dtype=torch.float32, seed=0):
    """Blocks of the cube [-bound, bound]^3 active, embeddings ~ U(-1, 1)."""
    from ash import SparseDenseGrid

    grid = SparseDenseGrid(in_dim=3, num_embeddings=num_embeddings, embedding_dim=D, grid_dim=G, device=DEV)
    r = torch.arange(-bound, bound + 1, dtype=torch.int, device=DEV)
    blocks = G * torch.stack(torch.meshgrid(r, r, r, indexing="ij"), dim=-1).view(-1, 3)
    grid.spatial_init_(blocks, dilation=0)
    g = torch.Generator(device=DEV).manual_seed(seed)
    with torch.no_grad():
        grid.embeddings.copy_(torch.rand(grid.embeddings.shape, generator=g, device=DEV) * 2 - 1)
    if dtype == torch.float64:
        grid.embeddings = torch.nn.Parameter(grid.embeddings.detach().double())
    grid.construct_grid_neighbor_lut_(radius=1, bidirectional=False)
    return grid


def test_init_linearize_neighbor_items():
    """unittests/test_sparsedense_grid.py:21-104."""
    from ash import SparseDenseGrid

    for D, G in ((1, 4), (5, 8), (2, 16), (1, 3), (1, 2)):
        grid = SparseDenseGrid(3, 1000, D, G, DEV)
        assert grid.embeddings.shape == (1000, G**3, D)
        idx = torch.randint(grid.num_cells_per_grid, (100,), device=DEV)
        coords = grid._delinearize_cell_indices(idx)
        assert torch.all(grid._linearize_cell_coords(coords) == idx)
        assert torch.all(grid.lut_cell_nb2cell_idx[idx, 0] == idx)
        last = grid._delinearize_cell_indices(grid.lut_cell_nb2cell_idx[idx, -1])
        assert torch.all(last == (coords + 1) % G)
        keys = torch.arange(-1, 1, 1, dtype=torch.long, device=DEV).view(-1, 1).tile((1, 3))
        grid.spatial_init_(keys, dilation=0)
        gc, cc, gi, ci = grid.items()
        assert (gc * G + cc).shape == (2, G**3, 3)
        assert grid.embeddings[gi, ci].shape == (2, G**3, D)


@pytest.mark.parametrize("D,G", [(1, 2), (1, 8), (5, 8), (16, 8)])
def test_query_integer_positions_and_nearest(D, G):
    """unittests/test_sparsedense_grid.py:106-137."""
    from ash import SparseDenseGrid

    grid = SparseDenseGrid(3, 1000, D, G, DEV)
    torch.nn.init.uniform_(grid.embeddings, -1, 1)
    blocks = G * torch.arange(-1, 2, 1, dtype=torch.int, device=DEV).view(-1, 1).tile((1, 3))
    grid.spatial_init_(blocks, dilation=0)
    gc, cc, gi, ci = grid.items()
    coords = (gc * G + cc).view(-1, 3)
    gi2, ci2, offsets, masks = grid.query(coords)
    assert gi2.shape == (3 * G**3,) and ci2.shape == (3 * G**3,)
    assert torch.count_nonzero(offsets) == 0 and masks.all()
    feats, masks = grid(coords, interpolation="nearest")
    feats.sum().backward(retain_graph=True)
    assert grid.embeddings.grad is not None and masks.all()
    assert torch.allclose(feats, grid.embeddings[gi2, ci2])


@pytest.mark.parametrize("G", [1, 4, 8])
def test_linear_reproduces_coordinates(G):
    """Analytic known-answer test of unittests/test_sparsedense_grid.py:139-181: with
    embeddings[..., :3] = cell coordinates, linear interpolation returns the query point."""
    from ash import SparseDenseGrid

    bound = 3
    grid = SparseDenseGrid(3, 1000, 3, G, DEV)
    r = torch.arange(-bound, bound + 1, dtype=torch.int, device=DEV)
    blocks = G * torch.stack(torch.meshgrid(r, r, r, indexing="ij"), dim=-1).view(-1, 3)
    grid.spatial_init_(blocks, dilation=0)
    gc, cc, gi, ci = grid.items()
    coords = (gc * G + cc).view(-1, 3).float()
    with torch.no_grad():
        grid.embeddings[gi, ci, :3] = coords.view(gi.shape[0], ci.shape[1], 3)
    q = (2 * G * bound - 1) * torch.rand(1000, 3, device=DEV) - G * bound
    out, masks = grid(q, interpolation="linear")
    assert masks.all() and torch.allclose(out[..., :3], q)


def _oracle_inputs(grid, x):
    gi, ci, off, masks = grid.query(grid.transform_world_to_cell(x))
    t = lambda a: a.detach().cpu().numpy()
    return (gi, ci, off, masks), dict(
        emb=t(grid.embeddings), offsets=t(off), grid_indices=t(gi), cell_indices=t(ci), masks=t(masks),
        g2g=t(grid.lut_grid_nb2grid_idx), c2c=t(grid.lut_cell_nb2cell_idx), c2g=t(grid.lut_cell_nb2grid_nb))


def _close(a, b, rtol=RTOL, atol=ATOL):
    a = a.detach().cpu().numpy() if torch.is_tensor(a) else a
    np.testing.assert_allclose(a, b, rtol=rtol, atol=atol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("interp", ["linear", "smooth_step"])
@pytest.mark.parametrize("D,G", [(1, 8), (16, 8), (5, 8), (3, 4), (2, 1), (8, 2), (12, 4), (7, 3)])
def test_forward_backward_double_backward_vs_oracle(D, G, interp, dtype):
    import __ash

    grid = _cube_grid(G, D, bound=2, dtype=dtype, seed=D * 31 + G)
    n = 3000
    gen = torch.Generator(device=DEV).manual_seed(7 + D + G)
    # Reaches past the active cube on every side: exercises misses (mask False) and
    # queries whose +x/+y/+z neighbour block is absent (zero row, mask True).
    x = (torch.rand(n, 3, generator=gen, device=DEV) * (2 * 2 + 1.6) - 2.3) * G
    (gi, ci, off, masks), o = _oracle_inputs(grid, x)
    assert 0 < masks.sum() < n
    emb = grid.embeddings.detach()
    luts = (grid.lut_grid_nb2grid_idx, grid.lut_cell_nb2cell_idx, grid.lut_cell_nb2grid_nb)
    f32 = dtype == torch.float32
    z = torch.rand(n, D, generator=gen, device=DEV, dtype=dtype) - 0.5
    ggo = torch.rand(n, 3, generator=gen, device=DEV, dtype=dtype) - 0.5
    o64 = sb.as_float64(o)
    z64, ggo64 = z.double().cpu().numpy(), ggo.double().cpu().numpy()
    mag = sb.magnitudes(o, interp, z=z64, ggo=ggo64) if f32 else None

    def check(got, exact, what, extra=0.0):
        got = got.detach().cpu().numpy()
        if f32:   # 1e-5 * sum|terms| + 1e-6 against the float64 oracle
            sb.assert_within(got, exact, mag[what] + extra, what, RTOL, ATOL)
        else:     # the scattered sums meet in nondeterministic order: a few ulps
            np.testing.assert_allclose(got, exact, rtol=1e-11, atol=1e-12)

    y = __ash.query_forward(emb, off, gi, ci, masks, *luts, G, interp)
    y_ref = oracle.query_forward(interpolation=interp, **o64)
    check(y, y_ref, "y")
    if f32:  # the plain statement of the tolerance holds too where nothing is scattered
        _close(y, oracle.query_forward(interpolation=interp, **o), RTOL, ATOL)
    zero_rows = (y_ref == 0).all(axis=1) & o["masks"]
    assert zero_rows.any(), "test must include queries with an absent neighbour block"

    ge, go = __ash.query_backward_forward(z, emb, off, gi, ci, masks, *luts, G, interp)
    ge_ref, go_ref = oracle.query_backward_forward(z64, interpolation=interp, **o64)
    check(go, go_ref, "grad_off")
    check(ge, ge_ref, "grad_emb")

    gz, ge2, go2 = __ash.query_backward_backward(None, ggo, z, emb, off, gi, ci, masks, *luts, G, interp)
    gz_ref, ge2_ref, go2_ref = oracle.query_backward_backward(ggo64, z64, interpolation=interp, **o64)
    check(gz, gz_ref, "grad_z")
    check(ge2, ge2_ref, "grad2_emb")
    assert torch.count_nonzero(go2) == 0

    # accumulate-in-place mode adds on top of what is there (the 1 already there is one more term)
    acc = torch.ones_like(emb)
    __ash.query_backward_forward(z, emb, off, gi, ci, masks, *luts, G, interp, grad_embeddings_out=acc)
    check(acc - 1, ge_ref, "grad_emb", extra=1.0)


@pytest.mark.parametrize("D,G", [(2, 1), (1, 2), (4, 4), (8, 8)])
def test_autograd_first_order_matches_oracle(D, G):
    """The autograd path of unittests/test_sparsedense_grid.py:183-281 (d/dx and d/d embeddings
    through SparseDenseGridQuery), checked against the oracle's analytic gradients instead of
    finite differences."""
    grid = _cube_grid(G, D, bound=1, num_embeddings=64)
    n = 1000
    gen = torch.Generator(device=DEV).manual_seed(3)
    x = (torch.rand(n, 3, generator=gen, device=DEV) * 2.0 - 1.0) * G
    x.requires_grad_(True)
    for interp in ("linear", "smooth_step"):
        grid.embeddings.grad = None
        y, masks = grid(x, interpolation=interp)
        w = torch.rand(y.shape, generator=gen, device=DEV)
        (gx,) = torch.autograd.grad((y * w).sum(), x, retain_graph=True)
        (y * w).sum().backward()
        _, o = _oracle_inputs(grid, x.detach())
        w64 = w.double().cpu().numpy()
        ge_ref, go_ref = oracle.query_backward_forward(w64, interpolation=interp, **sb.as_float64(o))
        mag = sb.magnitudes(o, interp, z=w64)
        sb.assert_within(gx.cpu().numpy(), go_ref, mag["grad_off"], "grad_x")  # d offset / d x == 1 for the unit transform
        sb.assert_within(grid.embeddings.grad.cpu().numpy(), ge_ref, mag["grad_emb"], "grad_emb")


@pytest.mark.parametrize("D,G", [(1, 2), (4, 4), (16, 8)])
def test_autograd_double_backward_eikonal(D, G):
    """Gradient-of-gradient training signal (eikonal-style), the use the reference's
    SparseDenseGridQueryBackward exists for (demo/train_scene_recon.py:103-108, :326): compare
    d loss / d embeddings with the oracle's double backward."""
    grid = _cube_grid(G, D, bound=1, num_embeddings=64)
    n = 500
    gen = torch.Generator(device=DEV).manual_seed(11)
    x = ((torch.rand(n, 3, generator=gen, device=DEV) * 2.0 - 1.0) * G).requires_grad_(True)
    y, masks = grid(x, interpolation="linear")
    ones = torch.ones_like(y)
    (gx,) = torch.autograd.grad(y, x, grad_outputs=ones, create_graph=True)
    loss = ((gx.norm(dim=-1) - 1) ** 2).mean()
    grid.embeddings.grad = None
    loss.backward()
    # by hand: dloss/dgx, then the oracle's backward_backward with z = ones
    gx_d = gx.detach()
    nrm = gx_d.norm(dim=-1, keepdim=True)
    dl_dgx = (2 * (nrm - 1) / n) * gx_d / nrm.clamp_min(1e-30)
    _, o = _oracle_inputs(grid, x.detach())
    ggo64, ones64 = dl_dgx.double().cpu().numpy(), ones.double().cpu().numpy()
    _, ge_ref, _ = oracle.query_backward_backward(ggo64, ones64, interpolation="linear", **sb.as_float64(o))
    mag = sb.magnitudes(o, "linear", z=ones64, ggo=ggo64)
    sb.assert_within(grid.embeddings.grad.cpu().numpy(), ge_ref, mag["grad2_emb"], "eikonal grad_emb")


def test_gradcheck_float64():
    """Finite-difference check of both autograd levels in float64 (the helper the reference
    defines at unittests/test_sparsedense_grid.py:283-347 but never calls)."""
    from ash import SparseDenseGridQuery, SparseDenseGridQueryBackward

    G, D = 2, 3
    grid = _cube_grid(G, D, bound=1, num_embeddings=32, dtype=torch.float64)
    gen = torch.Generator(device=DEV).manual_seed(5)
    x = (torch.rand(50, 3, generator=gen, device=DEV) * 1.6 - 0.8) * G
    gi, ci, off, masks = grid.query(x)
    luts = (grid.lut_grid_nb2grid_idx, grid.lut_cell_nb2cell_idx, grid.lut_cell_nb2grid_nb)
    emb = grid.embeddings.detach().clone().requires_grad_(True)
    z = torch.rand(50, D, generator=gen, device=DEV, dtype=torch.float64).requires_grad_(True)

    f1 = lambda e: SparseDenseGridQuery.apply(e, off, gi, ci, masks, *luts, G, "smooth_step")
    assert torch.autograd.gradcheck(f1, (emb,), eps=1e-6, atol=1e-6, rtol=1e-6, nondet_tol=1e-12)
    f2 = lambda zz, e: SparseDenseGridQueryBackward.apply(zz, e, off, gi, ci, masks, *luts, G, "linear")[1]
    assert torch.autograd.gradcheck(f2, (z, emb), eps=1e-6, atol=1e-6, rtol=1e-6, nondet_tol=1e-12)
