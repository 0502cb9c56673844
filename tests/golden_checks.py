"""Checks of the Python layer + a native backend against the committed golden vectors
(tests/golden/*.npz, generated from the reference's Python layer by make_golden.py).
Shared by the CPU host-logic tests (backend = oracle stand-in) and the GPU parity tests
(backend = the CUDA library).  fp32 tolerance: 1e-5 relative / 1e-6 absolute."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
RTOL, ATOL = 1e-5, 1e-6


def load(name):
    return dict(np.load(os.path.join(GOLDEN, name + ".npz")))


def _t(a, device):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


def _np(t):
    return t.detach().cpu().numpy()


def _lexsort(k):
    return np.lexsort(k.T[::-1])


def check_hashmap(ash, device):
    g = load("hashmap")
    hm = ash.HashMap(3, {"sdf": 1, "rgb": 3}, 6000, device)
    hm.insert(_t(g["keys"], device), {"sdf": _t(g["sdf"], device), "rgb": _t(g["rgb"], device)})
    masks, indices, values = hm.find(_t(g["queries"], device), return_values=True)
    assert np.array_equal(_np(masks), g["masks"])
    assert (indices[~masks] == 0).all()
    assert np.array_equal(_np(values["sdf"] * masks[:, None]), g["found_sdf"])
    assert np.array_equal(_np(values["rgb"] * masks[:, None]), g["found_rgb"])
    hm.erase(_t(g["erase"], device))
    assert np.array_equal(_np(hm.find(_t(g["queries"], device))[0]), g["masks_after_erase"])
    assert hm.size() == int(g["size_after_erase"])
    k = _np(hm.keys())
    assert np.array_equal(k[_lexsort(k)], g["keys_after_erase"])


def build_grid(ash, device, g):
    G, D = int(g["G"]), int(g["D"])
    grid = ash.UnBoundedSparseDenseGrid(3, 200, D, G, cell_size=float(g["cell_size"]), device=device)
    coords, cell_coords, gi, ci = grid.spatial_init_(_t(g["points"], device), dilation=1, bidirectional=False)
    c = _np(coords).reshape(-1, 3)
    assert np.array_equal(c[_lexsort(c)], g["blocks"])
    assert cell_coords.shape == (1, G**3, 3) and gi.shape == (len(c), 1) and ci.shape == (1, G**3)
    idx, ok = grid.engine.find(_t(g["blocks"], device))
    assert ok.all()
    with torch.no_grad():
        grid.embeddings[idx] = _t(g["embeddings"], device)
    grid.construct_grid_neighbor_lut_(radius=1, bidirectional=False)
    return grid, idx


def check_grid(ash, device, name, rtol=RTOL, atol=ATOL):
    g = load(name)
    G = int(g["G"])
    grid, idx = build_grid(ash, device, g)
    x = _t(g["x"], device)
    gi, ci, off, mk = grid.query(grid.transform_world_to_cell(x))
    assert np.array_equal(_np(mk), g["masks"])
    assert np.array_equal(_np(ci), g["cell_indices"])
    assert np.array_equal(_np(off), g["offsets"])
    near, m = grid(x, "nearest")
    np.testing.assert_allclose(_np(near * m[:, None]), g["nearest"], rtol=rtol, atol=atol)
    for interp in ("linear", "smooth_step"):
        xr = x.clone().requires_grad_(True)
        grid.embeddings.grad = None
        y, m = grid(xr, interp)
        np.testing.assert_allclose(_np(y), g[f"{interp}_y"], rtol=rtol, atol=atol)
        w = _t(g[f"{interp}_w"], device)
        (gx,) = torch.autograd.grad((y * w).sum(), xr, create_graph=True)
        np.testing.assert_allclose(_np(gx), g[f"{interp}_grad_x"], rtol=4 * rtol, atol=4 * atol)
        (y * w).sum().backward(retain_graph=True)
        np.testing.assert_allclose(_np(grid.embeddings.grad[idx]), g[f"{interp}_grad_emb"], rtol=4 * rtol, atol=4 * atol)
        grid.embeddings.grad = None
        ((gx.norm(dim=-1) - 1) ** 2).mean().backward()
        np.testing.assert_allclose(_np(grid.embeddings.grad[idx]), g[f"{interp}_grad2_emb"], rtol=1e-4, atol=4 * atol)
    bmin, bmax = grid.get_bbox()
    assert np.array_equal(_np(bmin), g["bbox_min"]) and np.array_equal(_np(bmax), g["bbox_max"])
    if "lut_r3_c2g" in g:
        assert np.array_equal(_np(grid.lut_cell_nb2grid_nb), g["lut_r1_c2g"])
        assert np.array_equal(_np(grid.lut_cell_nb2cell_idx), g["lut_r1_c2c"])
        c2g, c2c = grid.construct_cell_neighbor_lut(3, True)
        assert np.array_equal(_np(c2g), g["lut_r3_c2g"]) and np.array_equal(_np(c2c), g["lut_r3_c2c"])
        before = grid.embeddings.detach().clone()
        grid.gaussian_filter_(3, 1.0)
        np.testing.assert_allclose(_np(grid.embeddings[idx]), g["gauss3"], rtol=rtol, atol=10 * atol)
        with torch.no_grad():
            grid.embeddings.copy_(before)
        o, d = _t(g["ray_o"], device), _t(g["ray_d"], device)
        nears, fars = grid.ray_find_near_far(o, d, 0.0, 12.0, 0.05)
        assert np.array_equal(_np(nears), g["ray_nears"]) and np.array_equal(_np(fars), g["ray_fars"])
        hit = nears >= 0
        ri, tn, tf, prefix = grid.ray_sample(o[hit], d[hit], nears[hit], fars[hit], 32)
        assert np.array_equal(_np(prefix), g["ray_prefix"]) and np.array_equal(_np(ri), g["ray_idx"])
        assert np.array_equal(_np(tn), g["ray_t_near"]) and np.array_equal(_np(tf), g["ray_t_far"])


def check_bounded(ash, device):
    g = load("bounded")
    bg = ash.BoundedSparseDenseGrid(3, 300, 2, grid_dim=4, sparse_grid_dim=6, bbox_min=torch.tensor([-1.0, -2.0, 0.0]),
                                    bbox_max=torch.tensor([1.0, 1.0, 1.5]), device=device)
    assert abs(bg.cell_size - float(g["cell_size"])) < 1e-9
    coords, _, _, _ = bg.spatial_init_(_t(g["points"], device), dilation=1, bidirectional=True)
    c = _np(coords).reshape(-1, 3)
    assert np.array_equal(c[_lexsort(c)], g["blocks"])
    x = _t(g["x"], device)
    _, ci, off, mk = bg.query(bg.transform_world_to_cell(x))
    assert np.array_equal(_np(mk), g["masks"])
    # (x - bbox_min) / cell_size: a true division on the CPU, a multiplication by the float
    # reciprocal on a CUDA tensor; away from cell faces both give the same cell
    same = _np(ci) == g["cell_indices"]
    assert same.mean() > 0.98
    np.testing.assert_allclose(_np(off)[same], g["offsets"][same], rtol=0, atol=2e-4)
    first_two = _t(g["blocks"][:0], device)  # shape only
    sorted_coords = coords.view(-1, 3)[torch.from_numpy(_lexsort(c)).to(device)]
    # cell_to_world of the reference's first two returned blocks: compare as a set of rows
    ours = _np(bg.cell_to_world(coords, bg.cell_coords))
    ref = g["cell_to_world"]
    ours_set = {tuple(np.round(r, 5)) for r in ours}
    assert all(tuple(np.round(r, 5)) in ours_set for r in ref)
