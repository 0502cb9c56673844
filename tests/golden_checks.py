"""Checks of the Python layer + a native backend against the committed golden vectors
(tests/golden/*.npz, generated from the reference's Python layer by make_golden.py).
Shared by the CPU host-logic tests (backend = oracle stand-in) and the GPU parity tests
(backend = the CUDA library).  fp32 tolerance: 1e-5 relative / 1e-6 absolute; for gradients, which
are sums of signed terms (scattered in nondeterministic order on the GPU), relative to the sum of
the magnitudes of those terms (tests/sum_bounds.py)."""
import os

import numpy as np
import torch

import sum_bounds as sb

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
    o = dict(emb=_np(grid.embeddings), offsets=_np(off), grid_indices=_np(gi), cell_indices=_np(ci), masks=_np(mk),
             g2g=_np(grid.lut_grid_nb2grid_idx), c2c=_np(grid.lut_cell_nb2cell_idx), c2g=_np(grid.lut_cell_nb2grid_nb))
    inv_cell = 1.0 / float(g["cell_size"])      # d offset / d x
    rows = _np(idx)
    for interp in ("linear", "smooth_step"):
        xr = x.clone().requires_grad_(True)
        grid.embeddings.grad = None
        y, m = grid(xr, interp)
        np.testing.assert_allclose(_np(y), g[f"{interp}_y"], rtol=rtol, atol=atol)
        w = _t(g[f"{interp}_w"], device)
        (gx,) = torch.autograd.grad((y * w).sum(), xr, create_graph=True)
        dl_dgx = torch.autograd.grad(((gx.norm(dim=-1) - 1) ** 2).mean(), gx, retain_graph=True)[0]
        mag = sb.magnitudes(o, interp, z=_np(w), ggo=np.abs(_np(dl_dgx)) * inv_cell)
        sb.assert_within(_np(gx), g[f"{interp}_grad_x"], mag["grad_off"] * inv_cell, f"{name} {interp} grad_x", rtol, atol)
        (y * w).sum().backward(retain_graph=True)
        sb.assert_within(_np(grid.embeddings.grad[idx]), g[f"{interp}_grad_emb"], mag["grad_emb"][rows],
                         f"{name} {interp} grad_emb", rtol, atol)
        grid.embeddings.grad = None
        ((gx.norm(dim=-1) - 1) ** 2).mean().backward()
        # the incoming gradient of this pass is itself an fp32 function of grad_x: its relative error
        # (a few 1e-7) adds to the sum's, which the same bound absorbs
        sb.assert_within(_np(grid.embeddings.grad[idx]), g[f"{interp}_grad2_emb"], mag["grad2_emb"][rows],
                         f"{name} {interp} grad2_emb", rtol, atol)
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


def check_checkpoints(ash, device):
    """Checkpoints WRITTEN BY THE REFERENCE's Python layer (tests/golden/make_checkpoints.py; format of
    ash/core.py:69-135) load into this repository's classes and answer as the reference did."""
    ck = torch.load(os.path.join(GOLDEN, "ckpt_hashmap.pt"), map_location="cpu")
    c = ck["ctor"]
    hm = ash.HashMap(c["dim"], c["value_dims"], c["capacity"], device)
    assert set(hm.state_dict().keys()) == set(ck["state_dict"].keys())
    hm.load_state_dict(ck["state_dict"])
    assert hm.size() == ck["size"]
    masks, indices, values = hm.find(ck["queries"].to(device), return_values=True)
    assert torch.equal(masks.cpu(), ck["masks"])
    assert torch.equal((values["sdf"] * masks[:, None]).cpu(), ck["found_sdf"])
    assert torch.equal((values["rgb"] * masks[:, None]).cpu(), ck["found_rgb"])
    k = _np(hm.keys())
    assert np.array_equal(k[_lexsort(k)], ck["keys_sorted"].numpy())
    # the restored free-index stack keeps handing out unused indices: new keys do not disturb old values
    fresh = torch.tensor([[40, 41, 42], [43, 44, 45]], dtype=torch.int32, device=device)
    hm.insert(fresh, {"sdf": torch.full((2, 1), 5.0, device=device), "rgb": torch.full((2, 3), 6.0, device=device)})
    masks2, _, values2 = hm.find(ck["queries"].to(device), return_values=True)
    assert torch.equal(masks2.cpu(), ck["masks"]) and torch.equal((values2["sdf"] * masks2[:, None]).cpu(), ck["found_sdf"])
    assert hm.size() == ck["size"] + 2

    ck = torch.load(os.path.join(GOLDEN, "ckpt_grid.pt"), map_location="cpu")
    c = ck["ctor"]
    grid = ash.UnBoundedSparseDenseGrid(3, c["num_embeddings"], c["embedding_dim"], c["grid_dim"],
                                        cell_size=c["cell_size"], device=device)
    assert set(grid.state_dict().keys()) == set(ck["state_dict"].keys())
    grid.load_state_dict(ck["state_dict"])
    assert grid.engine.size() == ck["n_blocks"]
    for interp in ("linear", "smooth_step"):
        y, m = grid(ck["x"].to(device), interp)
        assert torch.equal(m.cpu(), ck["masks"])
        np.testing.assert_allclose(_np(y), ck[f"{interp}_y"].numpy(), rtol=RTOL, atol=ATOL)
    # and back: a checkpoint written here has the reference's keys, shapes and dtypes
    mine = grid.state_dict()
    for name, ref in ck["state_dict"].items():
        assert mine[name].shape == ref.shape and mine[name].dtype == ref.dtype, name


def check_resize(ash, device):
    """Growing keeps every live key at its index, keeps the values, keeps handing out only unused
    indices afterwards; shrinking (the reference's re-insertion, ash/core.py:266-302) keeps the
    key -> value association."""
    g = torch.Generator().manual_seed(9)
    keys = torch.randint(-30, 30, (900, 3), generator=g, dtype=torch.int32).to(device)
    val = lambda k: {"sdf": k[:, :1].float() * 0.5 + k[:, 1:2].float() * 11, "rgb": k.float()}
    hm = ash.HashMap(3, {"sdf": 1, "rgb": 3}, 1000, device)
    hm.insert(keys, val(keys))
    hm.erase(keys[:200])                               # the free-index stack is no longer the identity
    live_keys, live_idx = hm.engine.items()
    n = hm.size()
    hm.resize(2500)
    assert hm.engine.capacity == 2500 and hm.size() == n
    idx_after, ok = hm.engine.find(live_keys)
    assert ok.all() and torch.equal(idx_after, live_idx), "growing must not move live keys"
    masks, _, got = hm.find(live_keys, return_values=True)
    assert masks.all() and torch.equal(got["rgb"], live_keys.float())
    fresh = (torch.arange(1500, dtype=torch.int32).view(-1, 1) + 100).tile((1, 3)).to(device)
    hm.insert(fresh, val(fresh))                       # fills the map beyond its old capacity
    assert hm.size() == n + 1500
    all_keys, all_idx = hm.engine.items()
    assert torch.unique(all_idx).numel() == n + 1500 and int(all_idx.max()) < 2500 and int(all_idx.min()) >= 0
    masks, _, got = hm.find(all_keys, return_values=True)
    assert masks.all() and torch.equal(got["rgb"], all_keys.float())
    assert torch.equal(hm.engine.find(live_keys)[0], live_idx)
    hm.erase(fresh[:1400])
    hm.resize(n + 150)                                 # shrink: re-insertion, indices may change
    assert hm.size() == n + 100
    masks, _, got = hm.find(all_keys, return_values=True)
    assert int(masks.sum()) == n + 100 and torch.equal(got["rgb"][masks], all_keys[masks].float())
    # an empty map and a set grow too
    empty = ash.HashSet(2, 10, device)
    empty.resize(50)
    assert empty.size() == 0 and empty.engine.capacity == 50
    empty.insert(torch.arange(80, dtype=torch.int32).view(-1, 2).to(device))
    assert empty.size() == 40
