"""Generate tests/golden/*.npz from the REFERENCE's Python layer.

    python tests/golden/make_golden.py /path/to/torch-ash

The reference's unmodified ``ash`` package is imported from the given tree and runs on
``device="cpu"`` on top of the CPU oracle's stand-in for its native module
(oracle/ref_backend).  Everything host-side -- block/cell/offset split, lookup tables,
spatial_init_, coordinate transforms, autograd wiring, Gaussian weights -- is therefore the
reference's own code; only the native kernels are the oracle's restatement.  The vectors are
stored free of raw indices (their order is implementation defined): per-query results in query
order, per-cell tensors keyed by sorted block coordinate.

The fixtures are committed; this script only needs re-running if the oracle changes.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def main(ref_root):
    sys.path[:0] = [os.path.join(ROOT, "oracle", "ref_backend"), ROOT, ref_root]
    import torch

    import ash  # the reference's

    assert os.path.abspath(ash.__file__).startswith(os.path.abspath(ref_root))
    cpu = torch.device("cpu")
    torch.manual_seed(15213)
    rng = np.random.default_rng(15213)

    def by_block(grid, tensor):
        """(blocks sorted lexicographically (n,3), tensor rows of those blocks (n, cells, D))."""
        keys, idx = grid.engine.items()
        k = keys.numpy()
        order = np.lexsort(k.T[::-1])
        return k[order], tensor.detach()[idx[torch.from_numpy(order)]].numpy()

    # ---------------------------------------------------------------- hash map (config-1 shaped, small)
    keys = torch.from_numpy(rng.integers(-16, 16, (3000, 3)).astype(np.int32))
    sdf = keys[:, :1].float() * 0.25 + keys[:, 1:2].float() * 3 + keys[:, 2:3].float() * 100
    rgb = keys.float() * 0.5
    hm = ash.HashMap(3, {"sdf": 1, "rgb": 3}, 6000, cpu)
    hm.insert(keys, {"sdf": sdf, "rgb": rgb})
    queries = torch.from_numpy(rng.integers(-20, 20, (4000, 3)).astype(np.int32))
    masks, indices, values = hm.find(queries, return_values=True)
    erase = keys[:500]
    hm.erase(erase)
    masks2 = hm.find(queries)[0]
    items_keys = hm.keys().numpy()
    np.savez_compressed(
        os.path.join(HERE, "hashmap.npz"), keys=keys.numpy(), sdf=sdf.numpy(), rgb=rgb.numpy(), queries=queries.numpy(),
        masks=masks.numpy(), found_sdf=(values["sdf"] * masks[:, None]).numpy(),
        found_rgb=(values["rgb"] * masks[:, None]).numpy(), erase=erase.numpy(), masks_after_erase=masks2.numpy(),
        size_after_erase=hm.size(), keys_after_erase=items_keys[np.lexsort(items_keys.T[::-1])])

    # ---------------------------------------------------------------- grid query + autograd
    # The reference deduplicates candidate blocks in a hash set sized by the POINT count
    # (ash/grid.py:145); its behaviour when that overflows is undefined, so every case keeps
    # the number of distinct candidate blocks below the number of points.
    for name, G, D, n_pts, reach in (("grid_g4_d3", 4, 3, 150, 1.5), ("grid_g8_d4", 8, 4, 40, 0.9),
                                     ("grid_g4_d16", 4, 16, 40, 0.9), ("grid_g2_d1", 2, 1, 150, 1.5)):
        grid = ash.UnBoundedSparseDenseGrid(3, 200, D, G, cell_size=0.25, device=cpu)
        half = reach * G * 0.25
        pts = torch.from_numpy(rng.uniform(-half, half, (n_pts, 3)).astype(np.float32))
        unique_coords, _, _, _ = grid.spatial_init_(pts, dilation=1, bidirectional=False)
        with torch.no_grad():
            grid.embeddings.copy_(torch.from_numpy(rng.standard_normal(tuple(grid.embeddings.shape)).astype(np.float32)))
        blocks_sorted, emb_sorted = by_block(grid, grid.embeddings)
        grid.construct_grid_neighbor_lut_(radius=1, bidirectional=False)
        assert unique_coords.shape[0] < n_pts
        x = torch.from_numpy(rng.uniform(-half - 0.6 * G * 0.25, half + 1.2 * G * 0.25, (600, 3)).astype(np.float32))
        out = dict(points=pts.numpy(), blocks=blocks_sorted, embeddings=emb_sorted, x=x.numpy(), cell_size=0.25, G=G, D=D)
        gi, ci, off, mk = grid.query(grid.transform_world_to_cell(x))
        out.update(cell_indices=ci.numpy(), offsets=off.numpy(), masks=mk.numpy())
        out["nearest"] = (grid(x, "nearest")[0] * mk[:, None]).detach().numpy()
        for interp in ("linear", "smooth_step"):
            xr = x.clone().requires_grad_(True)
            grid.embeddings.grad = None
            y, m = grid(xr, interp)
            w = torch.from_numpy(rng.uniform(-1, 1, tuple(y.shape)).astype(np.float32))
            (gx,) = torch.autograd.grad((y * w).sum(), xr, create_graph=True)
            (y * w).sum().backward(retain_graph=True)
            ge = grid.embeddings.grad.clone()
            grid.embeddings.grad = None
            # eikonal-style second order signal
            ((gx.norm(dim=-1) - 1) ** 2).mean().backward()
            ge2 = grid.embeddings.grad.clone()
            out[f"{interp}_y"] = y.detach().numpy()
            out[f"{interp}_w"] = w.numpy()
            out[f"{interp}_grad_x"] = gx.detach().numpy()
            out[f"{interp}_grad_emb"] = by_block(grid, ge)[1]
            out[f"{interp}_grad2_emb"] = by_block(grid, ge2)[1]
        bmin, bmax = grid.get_bbox()
        out.update(bbox_min=bmin.numpy(), bbox_max=bmax.numpy())
        if G == 4:
            c2g, c2c = grid.construct_cell_neighbor_lut(3, True)
            out.update(lut_r1_c2g=grid.lut_cell_nb2grid_nb.numpy(), lut_r1_c2c=grid.lut_cell_nb2cell_idx.numpy(),
                       lut_r3_c2g=c2g.numpy().astype(np.int16), lut_r3_c2c=c2c.numpy().astype(np.int16))
            before = grid.embeddings.detach().clone()
            grid.gaussian_filter_(3, 1.0)
            out["gauss3"] = by_block(grid, grid.embeddings)[1]
            with torch.no_grad():
                grid.embeddings.copy_(before)
            # rays
            o = torch.from_numpy(rng.uniform(-4, 4, (300, 3)).astype(np.float32))
            tgt = torch.from_numpy(rng.uniform(-1.5, 1.5, (300, 3)).astype(np.float32))
            d = torch.nn.functional.normalize(tgt - o, dim=-1)
            nears, fars = grid.ray_find_near_far(o, d, 0.0, 12.0, 0.05)
            hit = nears >= 0
            ri, tn, tf, prefix = grid.ray_sample(o[hit], d[hit], nears[hit], fars[hit], 32)
            out.update(ray_o=o.numpy(), ray_d=d.numpy(), ray_nears=nears.numpy(), ray_fars=fars.numpy(),
                       ray_idx=ri.numpy(), ray_t_near=tn.numpy(), ray_t_far=tf.numpy(), ray_prefix=prefix.numpy())
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)

    # ---------------------------------------------------------------- bounded grid geometry
    bg = ash.BoundedSparseDenseGrid(3, 300, 2, grid_dim=4, sparse_grid_dim=6,
                                    bbox_min=torch.tensor([-1.0, -2.0, 0.0]), bbox_max=torch.tensor([1.0, 1.0, 1.5]),
                                    device=cpu)
    # cell_size is set by the shortest box side, so the 6 x 4 cells span 24 * cell_size from bbox_min
    lo = bg.bbox_min.numpy() - 0.1
    hi = bg.bbox_min.numpy() + 24 * bg.cell_size + 0.1
    pts = torch.from_numpy(rng.uniform(lo, hi, (1500, 3)).astype(np.float32))
    coords, _, _, _ = bg.spatial_init_(pts, dilation=1, bidirectional=True)
    blk = torch.floor(bg.transform_world_to_cell(pts) / 4)
    n_inside = int(((blk >= 0) & (blk < 6)).all(dim=1).sum())
    assert 8**3 < n_inside  # more in-bound points than candidate blocks (box + 1 ring): the temporary set cannot overflow
    c = coords.view(-1, 3).numpy()
    xb = torch.from_numpy(rng.uniform(lo, hi, (100, 3)).astype(np.float32))
    _, ci, off, mk = bg.query(bg.transform_world_to_cell(xb))
    np.savez_compressed(
        os.path.join(HERE, "bounded.npz"), points=pts.numpy(), cell_size=bg.cell_size, blocks=c[np.lexsort(c.T[::-1])],
        x=xb.numpy(), cell_indices=ci.numpy(), offsets=off.numpy(), masks=mk.numpy(),
        cell_to_world=bg.cell_to_world(coords[:2], bg.cell_coords).numpy())
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)) // 1024, "KB")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <torch-ash root>")
    main(sys.argv[1])
