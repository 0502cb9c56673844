"""Neighbourhood convolution, ray sampler and fused RGB-D integration on the GPU against the
CPU oracle.  None of these has a test in the reference; the oracle restates its kernels."""
import numpy as np
import pytest
import torch

import bench_workloads as bw
import oracle
from oracle import tsdf as otsdf

pytestmark = pytest.mark.gpu

DEV = torch.device("cuda:0")


def _shell_grid(G, D, cls="plain", n_blocks=300, seed=0, cell_size=0.05):
    """A blobby, non-convex set of active blocks with random embeddings."""
    import ash

    blocks = bw.block_coords_blob(n_blocks, DEV, n_blobs=3, seed=seed + 40)
    if cls == "unbounded":
        grid = ash.UnBoundedSparseDenseGrid(3, 2 * n_blocks, D, G, cell_size=cell_size, device=DEV)
    else:
        grid = ash.SparseDenseGrid(3, 2 * n_blocks, D, G, device=DEV)
    grid.engine.insert_keys(blocks)
    g = torch.Generator(device=DEV).manual_seed(seed)
    with torch.no_grad():
        grid.embeddings.copy_(torch.randn(grid.embeddings.shape, generator=g, device=DEV))
    return grid, blocks


@pytest.mark.parametrize("tiled", [True, False])
@pytest.mark.parametrize("G,D,size", [(8, 4, 7), (4, 1, 3), (8, 5, 3), (2, 3, 5), (8, 16, 3), (8, 2, 5), (4, 6, 9), (3, 2, 3)])
def test_convolution_vs_oracle(G, D, size, tiled):
    """tiled: the shared-memory halo kernel SparseDenseGrid.convolution uses for float32 windows
    within one block; not tiled: the table-driven kernel behind the reference's native interface."""
    grid, _ = _shell_grid(G, D, n_blocks=120, seed=G + D)
    grid.tiled_convolution = tiled
    r = size // 2
    gen = torch.Generator(device=DEV).manual_seed(1)
    weights = torch.rand(size, size, size, D, generator=gen, device=DEV)
    out = grid.convolution(grid.embeddings.detach(), weights)
    # oracle on the very same lookup tables
    c2g, c2c = grid.construct_cell_neighbor_lut(r, bidirectional=True)
    _, g2g = grid.construct_grid_neighbor_lut((r + G - 1) // G, bidirectional=True)
    _, _, gi, ci = grid.items()
    t = lambda a: a.detach().cpu().numpy()
    ref = oracle.convolution_forward(
        t(grid.embeddings), t(weights.view(-1, D)), np.ones(gi.numel() * G**3, np.uint8), t(gi), t(ci), t(g2g),
        t(c2c), t(c2g))
    np.testing.assert_allclose(t(out), ref, rtol=1e-5, atol=1e-5)
    assert np.count_nonzero(ref) > 0


@pytest.mark.parametrize("separable", [False, True])
@pytest.mark.parametrize("G,D,size,sigma", [(8, 4, 7, 1.0), (8, 16, 3, 0.5), (4, 3, 5, 2.0), (8, 1, 9, 1.5), (2, 2, 3, 1.0)])
def test_gaussian_filter_matches_reference_weights(G, D, size, sigma, separable):
    """gaussian_filter_: kernel of ash/grid.py:449-472, normalised, applied in place -- as the full
    size^3 window and as three 1-D passes (the window is an outer product) -- against the oracle's
    size^3-tap convolution with the reference's weights, on a blobby block set whose skin blocks
    miss neighbours (absent blocks count as zero in both)."""
    grid, _ = _shell_grid(G, D, n_blocks=60, seed=3 + size)
    grid.separable_gaussian = separable
    before = grid.embeddings.detach().clone()
    w = grid._gaussian_weights(size, sigma)
    assert w.shape == (size,) * 3 and abs(float(w.sum()) - 1) < 1e-6
    assert torch.allclose(w, w.flip(0)) and torch.allclose(w, w.permute(2, 1, 0))
    grid.gaussian_filter_(size, sigma)
    r = size // 2
    c2g, c2c = grid.construct_cell_neighbor_lut(r, bidirectional=True)
    _, g2g = grid.construct_grid_neighbor_lut((r + G - 1) // G, bidirectional=True)
    _, _, gi, ci = grid.items()
    t = lambda a: a.detach().cpu().numpy()
    ref = oracle.convolution_forward(
        t(before), t(w.view(-1, 1).repeat(1, D)), np.ones(gi.numel() * G**3, np.uint8), t(gi), t(ci), t(g2g), t(c2c),
        t(c2g))
    np.testing.assert_allclose(t(grid.embeddings), ref, rtol=1e-5, atol=1e-5)
    assert np.count_nonzero(ref) > 0


def _oracle_map_like(grid):
    keys, idx = grid.engine.items()
    om = oracle.OracleHashMap(3, grid.num_embeddings)
    om.insert_keys(keys.cpu().numpy())
    return om


@pytest.mark.parametrize("G", [8, 4])
def test_ray_near_far_and_sample_vs_oracle(G):
    """Bit-exact: both sides evaluate positions as fma(t, d, o) in float32."""
    grid, blocks = _shell_grid(G, 1, cls="unbounded", n_blocks=400, seed=9, cell_size=0.02)
    om = _oracle_map_like(grid)
    n = 2000
    gen = torch.Generator(device=DEV).manual_seed(4)
    bmin, bmax = grid.get_bbox()
    centre = (bmin + bmax) / 2
    extent = bmax - bmin
    # origins mostly inside the bounding box (a march that starts outside it ends at once,
    # ash/src/sampler.cu:46-52), some outside
    o = centre + (torch.rand(n, 3, generator=gen, device=DEV) - 0.5) * extent * 1.1
    tgt = centre + (torch.rand(n, 3, generator=gen, device=DEV) - 0.5) * extent * 0.6
    d = torch.nn.functional.normalize(tgt - o, dim=-1)
    t_min, t_max = 0.0, float(extent.max()) * 2
    nears, fars = grid.ray_find_near_far(o, d, t_min, t_max, 0.01)
    cs = grid.cell_size
    o_c, bmin_c, bmax_c = (o / cs).cpu().numpy(), (bmin / cs).cpu().numpy(), (bmax / cs).cpu().numpy()
    n_ref, f_ref = oracle.ray_find_near_far(om, o_c, d.cpu().numpy(), bmin_c, bmax_c, t_min / cs, t_max / cs, 0.01 / cs, float(G))
    np.testing.assert_array_equal(nears.cpu().numpy(), (torch.from_numpy(n_ref) * cs).numpy())
    np.testing.assert_array_equal(fars.cpu().numpy(), (torch.from_numpy(f_ref) * cs).numpy())
    assert (n_ref >= 0).sum() > 50 and (n_ref < 0).sum() > 0

    hit = nears >= 0
    o2, d2 = o[hit], d[hit]
    ri, tn, tf, prefix = grid.ray_sample(o2, d2, nears[hit], fars[hit], 64)
    r_ri, r_tn, r_tf, r_prefix = oracle.ray_sample(
        om, (o2 / cs).cpu().numpy(), d2.cpu().numpy(), (nears[hit] / cs).cpu().numpy(), (fars[hit] / cs).cpu().numpy(),
        bmin_c, bmax_c, 64, float(G))
    np.testing.assert_array_equal(prefix.cpu().numpy(), r_prefix)
    np.testing.assert_array_equal(ri.cpu().numpy(), r_ri)
    np.testing.assert_array_equal(tn.cpu().numpy(), (torch.from_numpy(r_tn) * cs).numpy())
    np.testing.assert_array_equal(tf.cpu().numpy(), (torch.from_numpy(r_tf) * cs).numpy())
    assert len(r_ri) > 1000
    # rays that miss everything produce no samples; scalar near/far are accepted too
    ri0, _, _, p0 = grid.ray_sample(o[:5], d[:5], 1e9, 1e9 + 1, 8)
    assert ri0.numel() == 0 and (p0 == 0).all()


@pytest.mark.parametrize("whole_sequence,dil", [(False, 1), (True, 1), (True, 2)])
@pytest.mark.parametrize("H,W", [(120, 160)])
def test_tsdf_fusion_vs_oracle(H, W, whole_sequence, dil):
    """Three frames fused by the two CUDA launches -- frame by frame through fuse_frame, or as one
    native call for the whole sequence through fuse_dataset -- vs the numpy restatement of
    fuse_frame: same set of blocks, and per block coordinate the same sdf / rgb / weight (bit-exact
    arithmetic contract; compared with a tiny tolerance)."""
    import ash
    from ash.fusion import TSDFFusion

    G, cell, depth_max, n_emb = 8, 0.04, 5.0, 6000 * dil
    grid = ash.UnBoundedSparseDenseGrid(3, n_emb, 5, G, cell_size=cell, device=DEV)
    fusion = TSDFFusion(grid, dil)
    ref = otsdf.OracleTSDF(n_emb, G, cell, dil)
    scene = bw.Scene(DEV)
    K = bw.intrinsics(H, W)
    frames = []
    for pose in bw.camera_poses(3, seed=77):
        E = torch.linalg.inv(pose)  # world -> camera
        depth, color = scene.render(K.to(DEV), pose.float().to(DEV), H, W)
        frames.append(ash.DotDict(depth=depth.clone(), depth_scale=1.0, depth_max=depth_max, intrinsic=K, extrinsic=E,
                                  rgb=color))
        ref.fuse_frame(depth.cpu().numpy(), color.cpu().numpy(), K.numpy(), E.numpy(), np.linalg.inv(E.numpy()), depth_max)
    if whole_sequence:
        counter = torch.zeros(1, dtype=torch.int64, device=DEV)
        fusion.fuse_dataset(frames, counter=counter)
        assert int(counter.item()) > 100 and fusion._stamp == 3
    else:
        for datum in frames:
            fusion.fuse_frame(datum)
    assert grid.engine.backend.status() == 0
    import __ash

    assert __ash.tsdf_copy_timeouts(DEV) == 0      # no bounded wait of the bulk copies ran out
    keys, idx = grid.engine.items()
    rkeys, ridx = ref.map.items()
    keys_np = keys.cpu().numpy()
    order, rorder = np.lexsort(keys_np.T[::-1]), np.lexsort(rkeys.T[::-1])
    assert len(keys_np) == len(rkeys) > 100
    np.testing.assert_array_equal(keys_np[order], rkeys[rorder])
    got = grid.embeddings.detach()[idx[torch.from_numpy(order).to(DEV)]].cpu().numpy()
    want = ref.emb[ridx[rorder]]
    assert (want[..., 4] > 0).mean() > 0.02
    np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("G", [8, 4, 2])
def test_isosurface_vertices_vs_oracle_and_sphere(G):
    """Vertex-only iso-surface (ash/src/grid.cu:453-604) against the CPU restatement as a SET of
    positions (the order is the order of an atomic counter), and a known answer: crossings of a
    sphere's signed distance lie on the sphere."""
    import ash

    cell = 0.05
    grid = ash.UnBoundedSparseDenseGrid(3, 6000, 2, G, cell_size=cell, device=DEV)
    gen = torch.Generator(device=DEV).manual_seed(G)
    dirs = torch.nn.functional.normalize(torch.randn(20000, 3, generator=gen, device=DEV), dim=-1)
    grid.spatial_init_(dirs * 0.8, dilation=1, bidirectional=True)
    gc, cc, gi, ci = grid.items()
    pos = grid.cell_to_world(gc, cc).view(gi.shape[0], -1, 3)
    sdf = torch.zeros(6000, G**3, device=DEV)
    w = torch.zeros(6000, G**3, device=DEV)
    sdf[gi.view(-1)] = pos.norm(dim=-1) - 0.8
    w[gi.view(-1)] = (torch.rand(pos.shape[:2], generator=gen, device=DEV) > 0.1).float() * 2  # some cells unobserved
    out = grid.marching_cubes(sdf, w, vertices_only=True, weight_thr=1.0)
    verts = out["positions"]
    assert verts.shape[0] > 500 and verts.shape[1] == 3
    # a linear interpolation of the distance along an edge of length `cell` is within cell^2 / r of the sphere
    assert ((verts.norm(dim=-1) - 0.8).abs() < cell * cell).all()
    t = lambda a: a.detach().cpu().numpy()
    _, idx = grid.engine.items()
    ref = oracle.isosurface_extraction(
        t(sdf), t(w), t(idx), t(grid.grid_coords), t(grid.lut_grid_nb2grid_idx), t(grid.cell_coords),
        t(grid.lut_cell_nb2cell_idx), t(grid.lut_cell_nb2grid_nb), G, 0.0, 1.0)
    got = t(verts / cell) if False else t(grid.transform_world_to_cell(verts))
    assert len(ref) == len(got)
    order_r, order_g = np.lexsort(np.round(ref, 3).T[::-1]), np.lexsort(np.round(got, 3).T[::-1])
    np.testing.assert_allclose(got[order_g], ref[order_r], rtol=0, atol=2e-3)
    assert grid.marching_cubes(sdf + 10.0, w, vertices_only=True) is None
