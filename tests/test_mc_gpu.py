"""Triangle extraction (marching cubes, ash/src/grid.cu:607-946) on the GPU: against the CPU
oracle as a set of triangles, and against what any correct mesh of a closed surface must satisfy."""
import os

import numpy as np
import pytest
import torch

import mesh_checks
import oracle

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _np(t):
    return t.detach().cpu().numpy()


def _tables(grid):
    _, idx = grid.engine.items()
    return (idx, grid.grid_coords, grid.lut_grid_nb2grid_idx, grid.cell_coords, grid.lut_cell_nb2cell_idx,
            grid.lut_cell_nb2grid_nb)


def _compare_with_oracle(grid, sdf, w, iso, thr):
    import __ash

    tables = _tables(grid)
    tris, verts = __ash.marching_cubes(sdf, w, *tables, grid.grid_dim, iso, thr)
    rtris, rverts = oracle.marching_cubes(_np(sdf), _np(w), *[_np(t) for t in tables], grid.grid_dim, iso, thr)
    assert tris.dtype == torch.int32 and verts.dtype == torch.float32
    assert verts.shape == rverts.shape and tris.shape == rtris.shape
    if len(rverts):
        got = _np(verts)
        np.testing.assert_array_equal(got[np.lexsort(got.T[::-1])], rverts[np.lexsort(rverts.T[::-1])])
        np.testing.assert_array_equal(mesh_checks.canonical_triangle_rows(got, _np(tris)),
                                      mesh_checks.canonical_triangle_rows(rverts, rtris))
    return _np(tris), _np(verts)


@pytest.mark.parametrize("G", [8, 4, 2])
def test_triangles_vs_oracle_on_a_partly_observed_sphere(G):
    import ash

    cell = 0.05
    grid = ash.UnBoundedSparseDenseGrid(3, 6000, 2, G, cell_size=cell, device=DEV)
    gen = torch.Generator(device=DEV).manual_seed(G)
    dirs = torch.nn.functional.normalize(torch.randn(20000, 3, generator=gen, device=DEV), dim=-1)
    grid.spatial_init_(dirs * 0.8, dilation=1, bidirectional=True)
    grid.construct_grid_neighbor_lut_(1, False)
    gc, cc, gi, ci = grid.items()
    pos = grid.cell_to_world(gc, cc).view(gi.shape[0], -1, 3)
    sdf = torch.zeros(6000, G**3, device=DEV)
    w = torch.zeros(6000, G**3, device=DEV)
    sdf[gi.view(-1)] = pos.norm(dim=-1) - 0.8
    w[gi.view(-1)] = (torch.rand(pos.shape[:2], generator=gen, device=DEV) > 0.05).float() * 2  # some cells unobserved
    tris, verts = _compare_with_oracle(grid, sdf, w, 0.0, 1.0)
    assert len(tris) > 500
    world = verts * cell
    assert (np.abs(np.linalg.norm(world, axis=1) - 0.8) < cell * cell).all()
    assert mesh_checks.signed_volume(world, tris) > 0          # normals towards increasing sdf


def test_fully_observed_sphere_is_watertight():
    import ash

    G, cell, r = 8, 0.04, 0.62
    grid = ash.UnBoundedSparseDenseGrid(3, 8000, 1, G, cell_size=cell, device=DEV)
    gen = torch.Generator(device=DEV).manual_seed(3)
    dirs = torch.nn.functional.normalize(torch.randn(40000, 3, generator=gen, device=DEV), dim=-1)
    grid.spatial_init_(dirs * r + 0.013, dilation=1, bidirectional=True)
    gc, cc, gi, ci = grid.items()
    pos = grid.cell_to_world(gc, cc).view(gi.shape[0], -1, 3)
    sdf = torch.zeros(8000, G**3, device=DEV)
    sdf[gi.view(-1)] = (pos - 0.013).norm(dim=-1) - r
    w = torch.ones_like(sdf)
    out = grid.marching_cubes(sdf, w, vertices_only=False, weight_thr=1.0)
    tris, verts = _np(out["triangles"]), _np(out["positions"])
    edges = mesh_checks.closed_and_consistently_oriented(tris)
    assert len(verts) - edges + len(tris) == 2                 # a sphere
    vol = mesh_checks.signed_volume(verts, tris)
    assert abs(vol - 4 / 3 * np.pi * r**3) / (4 / 3 * np.pi * r**3) < 0.01
    assert grid.marching_cubes(sdf + 10.0, w, vertices_only=False) is None


def test_noisy_field_full_of_ambiguous_cubes_vs_oracle_and_closed():
    import ash

    G, S = 4, 6
    grid = ash.BoundedSparseDenseGrid(3, S**3, 1, grid_dim=G, sparse_grid_dim=S, device=DEV)
    grid.dense_init_()
    grid.construct_grid_neighbor_lut_(1, False)
    gc, cc, gi, ci = grid.items()
    cells = (gc.view(-1, 1, 3) * G + cc.view(1, -1, 3)).float()          # (n, G^3, 3) integer cell positions
    gen = torch.Generator(device=DEV).manual_seed(11)
    field = torch.randn(cells.shape[:2], generator=gen, device=DEV)
    n = S * G
    # outside on the border of the observed region: every surface closes inside it (the cubes of the
    # last layer of cells have no +neighbour block and are not meshed, as in the reference)
    border = ((cells < 1) | (cells > n - 3)).any(dim=-1)
    field[border] = 1.0
    sdf = torch.zeros(S**3, G**3, device=DEV)
    sdf[gi.view(-1)] = field
    w = torch.ones_like(sdf)
    tris, verts = _compare_with_oracle(grid, sdf, w, 0.0, 1.0)
    assert len(tris) > 5000
    mesh_checks.closed_and_consistently_oriented(tris)
    assert mesh_checks.signed_volume(verts, tris) > 0


def test_ply_round_trip(tmp_path):
    import ash
    from ash.mesh import read_ply, write_ply

    G, cell = 4, 0.1
    grid = ash.UnBoundedSparseDenseGrid(3, 300, 1, G, cell_size=cell, device=DEV)
    r = torch.arange(-2, 2, device=DEV)
    pts = torch.stack(torch.meshgrid(r, r, r, indexing="ij"), -1).view(-1, 3).float() * (G * cell) + 0.01
    grid.spatial_init_(pts, dilation=0)
    gc, cc, gi, ci = grid.items()
    pos = grid.cell_to_world(gc, cc).view(gi.shape[0], -1, 3)
    sdf = torch.zeros(300, G**3, device=DEV)
    sdf[gi.view(-1)] = pos[..., 2] - 0.123
    out = grid.marching_cubes(sdf, torch.ones_like(sdf), vertices_only=False,
                              color_fn=lambda p: (p * 0.5 + 0.5).clamp(0, 1),
                              normal_fn=lambda p: torch.tensor([0.0, 0.0, 1.0], device=p.device).expand_as(p))
    path = os.path.join(tmp_path, "plane.ply")
    write_ply(path, out)
    back = read_ply(path)
    np.testing.assert_array_equal(back["positions"], _np(out["positions"]))
    np.testing.assert_array_equal(back["triangles"], _np(out["triangles"]))
    np.testing.assert_allclose(back["colors"], _np(out["colors"]), atol=0.5 / 255 + 1e-6)
    np.testing.assert_array_equal(back["normals"], _np(out["normals"]))
    # the plane z = 0.123 over 15 x 15 cubes: two triangles per cube, area of the square
    tri = _np(out["positions"])[_np(out["triangles"])]
    area = 0.5 * np.linalg.norm(np.cross(tri[:, 1] - tri[:, 0], tri[:, 2] - tri[:, 0]), axis=1).sum()
    assert len(tri) == 2 * 15 * 15 and abs(area - (15 * cell) ** 2) < 1e-4
    assert (np.cross(tri[:, 1] - tri[:, 0], tri[:, 2] - tri[:, 0])[:, 2] > 0).all()   # normals along +z


def test_fuser_pruning_on_the_gpu():
    import ash
    import prune_scenario

    prune_scenario.check_mesh_pruning(ash, DEV)
    prune_scenario.check_weight_pruning(ash, DEV)
