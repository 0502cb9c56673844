"""Oracle check on CPU: the iso-surface vertices of a plane's signed distance are the plane."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.skipif(torch.cuda.is_available(), reason="runs on the CPU stand-in only")


def test_plane_crossings_through_the_python_layer():
    import ash

    G, cell = 4, 0.1
    grid = ash.UnBoundedSparseDenseGrid(3, 200, 1, G, cell_size=cell, device=torch.device("cpu"))
    r = torch.arange(-2, 2)
    pts = torch.stack(torch.meshgrid(r, r, r, indexing="ij"), -1).view(-1, 3).float() * (G * cell) + 0.01
    grid.spatial_init_(pts, dilation=0)
    gc, cc, gi, ci = grid.items()
    pos = grid.cell_to_world(gc, cc).view(gi.shape[0], -1, 3)
    sdf = torch.zeros(200, G**3)
    w = torch.zeros(200, G**3)
    sdf[gi.view(-1)] = pos[..., 2] - 0.123            # plane z = 0.123
    w[gi.view(-1)] = 1.0
    out = grid.marching_cubes(sdf, w, vertices_only=True, weight_thr=1.0)
    v = out["positions"].numpy()
    # one crossing per (x, y) column of the 16 x 16 cells, all on the plane -- except the columns on
    # the +x / +y faces of the active region: their +x / +y neighbour BLOCK is missing, which ends the
    # cell's loop before the z axis is looked at (ash/src/grid.cu:508-510)
    assert v.shape == (15 * 15, 3)
    np.testing.assert_allclose(v[:, 2], 0.123, atol=1e-6)
    assert len({(round(a, 4), round(b, 4)) for a, b in v[:, :2]}) == 15 * 15


def test_plane_triangles_through_the_python_layer(tmp_path):
    """Marching cubes of a plane's signed distance on the CPU stand-in: two triangles per cube,
    all on the plane, normals towards increasing distance, total area = the observed square; and
    the PLY file of the mesh reads back unchanged."""
    import os

    import ash
    from ash.mesh import read_ply, write_ply

    G, cell = 4, 0.1
    grid = ash.UnBoundedSparseDenseGrid(3, 200, 1, G, cell_size=cell, device=torch.device("cpu"))
    r = torch.arange(-2, 2)
    pts = torch.stack(torch.meshgrid(r, r, r, indexing="ij"), -1).view(-1, 3).float() * (G * cell) + 0.01
    grid.spatial_init_(pts, dilation=0)
    gc, cc, gi, ci = grid.items()
    pos = grid.cell_to_world(gc, cc).view(gi.shape[0], -1, 3)
    sdf = torch.zeros(200, G**3)
    sdf[gi.view(-1)] = pos[..., 2] - 0.123
    out = grid.marching_cubes(sdf, torch.ones_like(sdf), vertices_only=False, weight_thr=1.0)
    v, t = out["positions"].numpy(), out["triangles"].numpy()
    assert t.shape == (2 * 15 * 15, 3) and v.shape == (16 * 16, 3)
    np.testing.assert_allclose(v[:, 2], 0.123, atol=1e-6)
    tri = v[t]
    normal = np.cross(tri[:, 1] - tri[:, 0], tri[:, 2] - tri[:, 0])
    assert (normal[:, 2] > 0).all()
    assert abs(0.5 * np.linalg.norm(normal, axis=1).sum() - (15 * cell) ** 2) < 1e-4
    path = os.path.join(tmp_path, "plane.ply")
    write_ply(path, out)
    back = read_ply(path)
    np.testing.assert_array_equal(back["positions"], v)
    np.testing.assert_array_equal(back["triangles"], t)


def test_oracle_mesh_of_a_sphere_is_closed_and_oriented():
    import ash
    import mesh_checks

    G, cell, r = 4, 0.05, 0.4
    grid = ash.UnBoundedSparseDenseGrid(3, 3000, 1, G, cell_size=cell, device=torch.device("cpu"))
    gen = torch.Generator().manual_seed(2)
    dirs = torch.nn.functional.normalize(torch.randn(20000, 3, generator=gen), dim=-1)
    grid.spatial_init_(dirs * r, dilation=1, bidirectional=True)
    gc, cc, gi, ci = grid.items()
    pos = grid.cell_to_world(gc, cc).view(gi.shape[0], -1, 3)
    sdf = torch.zeros(3000, G**3)
    sdf[gi.view(-1)] = pos.norm(dim=-1) - r
    out = grid.marching_cubes(sdf, torch.ones_like(sdf), vertices_only=False)
    v, t = out["positions"].numpy(), out["triangles"].numpy()
    edges = mesh_checks.closed_and_consistently_oriented(t)
    assert len(v) - edges + len(t) == 2
    vol = mesh_checks.signed_volume(v, t)
    assert abs(vol - 4 / 3 * np.pi * r**3) / (4 / 3 * np.pi * r**3) < 0.02
