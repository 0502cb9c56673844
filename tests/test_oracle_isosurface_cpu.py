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
