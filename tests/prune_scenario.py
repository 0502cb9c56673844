"""Scenario shared by the CPU and GPU tests of the fuser's pruning methods: a fused volume that
holds a large sphere and, apart from it, a small one."""
import numpy as np
import torch

C2 = (1.2, 0.0, 0.0)
R_BIG, R_SMALL = 0.5, 0.12


def build(ash, device):
    G, cell = 4, 0.05
    grid = ash.UnBoundedSparseDenseGrid(3, 4000, 5, G, cell_size=cell, device=device)
    gen = torch.Generator().manual_seed(5)
    dirs = torch.nn.functional.normalize(torch.randn(30000, 3, generator=gen), dim=-1)
    c2 = torch.tensor(C2)
    pts = torch.cat([dirs * R_BIG, dirs[:4000] * R_SMALL + c2]).to(device)
    grid.spatial_init_(pts, dilation=1, bidirectional=True)
    gc, cc, gi, ci = grid.items()
    pos = grid.cell_to_world(gc, cc).view(gi.shape[0], -1, 3)
    sdf = torch.minimum(pos.norm(dim=-1) - R_BIG, (pos - c2.to(device)).norm(dim=-1) - R_SMALL)
    with torch.no_grad():
        grid.embeddings[gi.view(-1), :, 0] = sdf
        grid.embeddings[gi.view(-1), :, 4] = 2.0
    return grid


def block_centres(grid):
    coords = grid.items()[0].view(-1, 3).float()
    return (coords + 0.5) * grid.grid_dim * grid.cell_size


def check_mesh_pruning(ash, device):
    from ash.fusion import TSDFFusion

    grid = build(ash, device)
    fuser = TSDFFusion(grid, dilation=1)
    c2 = torch.tensor(C2, device=device)
    before = block_centres(grid)
    n_small_before = int(((before - c2).norm(dim=-1) < 0.45).sum())
    assert n_small_before > 10
    erased = fuser.prune_by_mesh_connected_components_(ratio_to_largest_component=0.5)
    after = block_centres(grid)
    assert erased > 0 and len(after) == len(before) - erased == grid.engine.size()
    assert int(((after - c2).norm(dim=-1) < 0.45).sum()) == 0            # the small sphere is gone
    # every block the large surface passes through is still there
    mesh = grid.marching_cubes(grid.embeddings[..., 0].contiguous(), grid.embeddings[..., 4].contiguous(),
                               vertices_only=False)
    radii = mesh["positions"].norm(dim=-1)
    assert mesh["positions"].shape[0] > 1000 and float((radii - R_BIG).abs().max()) < 0.01
    area = 4 * np.pi * R_BIG**2
    tri = mesh["positions"][mesh["triangles"].long()]
    got = 0.5 * torch.linalg.cross(tri[:, 1] - tri[:, 0], tri[:, 2] - tri[:, 0]).norm(dim=-1).sum()
    assert abs(float(got) - area) / area < 0.02                          # the whole large sphere is meshed


def check_weight_pruning(ash, device):
    from ash.fusion import TSDFFusion

    grid = build(ash, device)
    fuser = TSDFFusion(grid, dilation=1)
    gc, _, gi, _ = grid.items()   # one enumeration: its order may differ from call to call
    far = ((gc.view(-1, 3).float() + 0.5) * grid.grid_dim * grid.cell_size)[:, 0] > 0.9
    with torch.no_grad():
        grid.embeddings[gi.view(-1)[far], :, 4] = 0.2
    n = fuser.prune_by_weight_(grid_mean_weight_thr=1)
    assert n == int(far.sum()) > 0 and grid.engine.size() == len(far) - n
    assert bool((block_centres(grid)[:, 0] <= 0.9).all())
    assert float(grid.embeddings.detach()[gi.view(-1)[far]].abs().max()) == 0.0
