"""Host logic of the fuser's pruning (erase + marching cubes + connected components) on the CPU
stand-in, and the connected-components labelling against scipy."""
import numpy as np
import pytest
import torch

import prune_scenario


def test_connected_triangle_components_match_scipy():
    import scipy.sparse as sp
    from scipy.sparse.csgraph import connected_components

    from ash.mesh import connected_triangle_components

    rng = np.random.default_rng(3)
    n_vertices = 3000
    # a soup of strips: triangles between nearby vertex ids, so that components of many sizes appear
    a = rng.integers(0, n_vertices - 3, 2500)
    tris = np.stack([a, a + rng.integers(1, 3, len(a)), a + rng.integers(1, 4, len(a))], 1)
    tris = tris[(tris[:, 0] != tris[:, 1]) & (tris[:, 1] != tris[:, 2]) & (tris[:, 0] != tris[:, 2])]
    comp, sizes = connected_triangle_components(torch.from_numpy(tris), n_vertices)
    rows = np.concatenate([tris[:, 0], tris[:, 1]])
    cols = np.concatenate([tris[:, 1], tris[:, 2]])
    graph = sp.coo_matrix((np.ones(len(rows)), (rows, cols)), shape=(n_vertices, n_vertices))
    _, want = connected_components(graph, directed=False)
    want_tri = want[tris[:, 0]]
    comp = comp.numpy()
    # same partition of the triangles, whatever the numbering
    pairs = set(zip(comp.tolist(), want_tri.tolist()))
    assert len(pairs) == len(set(comp.tolist())) == len(set(want_tri.tolist()))
    assert sorted(sizes.tolist()) == sorted(np.bincount(np.unique(want_tri, return_inverse=True)[1]).tolist())
    e, s = connected_triangle_components(torch.zeros((0, 3), dtype=torch.int32), 10)
    assert e.numel() == 0 and s.numel() == 0


@pytest.mark.skipif(torch.cuda.is_available(), reason="runs on the CPU stand-in only")
def test_prune_by_mesh_connected_components_on_the_stand_in():
    import ash

    prune_scenario.check_mesh_pruning(ash, torch.device("cpu"))


@pytest.mark.skipif(torch.cuda.is_available(), reason="runs on the CPU stand-in only")
def test_prune_by_weight_on_the_stand_in():
    import ash

    prune_scenario.check_weight_pruning(ash, torch.device("cpu"))
