"""Checks a triangle mesh must pass whatever table produced it (shared by the CPU and GPU tests)."""
import numpy as np


def closed_and_consistently_oriented(triangles):
    """Every edge is shared by exactly two triangles that traverse it in opposite directions.
    Returns the number of undirected edges."""
    t = np.asarray(triangles, dtype=np.int64)
    directed = np.concatenate([t[:, [0, 1]], t[:, [1, 2]], t[:, [2, 0]]])
    assert (directed[:, 0] != directed[:, 1]).all(), "degenerate triangle"
    n = int(t.max()) + 1
    key = directed[:, 0] * n + directed[:, 1]
    assert len(np.unique(key)) == len(key), "an edge is traversed twice in the same direction"
    opposite = directed[:, 1] * n + directed[:, 0]
    assert np.isin(opposite, key).all(), "an edge has no opposite partner: the mesh has a crack"
    return len(key) // 2


def signed_volume(vertices, triangles):
    v = np.asarray(vertices, dtype=np.float64)
    t = np.asarray(triangles, dtype=np.int64)
    a, b, c = v[t[:, 0]], v[t[:, 1]], v[t[:, 2]]
    return float(np.einsum("ij,ij->i", a, np.cross(b, c)).sum() / 6.0)


def canonical_triangle_rows(vertices, triangles):
    """Triangles as rows of 9 coordinates, each rotated (orientation kept) so that its
    lexicographically smallest corner comes first, rows sorted: equal for two meshes that differ
    only in vertex numbering, corner rotation and triangle order."""
    v = np.asarray(vertices)
    t = np.asarray(triangles, dtype=np.int64)
    p = v[t]                                              # (T, 3, 3)
    first = np.lexsort((p[:, :, 2], p[:, :, 1], p[:, :, 0]), axis=1)[:, 0]
    rows = np.stack([p[np.arange(len(t)), (first + k) % 3] for k in range(3)], 1).reshape(len(t), 9)
    return rows[np.lexsort(rows.T[::-1])]
