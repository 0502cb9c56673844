"""The generated marching-cubes table (oracle/gen_mc_tables.py) is derived, not
transcribed, so it is validated by what a triangulation table must guarantee: on closed surfaces
every mesh edge is shared by exactly two triangles that traverse it in opposite directions (no
cracks, consistent orientation), the Euler characteristic is that of the surface, normals point
to the outside (positive enclosed volume), and the committed header is what the generator emits."""
import importlib.util
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_spec = importlib.util.spec_from_file_location("gen_mc_tables", os.path.join(ROOT, "oracle", "gen_mc_tables.py"))
gen = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(gen)
TRIS, MASKS = gen.build()


def mesh_of(field, iso=0.0):
    """Marching cubes over a dense lattice with the generated table (pure Python, small grids).
    Vertices are keyed by (owner cell, direction) and placed by linear interpolation."""
    n = field.shape[0] - 1
    inside = (field - iso) < 0
    vid, verts, tris = {}, [], []
    for x in range(n):
        for y in range(n):
            for z in range(n):
                code = 0
                for c in range(8):
                    ox, oy, oz = gen.corner_offset(c)
                    code |= int(inside[x + ox, y + oy, z + oz]) << c
                row = TRIS[code]
                for t in range(0, len(row), 3):
                    tri = []
                    for e in row[t:t + 3]:
                        a, _ = gen.edge_corners(e)
                        d = e // 4
                        o = gen.corner_offset(a)
                        key = (x + o[0], y + o[1], z + o[2], d)
                        if key not in vid:
                            p = np.array(key[:3], float)
                            q = p.copy()
                            q[d] += 1
                            f0 = field[tuple(p.astype(int))] - iso
                            f1 = field[tuple(q.astype(int))] - iso
                            assert (f0 < 0) != (f1 < 0), "table refers to an edge the surface does not cut"
                            vid[key] = len(verts)
                            verts.append(p + (f0 / (f0 - f1)) * (q - p))
                        tri.append(vid[key])
                    tris.append(tri)
    return np.array(verts), np.array(tris)


def check_closed_oriented(tris):
    directed = {}
    for a, b, c in tris:
        for u, v in ((a, b), (b, c), (c, a)):
            assert u != v
            assert (u, v) not in directed, "an edge is traversed twice in the same direction"
            directed[(u, v)] = 1
    for (u, v) in directed:
        assert (v, u) in directed, "an edge has no opposite partner: the mesh has a crack"
    return len(directed) // 2


def lattice(n):
    g = np.arange(n + 1, dtype=float)
    return np.stack(np.meshgrid(g, g, g, indexing="ij"), -1)


def signed_volume(verts, tris):
    a, b, c = verts[tris[:, 0]], verts[tris[:, 1]], verts[tris[:, 2]]
    return float(np.einsum("ij,ij->i", a, np.cross(b, c)).sum() / 6.0)


def test_committed_header_is_the_generators_output():
    for folder in (os.path.join(ROOT, "torch-ash_b200", "csrc"), os.path.join(ROOT, "oracle")):
        with open(os.path.join(folder, "mc_tables.h")) as f:
            assert f.read() == gen.render(TRIS, MASKS)


def test_every_pattern_uses_exactly_its_cut_edges_and_complements_mirror():
    for code in range(256):
        cut = 0
        for e in range(12):
            a, b = gen.edge_corners(e)
            if ((code >> a) & 1) != ((code >> b) & 1):
                cut |= 1 << e
        assert MASKS[code] == cut
        used = 0
        for e in TRIS[code]:
            used |= 1 << e
        assert used == cut
        assert len(TRIS[code]) <= 15
    assert TRIS[0] == [] and TRIS[255] == []


def test_sphere_is_closed_oriented_genus_zero_with_the_right_volume():
    n, r = 14, 4.3
    p = lattice(n)
    field = np.linalg.norm(p - np.array([7.1, 6.8, 7.3]), axis=-1) - r
    verts, tris = mesh_of(field)
    edges = check_closed_oriented(tris)
    assert len(verts) - edges + len(tris) == 2
    vol = signed_volume(verts, tris)
    assert vol > 0 and abs(vol - 4 / 3 * np.pi * r**3) / (4 / 3 * np.pi * r**3) < 0.05


def test_torus_has_euler_characteristic_zero():
    n = 18
    p = lattice(n) - np.array([9.2, 8.9, 9.1])
    ring = np.sqrt(p[..., 0] ** 2 + p[..., 1] ** 2) - 5.2
    field = np.sqrt(ring**2 + p[..., 2] ** 2) - 2.1
    verts, tris = mesh_of(field)
    edges = check_closed_oriented(tris)
    assert len(verts) - edges + len(tris) == 0
    assert signed_volume(verts, tris) > 0


def test_random_fields_full_of_ambiguous_faces_have_no_cracks():
    rng = np.random.default_rng(15213)
    seen_codes = set()
    for trial in range(6):
        n = 9
        field = rng.standard_normal((n + 1,) * 3)
        field[0], field[-1] = 1.0, 1.0          # outside on the whole boundary: closed surfaces only
        field[:, 0], field[:, -1] = 1.0, 1.0
        field[:, :, 0], field[:, :, -1] = 1.0, 1.0
        verts, tris = mesh_of(field)
        check_closed_oriented(tris)
        assert signed_volume(verts, tris) > 0
        inside = field < 0
        for x in range(n):
            for y in range(n):
                for z in range(n):
                    code = 0
                    for c in range(8):
                        o = gen.corner_offset(c)
                        code |= int(inside[x + o[0], y + o[1], z + o[2]]) << c
                    seen_codes.add(code)
    assert len(seen_codes) == 256  # every pattern was exercised
