"""Generates ``mc_tables.h``: the per-cube triangulation table of the iso-surface mesher.

    python oracle/gen_mc_tables.py     # rewrites mc_tables.h next to this file and beside the CUDA kernels

The table is DERIVED here, not transcribed from anywhere: for each of the 256 inside/outside
patterns of a cube's corners the iso-surface is traced on the cube's faces and the resulting closed
loops are triangulated without diagonals that lie in a cube face.

Conventions (shared by the CUDA kernels and the CPU oracle through the generated header):
  corner c in [0, 8)   offset (c & 1, (c >> 1) & 1, (c >> 2) & 1)  -- the query's corner order
  bit c of a code      corner c is INSIDE (value - iso < 0)
  edge e in [0, 12)    axis d = e // 4, parallel to it; j = e % 4 places it: bit 0 of j is the
                       offset along axis (d + 1) % 3, bit 1 along axis (d + 2) % 3.  Its lower
                       corner is the cell that owns the edge's vertex (direction d).
  face rule            on a face whose corners alternate inside / outside the surface cuts off
                       each INSIDE corner on its own.  The rule reads only the face's own four
                       signs, so the two cubes sharing a face agree and the mesh has no cracks.
  orientation          triangle normals (right-hand rule) point to the OUTSIDE (increasing value):
                       the winding of the reference's OUTPUT -- its table (ash/src/mc_macros.h) holds
                       the mirrored winding and its kernel writes every triangle in reverse vertex
                       order (ash/src/grid.cu:836).
"""
import os

HERE = os.path.dirname(os.path.abspath(__file__))


def corner_offset(c):
    return (c & 1, (c >> 1) & 1, (c >> 2) & 1)


def edge_corners(e):
    d, j = divmod(e, 4)
    u, v = (d + 1) % 3, (d + 2) % 3
    a = ((j & 1) << u) | ((j >> 1) << v)
    return a, a | (1 << d)


EDGE_OF = {}
for _e in range(12):
    _a, _b = edge_corners(_e)
    EDGE_OF[(_a, _b)] = EDGE_OF[(_b, _a)] = _e


def face_cycles():
    """The four corners of each of the 6 faces in cyclic order."""
    out = []
    for n in range(3):
        u, v = (n + 1) % 3, (n + 2) % 3
        for side in (0, 1):
            base = side << n
            out.append([base, base | (1 << u), base | (1 << u) | (1 << v), base | (1 << v)])
    return out


FACES = face_cycles()


def midpoint(e):
    a, b = edge_corners(e)
    pa, pb = corner_offset(a), corner_offset(b)
    return tuple((x + y) / 2.0 for x, y in zip(pa, pb))


def cross(a, b):
    return (a[1] * b[2] - a[2] * b[1], a[2] * b[0] - a[0] * b[2], a[0] * b[1] - a[1] * b[0])


def loops_of(code):
    inside = [(code >> c) & 1 for c in range(8)]
    link = {}  # crossing edge -> the (two) crossing edges it is joined to across the faces

    def join(e0, e1):
        link.setdefault(e0, []).append(e1)
        link.setdefault(e1, []).append(e0)

    for cyc in FACES:
        cuts = [i for i in range(4) if inside[cyc[i]] != inside[cyc[(i + 1) % 4]]]  # edge i: corner i -> i+1
        edges = [EDGE_OF[(cyc[i], cyc[(i + 1) % 4])] for i in range(4)]
        if len(cuts) == 2:
            join(edges[cuts[0]], edges[cuts[1]])
        elif len(cuts) == 4:
            for i in range(4):  # cut off every inside corner: join the two face edges that meet at it
                if inside[cyc[i]]:
                    join(edges[i], edges[(i - 1) % 4])
    assert all(len(v) == 2 for v in link.values()), code
    loops, seen = [], set()
    for start in sorted(link):
        if start in seen:
            continue
        loop, prev, cur = [start], None, start
        while True:
            first, second = link[cur]  # two distinct edges: cube edges share at most one face
            nxt = second if first == prev else first
            if nxt == start:
                break
            assert nxt not in seen, code
            loop.append(nxt)
            seen.add(nxt)
            prev, cur = cur, nxt
        seen.add(start)
        loops.append(loop)
    # Orientation from the loop's first segment, which lies in a cube face with outward normal N:
    # with t the segment, q the inside corner at its start edge and m0 the segment's start, the
    # bounded patch lies to the left of t (seen against the surface normal, which points away
    # from the inside) exactly when ((q - m0) x t) . N > 0.
    oriented = []
    for loop in loops:
        e0, e1 = loop[0], loop[1]
        (face,) = [f for f, cyc in enumerate(FACES) if set(edge_corners(e0)) <= set(cyc) and set(edge_corners(e1)) <= set(cyc)]
        axis, side = divmod(face, 2)
        normal = [0.0, 0.0, 0.0]
        normal[axis] = 1.0 if side else -1.0
        m0, m1 = midpoint(e0), midpoint(e1)
        a, b = edge_corners(e0)
        q = corner_offset(a if inside[a] else b)
        w = [q[k] - m0[k] for k in range(3)]
        t = [m1[k] - m0[k] for k in range(3)]
        c = cross(w, t)
        if sum(c[k] * normal[k] for k in range(3)) < 0:
            loop = [loop[0]] + loop[:0:-1]
        oriented.append(loop)
    return oriented


def share_face(e0, e1):
    c = set(edge_corners(e0)) | set(edge_corners(e1))
    return any(c <= set(cyc) for cyc in FACES)


def triangulations(idx):
    """All triangulations of the polygon with vertex positions ``idx`` (a list), as lists of
    index triples in the polygon's orientation."""
    if len(idx) < 3:
        return [[]]
    out = []
    a, b = idx[0], idx[-1]
    for k in range(1, len(idx) - 1):
        for left in triangulations(idx[:k + 1]):
            for right in triangulations(idx[k:]):
                out.append(left + [(a, idx[k], b)] + right)
    return out


def triangulate(loop):
    """Triangles of a loop such that no interior diagonal joins two vertices of one cube face: such
    a diagonal lies IN the face, where the neighbouring cube may place the same diagonal, and the
    two surfaces would touch along it (an edge with four triangles)."""
    n = len(loop)
    for cand in triangulations(list(range(n))):
        ok = True
        for tri in cand:
            for u, v in ((tri[0], tri[1]), (tri[1], tri[2]), (tri[2], tri[0])):
                consecutive = (u - v) % n in (1, n - 1)
                if not consecutive and share_face(loop[u], loop[v]):
                    ok = False
        if ok:
            return [[loop[i] for i in tri] for tri in cand]
    raise AssertionError(f"no admissible triangulation for loop {loop}")


def build():
    tris, masks = [], []
    for code in range(256):
        row = []
        mask = 0
        for loop in loops_of(code):
            for e in loop:
                mask |= 1 << e
            for tri in triangulate(loop):
                row += tri
        tris.append(row)
        masks.append(mask)
    return tris, masks


def render(tris, masks):
    width = max(len(r) for r in tris)
    lines = [
        "// GENERATED by gen_mc_tables.py -- do not edit.  Conventions are documented there.",
        "#pragma once",
        "#include <stdint.h>",
        "",
        "// storage class of the tables: the CUDA side defines this as `static __device__ const`",
        "#ifndef ASHB_MC_TABLE",
        "#define ASHB_MC_TABLE static const",
        "#endif",
        "",
        f"#define ASHB_MC_MAX_TRIS {width // 3}",
        "",
        "// number of triangles of each corner pattern",
        "ASHB_MC_TABLE uint8_t kMcTriCount[256] = {",
    ]
    counts = [len(r) // 3 for r in tris]
    for i in range(0, 256, 32):
        lines.append("    " + ", ".join(str(c) for c in counts[i:i + 32]) + ",")
    lines += ["};", "", "// edges cut by the surface, one bit per edge", "ASHB_MC_TABLE uint16_t kMcEdgeMask[256] = {"]
    for i in range(0, 256, 16):
        lines.append("    " + ", ".join(f"0x{m:03x}" for m in masks[i:i + 16]) + ",")
    lines += ["};", "", "// edge ids of the triangles' vertices, 3 per triangle, padded with -1",
              f"ASHB_MC_TABLE int8_t kMcTris[256][{width}] = {{"]
    for r in tris:
        lines.append("    {" + ", ".join(f"{v:2d}" for v in r + [-1] * (width - len(r))) + "},")
    lines += ["};", ""]
    return "\n".join(lines)


if __name__ == "__main__":
    t, m = build()
    # one copy beside the CPU oracle (which builds on its own), one beside the CUDA kernels
    for folder in (HERE, os.path.join(HERE, "..", "torch-ash_b200", "csrc")):
        with open(os.path.join(folder, "mc_tables.h"), "w") as f:
            f.write(render(t, m))
    print("max triangles per cube:", max(len(r) for r in t) // 3, "total:", sum(len(r) for r in t) // 3)
