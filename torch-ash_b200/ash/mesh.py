"""Writing extracted surfaces to disk without a viewer or a geometry package.

The reference hands the arrays of ``SparseDenseGrid.marching_cubes`` to Open3D geometry objects
(ash/grid.py:675-712) and its demos save or display those; here the dict that ``marching_cubes``
returns is stored as a binary little-endian PLY file, which any mesh tool reads.
"""
from typing import Dict

import numpy as np
import torch


def _array(t, dtype, cols):
    a = t.detach().cpu().numpy() if isinstance(t, torch.Tensor) else np.asarray(t)
    a = np.ascontiguousarray(a, dtype=dtype)
    if a.ndim != 2 or a.shape[1] != cols:
        raise ValueError(f"expected an (n, {cols}) array, got {a.shape}")
    return a


def write_ply(path: str, surface: Dict[str, torch.Tensor]) -> None:
    """Store ``surface`` -- ``positions`` (V, 3), optional ``triangles`` (T, 3), ``colors``
    (V, 3) in [0, 1] and ``normals`` (V, 3) -- as binary PLY (a point cloud when there are no
    triangles)."""
    pos = _array(surface["positions"], np.float32, 3)
    fields = [("x", "<f4"), ("y", "<f4"), ("z", "<f4")]
    columns = [pos[:, 0], pos[:, 1], pos[:, 2]]
    if surface.get("normals") is not None:
        nrm = _array(surface["normals"], np.float32, 3)
        if len(nrm) != len(pos):
            raise ValueError("normals and positions differ in length")
        fields += [("nx", "<f4"), ("ny", "<f4"), ("nz", "<f4")]
        columns += [nrm[:, 0], nrm[:, 1], nrm[:, 2]]
    if surface.get("colors") is not None:
        col = _array(surface["colors"], np.float32, 3)
        if len(col) != len(pos):
            raise ValueError("colors and positions differ in length")
        rgb = np.clip(np.rint(col * 255.0), 0, 255).astype(np.uint8)
        fields += [("red", "u1"), ("green", "u1"), ("blue", "u1")]
        columns += [rgb[:, 0], rgb[:, 1], rgb[:, 2]]
    vertex = np.empty(len(pos), dtype=fields)
    for (name, _), column in zip(fields, columns):
        vertex[name] = column
    tris = None
    if surface.get("triangles") is not None:
        tris = _array(surface["triangles"], np.int32, 3)
        if len(tris) and (tris.min() < 0 or tris.max() >= len(pos)):
            raise ValueError("triangle refers to a vertex that does not exist")
    ply_type = {"<f4": "float", "u1": "uchar"}
    header = ["ply", "format binary_little_endian 1.0", f"element vertex {len(pos)}"]
    header += [f"property {ply_type[t]} {name}" for name, t in fields]
    if tris is not None:
        header += [f"element face {len(tris)}", "property list uchar int vertex_indices"]
    header.append("end_header")
    with open(path, "wb") as f:
        f.write(("\n".join(header) + "\n").encode("ascii"))
        f.write(vertex.tobytes())
        if tris is not None:
            face = np.empty(len(tris), dtype=[("n", "u1"), ("v", "<i4", (3,))])
            face["n"] = 3
            face["v"] = tris
            f.write(face.tobytes())


def read_ply(path: str) -> Dict[str, np.ndarray]:
    """Read back a file written by ``write_ply`` (numpy arrays; colours in [0, 1])."""
    with open(path, "rb") as f:
        if f.readline().strip() != b"ply":
            raise ValueError("not a PLY file")
        n_vertex = n_face = 0
        props = []
        while True:
            line = f.readline().decode("ascii").strip()
            if line == "end_header":
                break
            parts = line.split()
            if parts[:2] == ["element", "vertex"]:
                n_vertex = int(parts[2])
            elif parts[:2] == ["element", "face"]:
                n_face = int(parts[2])
            elif parts[0] == "property" and parts[1] != "list":
                props.append((parts[2], {"float": "<f4", "uchar": "u1"}[parts[1]]))
        vertex = np.frombuffer(f.read(n_vertex * np.dtype(props).itemsize), dtype=props)
        out = {"positions": np.stack([vertex["x"], vertex["y"], vertex["z"]], 1)}
        if "nx" in vertex.dtype.names:
            out["normals"] = np.stack([vertex["nx"], vertex["ny"], vertex["nz"]], 1)
        if "red" in vertex.dtype.names:
            out["colors"] = np.stack([vertex["red"], vertex["green"], vertex["blue"]], 1).astype(np.float32) / 255.0
        if n_face:
            face = np.frombuffer(f.read(n_face * 13), dtype=[("n", "u1"), ("v", "<i4", (3,))])
            out["triangles"] = face["v"].copy()
    return out


def connected_triangle_components(triangles: torch.Tensor, n_vertices: int):
    """Connected components of a triangle mesh (triangles joined through shared vertices):
    ``(component of every triangle (T,) int64 in [0, n), triangles per component (n,) int64)``.
    Label propagation with pointer jumping in torch ops, on whatever device ``triangles`` is on."""
    t = triangles.long()
    if t.numel() == 0:
        return t.new_zeros(0), t.new_zeros(0)
    label = torch.arange(n_vertices, device=t.device)
    flat = t.reshape(-1)
    while True:
        lowest = label[t].min(dim=1).values
        new = label.scatter_reduce(0, flat, lowest.repeat_interleave(3), reduce="amin")
        for _ in range(4):
            new = new[new]
        if torch.equal(new, label):
            break
        label = new
    _, component, sizes = torch.unique(label[t[:, 0]], return_inverse=True, return_counts=True)
    return component, sizes
