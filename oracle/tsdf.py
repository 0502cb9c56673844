"""CPU restatement of one RGB-D TSDF fusion step.  TEST INFRASTRUCTURE ONLY.

Follows TSDFFusion.fuse_frame / project_points_to_rgbd of the reference demo
(demo/rgbd_fusion.py:76-110, :199-254) and SparseDenseGrid.spatial_init_ /
cell_to_world (ash/grid.py:121-159, :275-288) in float32 numpy.

Two substitutions, both stated where they happen:
* the depth unprojection of the demo is Open3D's create_from_depth_image (third party,
  version unpinned, not installed here; demo/rgbd_fusion.py:57-74): the textbook pinhole
  formula stands in for it, so parity with that call is unpinned;
* world -> cell -> block divides become multiplications by float32 reciprocals, which is
  what the Python layer computes when its tensors live on a CUDA device.
Every product and sum is rounded separately (numpy float32), the contract the CUDA
kernels follow too, so block and pixel assignment can be compared exactly.
"""
import numpy as np

from . import OracleHashMap

f32 = np.float32


def _affine(M, x, y, z):
    """((m0*x + m1*y) + m2*z) + m3 per row, each operation rounded to float32."""
    return [((M[r, 0] * x + M[r, 1] * y) + M[r, 2] * z) + M[r, 3] for r in range(3)]


def unproject(depth, K, cam_to_world, depth_max):
    """Pinhole stand-in for demo/rgbd_fusion.py:57-74: world points of the pixels with
    0 < depth < depth_max, row-major pixel order."""
    K = K.astype(f32)
    Ei = cam_to_world.astype(f32)
    v, u = np.nonzero((depth > 0) & (depth < f32(depth_max)))
    d = depth[v, u].astype(f32)
    xc = (u.astype(f32) - K[0, 2]) * d / K[0, 0]
    yc = (v.astype(f32) - K[1, 2]) * d / K[1, 1]
    return np.stack(_affine(Ei, xc, yc, d), axis=1)


def touched_blocks(points, cell_size, origin, G, dilation, bounds=None):
    """ash/grid.py:132-148 with bidirectional dilation: unique block coordinates."""
    # reciprocals formed in double and rounded once, as torch does for `tensor / python_float`
    inv_cell, inv_G = f32(1.0 / float(cell_size)), f32(1.0 / float(G))
    cells = (points - np.asarray(origin, f32)) * inv_cell
    blocks = np.floor(cells * inv_G).astype(np.int32)
    r = np.arange(-dilation, dilation + 1, dtype=np.int32)
    offs = np.stack(np.meshgrid(r, r, r, indexing="ij"), -1).reshape(-1, 3)
    cand = (blocks[:, None, :] + offs[None, :, :]).reshape(-1, 3)
    cand = np.unique(cand, axis=0)
    if bounds is not None:
        lo, hi = bounds
        cand = cand[((cand >= np.asarray(lo)) & (cand < np.asarray(hi))).all(axis=1)]
    return cand


def project(cell_pos, K, world_to_cam, color, depth, depth_max, trunc):
    """demo/rgbd_fusion.py:76-110: (sdf, rgb, weight) per cell position."""
    H, W = depth.shape
    K = K.astype(f32)
    E = world_to_cam.astype(f32)
    x, y, z = _affine(E, cell_pos[:, 0], cell_pos[:, 1], cell_pos[:, 2])
    un = (K[0, 0] * x + K[0, 1] * y) + K[0, 2] * z
    vn = (K[1, 0] * x + K[1, 1] * y) + K[1, 2] * z
    d = (K[2, 0] * x + K[2, 1] * y) + K[2, 2] * z
    with np.errstate(divide="ignore", invalid="ignore"):
        uf, vf = np.rint(un / d), np.rint(vn / d)
    inside = (d > 0) & (uf >= 0) & (vf >= 0) & (uf < W) & (vf < H)
    u, v = uf[inside].astype(np.int64), vf[inside].astype(np.int64)
    depth_r = np.zeros_like(d)
    depth_r[inside] = depth[v, u]
    rgb = np.zeros((len(d), 3), f32)
    rgb[inside] = color[v, u, :]
    sdf = depth_r - d
    ok = (depth_r > 0) & (depth_r < f32(depth_max)) & (sdf >= -f32(trunc))
    sdf = np.where(sdf >= f32(trunc), f32(trunc), sdf)
    return sdf.astype(f32), rgb, (ok & inside).astype(f32)


class OracleTSDF:
    """Unbounded (origin 0) or bounded (origin = bbox_min) grid state on the CPU."""

    def __init__(self, num_embeddings, G, cell_size, dilation, D=5, origin=(0, 0, 0), bounds=None):
        self.G, self.cell_size, self.dilation, self.origin, self.bounds = G, float(cell_size), dilation, origin, bounds
        self.map = OracleHashMap(3, num_embeddings)
        self.emb = np.zeros((num_embeddings, G**3, D), f32)
        self.trunc = f32(dilation * cell_size * G)
        c = np.arange(G**3)
        self.cell_coords = np.stack([c % G, (c // G) % G, c // (G * G)], 1).astype(np.int32)  # ash/grid.py:307-317

    def fuse_frame(self, depth, color, K, world_to_cam, cam_to_world, depth_max):
        """demo/rgbd_fusion.py:199-254.  ``world_to_cam`` is the demo's extrinsic, ``cam_to_world``
        its inverse (both (4, 4), rounded to float32 here).  Returns the touched block coordinates."""
        depth = depth.astype(f32)
        pts = unproject(depth, K, cam_to_world[:3], depth_max)
        if len(pts) == 0:
            return np.zeros((0, 3), np.int32)
        blocks = touched_blocks(pts, self.cell_size, self.origin, self.G, self.dilation, self.bounds)
        self.map.insert_keys(blocks)
        idx, ok = self.map.find(blocks)
        assert ok.all()
        # ash/grid.py:275-288 cell_to_world
        cells = (blocks[:, None, :] * self.G + self.cell_coords[None, :, :]).astype(f32)
        pos = (cells * f32(self.cell_size) + np.asarray(self.origin, f32)).reshape(-1, 3)
        sdf, rgb, w = project(pos, K, world_to_cam[:3], color.astype(f32), depth, depth_max, self.trunc)
        e = self.emb[idx]  # (n, cells, D)
        n = len(blocks)
        w = w.reshape(n, -1, 1)
        sdf = sdf.reshape(n, -1, 1)
        rgb = rgb.reshape(n, -1, 3)
        w_sum = e[..., 4:5]
        w_new = w_sum + w
        den = w_new + f32(1e-6)
        e[..., 0:1] = (e[..., 0:1] * w_sum + sdf * w) / den
        e[..., 1:4] = (e[..., 1:4] * w_sum + rgb * w) / den
        e[..., 4:5] = w_new
        self.emb[idx] = e
        return blocks
