"""RGB-D TSDF fusion into a sparse-dense grid (API of the reference demo's TSDFFusion).

The reference implements one frame of fusion in Python (demo/rgbd_fusion.py:199-254):
unproject the depth image, ``spatial_init_`` the blocks around the points (temporary hash
set, insert, find), build every cell position of the touched blocks, project them back into
the frame, gather depth and colour, and update the running weighted averages -- about forty
torch launches and several multi-megabyte temporaries per frame.  Here a frame is two CUDA
launches (``tsdf_touch`` + ``tsdf_integrate``) with no temporaries and no host round trip.

Embedding layout as in the demo (:239-241): channel 0 sdf, 1..3 rgb, 4 weight.
"""
from typing import Union

import numpy as np
import torch

from .common import _get_c_extension
from .grid import BoundedSparseDenseGrid, UnBoundedSparseDenseGrid

backend = _get_c_extension()


def _host_matrix(m) -> np.ndarray:
    """A small camera matrix as float64 numpy on the host, whatever it arrived as."""
    if torch.is_tensor(m):
        m = m.detach().cpu().numpy()
    return np.asarray(m, dtype=np.float64)


class TSDFFusion:
    def __init__(self, grid: Union[UnBoundedSparseDenseGrid, BoundedSparseDenseGrid], dilation: int):
        assert grid.embedding_dim >= 5, "embeddings must hold sdf(1) + rgb(3) + weight(1)"
        self.grid = grid
        self.voxel_size = grid.cell_size
        self.dilation = dilation
        self.trunc = dilation * self.voxel_size * grid.grid_dim  # demo/rgbd_fusion.py:44
        dev = grid.device
        # per-block scratch kept across frames: coordinate of each block and the last frame
        # (stamp) that touched it
        self._coords = torch.zeros((grid.num_embeddings, 3), dtype=torch.int32, device=dev)
        self._touched = torch.zeros(grid.num_embeddings, dtype=torch.int32, device=dev)
        self._list = torch.zeros(grid.num_embeddings, dtype=torch.int32, device=dev)  # blocks touched by the frame
        self._count = torch.zeros(1, dtype=torch.int32, device=dev)
        self._stamp = 0
        self._c_frame = None   # origin / bounds as C arrays, built on first use
        self._list2 = self._count2 = None
        if isinstance(grid, BoundedSparseDenseGrid):
            self._origin = [float(v) for v in grid.bbox_min.tolist()]
            self._bounds = ([0, 0, 0], [grid.sparse_grid_dim] * 3)
        else:
            self._origin = [0.0, 0.0, 0.0]
            self._bounds = (None, None)

    @torch.no_grad()
    def fuse_frame(self, datum, counter=None) -> None:
        """``datum``: depth (H, W) raw, depth_scale, depth_max, intrinsic (3, 3), extrinsic (4, 4)
        world -> camera, rgb (H, W, 3); as demo/rgbd_fusion.py:199-254 (``datum.depth`` is scaled to
        metres in place there too).  ``counter``: optional int64 device tensor incremented by the
        number of blocks fused."""
        datum.depth *= datum.depth_scale
        depth = datum.depth
        K = _host_matrix(datum.intrinsic)
        E = _host_matrix(datum.extrinsic)
        Ei = np.linalg.inv(E)
        self._stamp = self._stamp % 0x7FFFFFFF + 1
        g = self.grid
        if hasattr(backend, "tsdf_fuse_frame") and depth.is_cuda:
            # one foreign call per frame: both launches, camera matrices passed as C arrays
            import ctypes

            f32 = ctypes.c_float
            color = datum.rgb
            if depth.dtype != torch.float32 or not depth.is_contiguous():
                depth = depth.float().contiguous()
            if color.dtype != torch.float32 or not color.is_contiguous():
                color = color.float().contiguous()
            org, lo3, hi3 = self._c_frame_arrays()
            backend.tsdf_fuse_frame(
                g.engine.backend, g.embeddings.data, g.grid_dim, depth, color, (f32 * 9)(*K.reshape(-1)[:9]),
                (f32 * 12)(*E.reshape(-1)[:12]), (f32 * 12)(*Ei.reshape(-1)[:12]), datum.depth_max, g.cell_size, org,
                self.dilation, self.trunc, self._coords, self._touched, self._stamp, self._list, self._count, lo3, hi3,
                counter)
            g.engine._size_bound = g.engine.capacity
            return
        backend.tsdf_touch(
            g.engine.backend, depth, K, Ei, datum.depth_max, g.cell_size, self._origin, g.grid_dim, self.dilation,
            self._coords, self._touched, self._stamp, *self._bounds, touched_list=self._list,
            touched_count=self._count)
        backend.tsdf_integrate(
            g.embeddings.data, g.grid_dim, self._coords, self._touched, self._stamp, depth, datum.rgb, K, E,
            datum.depth_max, g.cell_size, self._origin, self.trunc, counter=counter, touched_list=self._list,
            touched_count=self._count)
        # the engine's host-side size bound is stale after native insertions
        g.engine._size_bound = g.engine.capacity

    def _c_frame_arrays(self):
        import ctypes

        if self._c_frame is None:
            lo, hi = self._bounds
            f32, i32 = ctypes.c_float, ctypes.c_int32
            self._c_frame = ((f32 * 3)(*self._origin), (i32 * 3)(*lo) if lo is not None else None,
                             (i32 * 3)(*hi) if hi is not None else None)
        return self._c_frame

    @torch.no_grad()
    def fuse_dataset(self, frames, counter=None) -> None:
        """Fuse a sequence of frames (demo/rgbd_fusion.py:256-262).  Frames of one size and depth_max on the
        GPU go to the library as ONE call that enqueues both launches of every frame back to back."""
        frames = list(frames)
        g = self.grid
        same = (len(frames) > 1 and hasattr(backend, "tsdf_fuse_frames") and all(
            f.depth.is_cuda and f.depth.shape == frames[0].depth.shape and f.depth_max == frames[0].depth_max
            for f in frames) and self._stamp + len(frames) < 0x7FFFFFFF)
        if not same:
            for datum in frames:
                self.fuse_frame(datum, counter=counter)
            return
        depths, colors = [], []
        for f in frames:
            f.depth *= f.depth_scale
            depths.append(f.depth if f.depth.dtype == torch.float32 and f.depth.is_contiguous() else f.depth.float().contiguous())
            colors.append(f.rgb if f.rgb.dtype == torch.float32 and f.rgb.is_contiguous() else f.rgb.float().contiguous())
        K = np.stack([_host_matrix(f.intrinsic) for f in frames])
        E = np.stack([_host_matrix(f.extrinsic) for f in frames])
        Ei = np.linalg.inv(E)
        org, lo3, hi3 = self._c_frame_arrays()
        if self._list2 is None:   # two work lists: the allocation of a frame overlaps the fusion of the one before
            self._list2 = torch.zeros(2 * g.num_embeddings, dtype=torch.int32, device=g.device)
            self._count2 = torch.zeros(2, dtype=torch.int32, device=g.device)
        backend.tsdf_fuse_frames(
            g.engine.backend, g.embeddings.data, g.grid_dim, depths, colors, K, E, Ei, frames[0].depth_max, g.cell_size,
            org, self.dilation, self.trunc, self._coords, self._touched, self._stamp + 1, self._list2, self._count2, lo3,
            hi3, counter)
        self._stamp += len(frames)
        g.engine._size_bound = g.engine.capacity

    @torch.no_grad()
    def prune_by_weight_(self, grid_mean_weight_thr: float = 1) -> int:
        """Erase the blocks whose mean fusion weight stays below the threshold and clear their rows
        (demo/rgbd_fusion.py:112-128); returns how many were erased."""
        grid_coords, _, grid_indices, _ = self.grid.items()
        if grid_indices.numel() == 0:
            return 0
        rows = grid_indices.view(-1)
        weak = self.grid.embeddings[rows, :, 4].mean(dim=1) < grid_mean_weight_thr
        n = int(weak.sum())
        if n:
            self.grid.engine.erase(grid_coords.view(-1, 3)[weak].contiguous())
            self.grid.embeddings[rows[weak]] = 0
        self.grid.construct_grid_neighbor_lut_(radius=1, bidirectional=False)
        return n

    @torch.no_grad()
    def prune_by_mesh_connected_components_(self, ratio_to_largest_component: float = 0.5) -> int:
        """Keep only the blocks around the large connected pieces of the fused surface
        (demo/rgbd_fusion.py:130-197): mesh the volume, drop the components with fewer triangles
        than ``ratio_to_largest_component`` of the largest, re-derive the blocks within one block of
        the remaining vertices, erase every other block.  Returns how many blocks were erased."""
        from .hashmap import HashSet
        from .mesh import connected_triangle_components

        g = self.grid
        sdf = g.embeddings[..., 0].contiguous()
        weight = g.embeddings[..., 4].contiguous()
        mesh = g.marching_cubes(sdf, weight, vertices_only=False, iso_value=0.0, weight_thr=1)
        if mesh is None:
            return 0
        triangles, positions = mesh["triangles"], mesh["positions"]
        component, sizes = connected_triangle_components(triangles, positions.shape[0])
        keep_component = sizes > ratio_to_largest_component * sizes.max()
        kept_vertices = torch.unique(triangles[keep_component[component]].long().reshape(-1))
        xyz = positions[kept_vertices]

        around = UnBoundedSparseDenseGrid(3, g.num_embeddings, 1, g.grid_dim, cell_size=g.cell_size, device=g.device) \
            if not isinstance(g, BoundedSparseDenseGrid) else \
            BoundedSparseDenseGrid(3, g.num_embeddings, 1, g.grid_dim, g.sparse_grid_dim, g.bbox_min, g.bbox_max, g.device)
        around.spatial_init_(xyz, dilation=1, bidirectional=True)
        all_coords = g.items()[0].view(-1, 3)
        kept_coords = around.items()[0].view(-1, 3)
        kept = HashSet(key_dim=3, capacity=int(len(all_coords) * 1.2) + 1, device=g.device)
        kept.insert(kept_coords)
        to_prune = all_coords[~kept.find(all_coords)].contiguous()
        if len(to_prune):
            g.engine.erase(to_prune)
        g.construct_grid_neighbor_lut_(radius=1, bidirectional=False)
        return int(len(to_prune))
