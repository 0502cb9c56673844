"""Sparse-dense grids: hashed blocks of G^3 dense cells (API of ash/grid.py).

``embeddings`` is a ``(num_embeddings, G**3, embedding_dim)`` parameter; block
``b`` of it belongs to the integer block coordinate the hash engine maps to
``b``.  A position ``x`` (in cell units) lives in block ``floor(x / G)``, cell
``x - G * block`` (linearised x fastest) at fractional ``offset``.  Class,
method and argument names follow ash/grid.py:28-863.
"""
from typing import Literal, Optional, Tuple, Union

import torch
import torch.nn as nn

from .common import _get_c_extension
from .core import ASHEngine, ASHModule, _as_device
from .grid_nns import enumerate_neighbor_coord_offsets
from .grid_query import FusedGridQuery, SparseDenseGridQuery
from .hashmap import HashSet

backend = _get_c_extension()


class SparseDenseGrid(ASHModule):
    """Sparse grid of dense ``grid_dim``^3 blocks, positions measured in cells."""

    def __init__(self, in_dim: int, num_embeddings: int, embedding_dim: int, grid_dim: int,
                 device: Optional[Union[str, torch.device]] = torch.device("cpu")):
        assert in_dim == 3, "Only 3D sparse-dense grid is supported for now."
        assert embedding_dim <= 16, "Embedding dim must be <= 16 for now."
        super().__init__()
        self.in_dim = in_dim
        self.num_embeddings = num_embeddings
        self.embedding_dim = embedding_dim
        self.grid_dim = grid_dim
        self.device = _as_device(device)
        self.num_cells_per_grid = grid_dim**in_dim

        self.transform_world_to_cell = lambda x: x
        self.transform_cell_to_world = lambda x: x

        self.engine = ASHEngine(in_dim, num_embeddings, self.device)
        self.embeddings = nn.Parameter(self._allocate_embeddings())

        # Dense (per-cell) structure is fixed by grid_dim and built once.
        self.cell_indices = torch.arange(self.num_cells_per_grid, dtype=torch.long, device=self.device)
        self.cell_coords = self._delinearize_cell_indices(self.cell_indices)
        self.lut_cell_nb2grid_nb, self.lut_cell_nb2cell_idx = self.construct_cell_neighbor_lut(
            radius=1, bidirectional=False)

        # Sparse (per-block) structure depends on the active set; built on demand.
        self.grid_indices = None
        self.grid_coords = None
        self.lut_grid_nb2grid_idx = None

        # forward() runs as ONE fused launch when the world <-> cell transform is the class's own
        # (it is described to the kernel by an origin and a cell size); set to False to force the
        # reference's split + find + pre-split kernel sequence.
        self.fused = True
        self.tiled_convolution = True
        self.separable_gaussian = True
        # "dense" (the reference's contract): every backward call returns a fresh, zero-filled,
        # table-sized gradient that autograd accumulates into embeddings.grad.  "in_place": the
        # fused backward passes add straight into embeddings.grad (created as zeros when missing),
        # which saves a table-sized allocation + zero-fill (+ add) per call; clear the gradient with
        # embeddings.grad.zero_() or zero_grad(set_to_none=False) between steps as usual.
        # "row_list": the fused backward passes return an uncoalesced SPARSE gradient (8 records per
        # query: block index, cell index, row) written with coalesced stores -- no table-sized buffer,
        # zero-fill or read-modify-write; embeddings.grad is then a sparse tensor, to be consumed by an
        # optimiser that accepts sparse gradients (torch.optim.SGD / SparseAdam) or by
        # apply_row_list_(), as with nn.Embedding(sparse=True).
        self.grad_mode = "dense"
        self._lut32 = None
        self._lut32_source = None
        self._own_transform = self.transform_world_to_cell

    def _allocate_embeddings(self) -> torch.Tensor:
        """Storage of the embedding table (overridden where the table lives elsewhere)."""
        return torch.zeros(self.num_embeddings, self.num_cells_per_grid, self.embedding_dim, device=self.device)

    # ------------------------------------------------------------------ allocation
    def spatial_init_(self, points: torch.Tensor, dilation: int = 1, bidirectional: bool = False):
        """Activate the blocks around ``points`` (world units), ash/grid.py:121-159.

        Returns ``(grid_coords (n,1,3) int32, cell_coords (1,G^3,3) int32, grid_indices (n,1)
        int64, cell_indices (1,G^3) int64)`` of the touched blocks, new or not.
        """
        if (self.fused and points.is_cuda and hasattr(backend, "grid_spatial_init")
                and self.transform_world_to_cell is self._own_transform):
            return self._spatial_init_fused(points, dilation, bidirectional)
        points = self.transform_world_to_cell(points)
        block = self.grids_in_bound(torch.floor(points / self.grid_dim).int())
        offsets, _ = enumerate_neighbor_coord_offsets(self.in_dim, dilation, bidirectional, self.device)
        candidates = (block.view(-1, 1, self.in_dim) + offsets.int().view(1, -1, self.in_dim)).view(-1, self.in_dim)
        candidates = self.grids_in_bound(candidates)

        # Deduplicate through a scratch hash set sized for the worst case (every
        # candidate distinct); the reference sizes it by the point count and leans
        # on duplicates (ash/grid.py:145), which can overflow.
        if candidates.shape[0] == 0:
            unique = candidates
            grid_indices = torch.empty(0, dtype=torch.long, device=self.device)
        else:
            scratch = HashSet(key_dim=self.in_dim, capacity=candidates.shape[0], device=self.device)
            scratch.insert(candidates)
            unique = scratch.keys()
            self.engine.insert_keys(unique)
            grid_indices, masks = self.engine.find(unique)
            assert masks.all(), "grid capacity exhausted during spatial_init_"
        return (
            unique.view(-1, 1, self.in_dim),
            self.cell_coords.view(1, -1, self.in_dim),
            grid_indices.view(-1, 1),
            self.cell_indices.view(1, -1),
        )

    def _block_bounds(self):
        """Half-open range of admissible block coordinates, or (None, None)."""
        return None, None

    def _spatial_init_fused(self, points: torch.Tensor, dilation: int, bidirectional: bool):
        """One launch: block of every point, neighbourhood, insert-if-absent, compact list of the
        touched blocks.  The temporary hash set, insert, keys() and find of the reference's
        sequence disappear; one device read (the list length) remains."""
        n_emb = self.num_embeddings
        if getattr(self, "_touch_scratch", None) is None:
            dev = self.device
            self._touch_scratch = (
                torch.zeros((n_emb, 3), dtype=torch.int32, device=dev), torch.zeros(n_emb, dtype=torch.int32, device=dev),
                torch.zeros(n_emb, dtype=torch.int32, device=dev), torch.zeros(1, dtype=torch.int32, device=dev))
            self._touch_stamp = 0
        coords, touched, tlist, tcount = self._touch_scratch
        self._touch_stamp = self._touch_stamp % 0x7FFFFFFF + 1
        origin, cell_size = self._cell_frame()
        lo, hi = self._block_bounds()
        backend.grid_spatial_init(
            self.engine.backend, points.to(torch.float32).contiguous().view(-1, self.in_dim), cell_size, origin,
            self.grid_dim, dilation, bidirectional, coords, touched, self._touch_stamp, tlist, tcount, lo, hi)
        n = int(tcount.item())
        st = self.engine.backend.status()
        assert not (st & backend.STATUS_CAPACITY), "grid capacity exhausted during spatial_init_"
        self.engine._size_bound = self.engine.capacity  # native insertions bypass the host-side bound
        grid_indices = tlist[:n].long()
        return (
            coords[grid_indices].view(-1, 1, self.in_dim),
            self.cell_coords.view(1, -1, self.in_dim),
            grid_indices.view(-1, 1),
            self.cell_indices.view(1, -1),
        )

    def ray_init_(self, ray_o, rays_d, rays_near, rays_far, dilation: int = 3) -> None:
        raise NotImplementedError("Ray-tracing initialization not implemented yet")

    # ------------------------------------------------------------------ query
    def query(self, x: torch.Tensor):
        """Split cell-unit positions into ``(grid_indices, cell_indices, offsets, masks)``
        (ash/grid.py:183-199)."""
        G = self.grid_dim
        block = (x / G).floor()
        local = x - block * G
        cell = local.floor()
        offsets = local - cell
        grid_indices, masks = self.engine.find(block.int())
        # `local` can round up to exactly G for tiny negative x; keep the cell in range.
        cell_indices = self._linearize_cell_coords(cell.int().clamp_(0, G - 1))
        return grid_indices, cell_indices, offsets, masks

    def forward(self, x: torch.Tensor, interpolation: Literal["nearest", "linear", "smooth_step"] = "smooth_step"):
        """Differentiable query at world positions ``x`` (N, 3): returns
        ``(features (N, embedding_dim), masks (N,))``; ash/grid.py:201-238."""
        if interpolation not in ("nearest", "linear", "smooth_step"):
            raise ValueError(f"Unknown interpolation: {interpolation}")
        if interpolation != "nearest" and (self.grid_coords is None or self.lut_grid_nb2grid_idx is None):
            self.construct_grid_neighbor_lut_(radius=1, bidirectional=False)

        if (interpolation != "nearest" and self.fused and x.is_cuda and x.dtype == torch.float32
                and hasattr(backend, "grid_query_forward")
                and self.transform_world_to_cell is self._own_transform):
            origin, cell_size = self._cell_frame()
            grad_buffer = None
            if self.grad_mode == "in_place" and self.embeddings.requires_grad and torch.is_grad_enabled():
                if self.embeddings.grad is None:
                    self.embeddings.grad = torch.zeros_like(self.embeddings)
                grad_buffer = self.embeddings.grad
            elif self.grad_mode == "row_list":
                if not hasattr(backend, "grid_query_backward_rows"):
                    raise ValueError("grad_mode 'row_list' needs the native row-list backward")
                grad_buffer = "row_list"
            elif self.grad_mode not in ("dense", "in_place"):
                raise ValueError(f"Unknown grad_mode: {self.grad_mode}")
            geom = (self.engine.backend, self._neighbor_lut32(), cell_size, origin, self.grid_dim, interpolation,
                    grad_buffer)
            return FusedGridQuery.apply(self.embeddings, x, geom)

        x = self.transform_world_to_cell(x)
        grid_indices, cell_indices, offsets, masks = self.query(x)

        if interpolation == "nearest":
            return self.embeddings[grid_indices, cell_indices], masks
        features = SparseDenseGridQuery.apply(
            self.embeddings, offsets, grid_indices, cell_indices, masks, self.lut_grid_nb2grid_idx,
            self.lut_cell_nb2cell_idx, self.lut_cell_nb2grid_nb, self.grid_dim, interpolation)
        return features, masks

    @torch.no_grad()
    def zero_grad_rows_(self, x: torch.Tensor) -> None:
        """Clear, in ``embeddings.grad``, exactly the rows that queries at world positions ``x``
        touch: with ``grad_mode = "in_place"`` this replaces the table-sized zero-fill between steps
        by one pass over the batch (call it with the positions of the step just taken)."""
        if self.embeddings.grad is None:
            return
        if self.lut_grid_nb2grid_idx is None:
            self.construct_grid_neighbor_lut_(radius=1, bidirectional=False)
        origin, cell_size = self._cell_frame()
        backend.grid_zero_rows(self.engine.backend, self.embeddings.grad, x.detach().to(torch.float32), cell_size,
                               origin, self.grid_dim, self._neighbor_lut32())

    @torch.no_grad()
    def apply_row_list_(self, target: torch.Tensor = None, alpha: float = 1.0) -> None:
        """Add ``alpha`` times the sparse gradient that ``grad_mode = "row_list"`` left in
        ``embeddings.grad`` to ``target`` (default: the embeddings themselves, i.e. a plain
        gradient-descent step with ``alpha = -learning_rate``), one pass over the list."""
        g = self.embeddings.grad
        if g is None:
            return
        if not g.is_sparse:
            raise ValueError("embeddings.grad is dense: apply_row_list_ is for grad_mode = 'row_list'")
        target = self.embeddings.data if target is None else target
        backend.rows_scatter_add(target, g._indices(), g._values(), alpha)

    def _cell_frame(self):
        """(origin, cell_size) such that cell position = (world - origin) / cell_size."""
        return [0.0, 0.0, 0.0], 1.0

    def _neighbor_lut32(self) -> torch.Tensor:
        """int32 copy of ``lut_grid_nb2grid_idx`` for the fused kernels, refreshed whenever that
        table is replaced (it is as stale or as fresh as the table the reference would read)."""
        if self._lut32 is None or self._lut32_source is not self.lut_grid_nb2grid_idx:
            self._lut32 = self.lut_grid_nb2grid_idx.to(torch.int32).contiguous()
            self._lut32_source = self.lut_grid_nb2grid_idx
        return self._lut32

    def items(self):
        """Active blocks in broadcastable form: ``(grid_coords (n,1,3), cell_coords (1,G^3,3),
        grid_indices (n,1), cell_indices (1,G^3))``; cell position = grid_coords * G + cell_coords,
        features = embeddings[grid_indices, cell_indices] (ash/grid.py:240-266)."""
        grid_coords, grid_indices = self.engine.items()
        return (
            grid_coords.view(-1, 1, self.in_dim),
            self.cell_coords.view(1, -1, self.in_dim),
            grid_indices.view(-1, 1),
            self.cell_indices.view(1, -1),
        )

    # ------------------------------------------------------------------ geometry
    @torch.no_grad()
    def get_bbox(self):
        return self.bbox_min, self.bbox_max

    def cell_to_world(self, grid_coords: torch.Tensor, cell_coords: torch.Tensor) -> torch.Tensor:
        """World positions (n * G^3, 3) of every cell of the given blocks."""
        cells = grid_coords.view(-1, 1, self.in_dim) * self.grid_dim + cell_coords.view(1, -1, self.in_dim)
        return self.transform_cell_to_world(cells).view(-1, self.in_dim)

    def grids_in_bound(self, grid_coords: torch.Tensor) -> torch.Tensor:
        return grid_coords

    @torch.no_grad()
    def _linearize_cell_coords(self, cell_coords: torch.Tensor) -> torch.Tensor:
        """(N, 3) cell coordinates -> linear cell index, x fastest."""
        assert cell_coords.dim() == 2 and cell_coords.shape[1] == self.in_dim
        strides = torch.tensor([self.grid_dim**d for d in range(self.in_dim)], dtype=torch.long,
                               device=cell_coords.device)
        return (cell_coords.long() * strides).sum(dim=1)

    @torch.no_grad()
    def _delinearize_cell_indices(self, cell_indices: torch.Tensor) -> torch.Tensor:
        """Linear cell index -> (…, 3) int32 cell coordinates."""
        digits = [
            torch.div(cell_indices, self.grid_dim**d, rounding_mode="floor") % self.grid_dim
            for d in range(self.in_dim)
        ]
        return torch.stack(digits, dim=1).int()

    # ------------------------------------------------------------------ sampling
    @torch.no_grad()
    def ray_sample(self, rays_o, rays_d, rays_near, rays_far, max_samples_per_ray: int):
        """Sample intervals inside active blocks along rays (ash/grid.py:322-377): returns
        ``(ray_indices (M,), t_near (M,), t_far (M,), prefix_sum (N,))``, lengths in world units."""
        bbox_min, bbox_max = self.get_bbox()
        ray_indices, t_nears, t_fars, prefix_sum = backend.ray_sample(
            self.engine.backend, self.transform_world_to_cell(rays_o), rays_d, rays_near / self.cell_size,
            rays_far / self.cell_size, self.transform_world_to_cell(bbox_min),
            self.transform_world_to_cell(bbox_max), max_samples_per_ray, float(self.grid_dim))
        return ray_indices, t_nears * self.cell_size, t_fars * self.cell_size, prefix_sum

    @torch.no_grad()
    def ray_find_near_far(self, rays_o, rays_d, t_min: float, t_max: float, t_step: float):
        """First / last occupied stretch along each ray (ash/grid.py:379-403)."""
        bbox_min, bbox_max = self.get_bbox()
        nears, fars = backend.ray_find_near_far(
            self.engine.backend, self.transform_world_to_cell(rays_o), rays_d,
            self.transform_world_to_cell(bbox_min), self.transform_world_to_cell(bbox_max),
            t_min / self.cell_size, t_max / self.cell_size, t_step / self.cell_size, float(self.grid_dim))
        return nears * self.cell_size, fars * self.cell_size

    def uniform_sample(self, num_samples: int, space: Literal["occupied", "empty"] = "occupied") -> torch.Tensor:
        """Uniform world positions inside randomly chosen active blocks (ash/grid.py:405-430)."""
        if space != "occupied":
            raise NotImplementedError("empty space sampling not implemented")
        active, _ = self.engine.items()
        pick = torch.randint(len(active), (num_samples,), device=self.device)
        inside = torch.rand(num_samples, self.in_dim, device=self.device)
        return self.transform_cell_to_world((active[pick].float() + inside) * self.grid_dim)

    # ------------------------------------------------------------------ filtering
    @staticmethod
    def _gaussian_weights_1d(size: int, sigma: float):
        """The 1-D factor of ash/grid.py:449-462: bin masses of a standard normal over ``size`` equal
        bins of [-sigma, sigma] (float64 numpy)."""
        import numpy as np
        import scipy.stats as st

        edges = np.linspace(-sigma, sigma, size + 1)
        return np.diff(st.norm.cdf(edges))

    @staticmethod
    def _gaussian_weights(size: int, sigma: float) -> torch.Tensor:
        """Separable kernel of ash/grid.py:449-462: the 1-D factor outer-multiplied and normalised."""
        import numpy as np

        k1 = SparseDenseGrid._gaussian_weights_1d(size, sigma)
        k3 = np.outer(k1, np.outer(k1, k1)).reshape(size, size, size)
        return torch.from_numpy(k3 / k3.sum()).float()

    @torch.no_grad()
    def gaussian_filter_(self, size: int, sigma: float) -> None:
        """In-place ``size``^3 Gaussian smoothing of every embedding channel.  The window is an outer
        product, so on the GPU it runs as three 1-D passes inside the shared-memory tile of the
        convolution (``separable_gaussian``; same values up to the order of the sums) instead of
        ``size``^3 taps per cell."""
        assert size % 2 == 1, "size must be odd"
        channels = self.embeddings.shape[-1]
        radius = size // 2
        emb = self.embeddings
        if (self.separable_gaussian and self.tiled_convolution and emb.is_cuda and emb.dtype == torch.float32
                and 1 <= radius <= self.grid_dim and hasattr(backend, "convolution_forward_separable")):
            k1 = self._gaussian_weights_1d(size, sigma)
            k1 = k1 / k1.sum()                       # (k1 (x) k1 (x) k1) / sum = product of the normalised factors
            w1 = torch.from_numpy(k1).float().view(1, size, 1).repeat(3, 1, channels).contiguous().to(emb.device)
            _, lut_g2g = self.construct_grid_neighbor_lut(1, bidirectional=True)
            _, _, grid_indices, _ = self.items()
            emb.copy_(backend.convolution_forward_separable(emb.data, w1, grid_indices, lut_g2g, self.grid_dim, radius))
            return
        weights = self._gaussian_weights(size, sigma).view(size, size, size, 1).repeat(1, 1, 1, channels)
        self.embeddings.copy_(self.convolution(self.embeddings, weights.to(self.embeddings.device)))

    def convolution(self, inputs: torch.Tensor, weights: torch.Tensor,
                    output_blocks: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Depth-wise (2R+1)^3 convolution over the sparse-dense structure (ash/grid.py:476-520).
        ``inputs`` (num_embeddings, G^3, C); ``weights`` (2R+1, 2R+1, 2R+1, C).  ``output_blocks``
        (int64 block indices) restricts the work to those output rows -- the others are left
        unwritten -- which is how ``ash.distributed.split_convolution`` divides it over ranks."""
        assert inputs.is_contiguous() and inputs.shape[:2] == self.embeddings.shape[:2]
        assert weights.is_contiguous() and weights.dim() == 4 and weights.shape[0] % 2 == 1
        radius = weights.shape[0] // 2
        assert weights.shape[:3] == (2 * radius + 1,) * 3
        assert weights.shape[3] == inputs.shape[-1] and weights.device == inputs.device

        grid_radius = (radius + self.grid_dim - 1) // self.grid_dim
        _, lut_g2g = self.construct_grid_neighbor_lut(grid_radius, bidirectional=True)
        _, _, grid_indices, cell_indices = self.items()
        if output_blocks is not None:
            grid_indices = output_blocks.to(torch.int64).view(-1, 1)
        if (self.tiled_convolution and inputs.is_cuda and inputs.dtype == torch.float32 and 1 <= radius <= self.grid_dim
                and hasattr(backend, "convolution_forward_tiled")):
            # the per-cell tables of this window are pure arithmetic: one CTA per block works
            # from a shared-memory halo tile instead of 2 x 343 table reads per cell
            return backend.convolution_forward_tiled(
                inputs, weights.view(-1, weights.shape[-1]), grid_indices, lut_g2g, self.grid_dim, radius)
        lut_c2g, lut_c2c = self.construct_cell_neighbor_lut(radius, bidirectional=True)
        return backend.convolution_forward(
            inputs, weights.view(lut_c2g.shape[1], weights.shape[-1]), torch.ones_like(inputs, dtype=torch.bool),
            grid_indices, cell_indices, lut_g2g, lut_c2c, lut_c2g, self.grid_dim)

    # ------------------------------------------------------------------ lookup tables
    @torch.no_grad()
    def construct_cell_neighbor_lut(self, radius: int, bidirectional: bool):
        """Per-cell neighbour tables ``(lut_cell_nb2grid_nb, lut_cell_nb2cell_idx)``, both
        (G^3, K) int64: for cell c and window offset k, which neighbouring block (numbered in the
        block-level window) and which cell inside it (ash/grid.py:525-564)."""
        G = self.grid_dim
        cell_offsets, _ = enumerate_neighbor_coord_offsets(self.in_dim, radius, bidirectional, self.device)
        _, block_offset2idx = enumerate_neighbor_coord_offsets(
            self.in_dim, (radius + G - 1) // G, bidirectional, self.device)
        nb = (self.cell_coords.view(-1, 1, self.in_dim) + cell_offsets.view(1, -1, self.in_dim)).view(-1, self.in_dim)
        block_shift = torch.div(nb, G, rounding_mode="floor").long()
        nb_cell = self._linearize_cell_coords(torch.remainder(nb, G))
        return (
            block_offset2idx(block_shift).view(self.num_cells_per_grid, -1),
            nb_cell.view(self.num_cells_per_grid, -1),
        )

    @torch.no_grad()
    def construct_grid_neighbor_lut(self, radius: int, bidirectional: bool):
        """Per-block tables ``(grid_coords (num_embeddings, 3) int32, lut_grid_nb2grid_idx
        (num_embeddings, K) int64)``; rows of inactive blocks and absent neighbours hold -1
        (ash/grid.py:566-617)."""
        coords, indices = self.engine.items()
        offsets, _ = enumerate_neighbor_coord_offsets(self.in_dim, radius, bidirectional, self.device)
        K = offsets.shape[0]
        grid_coords = torch.full((self.num_embeddings, self.in_dim), -1, dtype=torch.int32, device=self.device)
        lut = torch.full((self.num_embeddings, K), -1, dtype=torch.int64, device=self.device)
        if coords.shape[0] > 0:
            nb = (coords.view(-1, 1, self.in_dim) + offsets.int().view(1, -1, self.in_dim)).view(-1, self.in_dim)
            nb_indices, nb_masks = self.engine.find(nb)
            nb_indices = torch.where(nb_masks, nb_indices, torch.full_like(nb_indices, -1))
            grid_coords[indices] = coords
            lut[indices] = nb_indices.view(-1, K)
        return grid_coords, lut

    @torch.no_grad()
    def construct_grid_neighbor_lut_(self, radius: int, bidirectional: bool) -> None:
        if radius == 1 and not bidirectional and self.device.type == "cuda" and hasattr(backend, "grid_build_neighbor_lut"):
            # one table scan + 8 probes per block instead of items() + find(8n) + two scatters
            lut32, coords = backend.grid_build_neighbor_lut(self.engine.backend, self.num_embeddings, with_coords=True)
            self.grid_coords = coords
            self.lut_grid_nb2grid_idx = lut32.long()
            self._lut32, self._lut32_source = lut32, self.lut_grid_nb2grid_idx
            return
        self.grid_coords, self.lut_grid_nb2grid_idx = self.construct_grid_neighbor_lut(radius, bidirectional)

    # ------------------------------------------------------------------ surface extraction
    def marching_cubes(self, tsdfs, weights, color_fn=None, normal_fn=None, iso_value: float = 0.0,
                       weight_thr: float = 1.0, vertices_only=False):
        """Iso-surface of ``tsdfs`` (num_embeddings, G^3[, 1]) where ``weights`` >= ``weight_thr``.

        ``vertices_only=True``: the zero crossings along the +x/+y/+z cell edges
        (ash/src/grid.cu:453-604), returned as a dict of world ``positions`` (n, 3).
        ``vertices_only=False``: the triangle mesh (ash/src/grid.cu:607-946): a dict of world
        ``positions`` (V, 3) and ``triangles`` (T, 3) int32 vertex ids, normals (right-hand rule)
        towards increasing tsdf.  If the callbacks are given, ``colors`` / ``normals`` are evaluated
        at the positions.  The reference wraps the same arrays in Open3D geometry
        (ash/grid.py:657-712), a package this library does not depend on; ``ash.mesh.write_ply``
        stores the dict in a file.  Returns None when the surface is empty.
        """
        if self.grid_coords is None or self.lut_grid_nb2grid_idx is None:
            self.construct_grid_neighbor_lut_(radius=1, bidirectional=False)
        _, grid_indices = self.engine.items()
        tables = (grid_indices, self.grid_coords, self.lut_grid_nb2grid_idx, self.cell_coords,
                  self.lut_cell_nb2cell_idx, self.lut_cell_nb2grid_nb, self.grid_dim, iso_value, weight_thr)
        triangles = None
        if vertices_only:
            vertices = backend.isosurface_extraction(tsdfs, weights, *tables)
        else:
            triangles, vertices = backend.marching_cubes(tsdfs, weights, *tables)
        if len(vertices) == 0:
            return None
        positions = self.transform_cell_to_world(vertices)
        surface = {"positions": positions}
        if triangles is not None:
            surface["triangles"] = triangles
        if color_fn is not None:
            surface["colors"] = color_fn(positions)
        if normal_fn is not None:
            surface["normals"] = normal_fn(positions)
        return surface


class UnBoundedSparseDenseGrid(SparseDenseGrid):
    """Grid with a fixed metric ``cell_size`` and no fixed extent (ash/grid.py:714-776)."""

    def __init__(self, in_dim: int, num_embeddings: int, embedding_dim: int, grid_dim: int,
                 cell_size: float = 0.01, device: Optional[Union[str, torch.device]] = torch.device("cpu")):
        super().__init__(in_dim, num_embeddings, embedding_dim, grid_dim, device)
        self.cell_size = cell_size
        self.transform_world_to_cell = lambda x: x / self.cell_size
        self.transform_cell_to_world = lambda x: x * self.cell_size
        self._own_transform = self.transform_world_to_cell
        self.bbox_min = None
        self.bbox_max = None

    def _cell_frame(self):
        return [0.0, 0.0, 0.0], self.cell_size

    @torch.no_grad()
    def compute_bbox_(self):
        coords, _ = self.engine.items()
        lo = coords.min(dim=0)[0]
        hi = coords.max(dim=0)[0] + 1
        self.bbox_min = self.transform_cell_to_world(lo * self.grid_dim)
        self.bbox_max = self.transform_cell_to_world(hi * self.grid_dim)

    @torch.no_grad()
    def get_bbox(self, force_recompute: bool = False):
        if self.bbox_min is None or self.bbox_max is None or force_recompute:
            self.compute_bbox_()
        return self.bbox_min, self.bbox_max


# The spelling used by callers that write "Unbounded".
UnboundedSparseDenseGrid = UnBoundedSparseDenseGrid


class BoundedSparseDenseGrid(SparseDenseGrid):
    """Grid over a fixed box split into ``sparse_grid_dim``^3 blocks (ash/grid.py:779-863)."""

    def __init__(self, in_dim: int, num_embeddings: int, embedding_dim: int, grid_dim: int = 8,
                 sparse_grid_dim: int = 128, bbox_min: torch.Tensor = None, bbox_max: torch.Tensor = None,
                 device: Optional[Union[str, torch.device]] = None):
        assert in_dim == 3, "Only 3D is supported now"
        super().__init__(in_dim, num_embeddings, embedding_dim, grid_dim, device)
        self.sparse_grid_dim = sparse_grid_dim
        self.bbox_min = (-torch.ones(in_dim, device=self.device)) if bbox_min is None else bbox_min.to(self.device)
        self.bbox_max = torch.ones(in_dim, device=self.device) if bbox_max is None else bbox_max.to(self.device)
        self.cell_size = ((self.bbox_max - self.bbox_min) / (sparse_grid_dim * grid_dim - 1)).min().item()
        self.transform_world_to_cell = lambda x: (x - self.bbox_min) / self.cell_size
        self.transform_cell_to_world = lambda x: x * self.cell_size + self.bbox_min
        self._own_transform = self.transform_world_to_cell
        self._origin = [float(v) for v in self.bbox_min.tolist()]

    def _cell_frame(self):
        return self._origin, self.cell_size

    def grids_in_bound(self, grid_coords: torch.Tensor) -> torch.Tensor:
        inside = ((grid_coords >= 0) & (grid_coords < self.sparse_grid_dim)).all(dim=-1)
        return grid_coords[inside]

    def _block_bounds(self):
        return [0, 0, 0], [self.sparse_grid_dim] * 3

    def dense_init_(self):
        """Activate every block of the box."""
        r = torch.arange(self.sparse_grid_dim, device=self.device)
        coords = torch.stack(torch.meshgrid(r, r, r, indexing="ij")).reshape(self.in_dim, -1).T
        self.engine.insert_keys(coords.int().contiguous())
