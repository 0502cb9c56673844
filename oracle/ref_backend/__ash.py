"""Stand-in for the reference's native module ``__ash`` on CPU.  TEST INFRASTRUCTURE ONLY.

Exposes exactly the names the reference registers in ash/src/pybind.cpp:9-37
(except the mesh extraction functions), implemented on the CPU oracle, so that
the reference's UNMODIFIED Python layer (ash/*.py) can run on ``device="cpu"``:

    sys.path[:0] = ["<repo>/oracle/ref_backend", "<repo>", "<reference root>"]
    import ash                      # the reference's package, on top of this file

That stack pins the oracle against the reference's own known-answer tests and
generates the golden vectors in tests/golden.  Torch CPU tensors are passed to
the oracle as numpy views without copying.
"""
import numpy as np
import torch

import oracle as _o


STATUS_CAPACITY, STATUS_PROBE, STATUS_SPIN, STATUS_DUPLICATE = 1, 2, 4, 8


def _np(t: torch.Tensor):
    return t.detach().contiguous().numpy()


class HashMap:
    """ash/src/hashmap.h:18-61."""

    def __init__(self, key_dim, capacity, heap, device):
        assert torch.device(device).type == "cpu"
        self._device = torch.device(device)
        self._heap = heap  # aliased and mutated in place (ash/src/hashmap_impl.h:23)
        self._m = _o.OracleHashMap(key_dim, capacity, heap.numpy())
        self._status = 0

    def find(self, keys):
        idx, msk = self._m.find(_np(keys))
        return torch.from_numpy(idx), torch.from_numpy(msk)

    def insert_keys(self, keys):
        if self._m.insert_keys(_np(keys)):
            self._status |= STATUS_CAPACITY

    def status(self):
        """Read-and-clear status word of the product's native module (not in the reference)."""
        st, self._status = self._status, 0
        return st

    def insert(self, keys, values, external_values):
        if self._m.insert(
            _np(keys),
            {k: _np(v) for k, v in values.items()},
            {k: external_values[k].numpy() for k in values},
        ):
            self._status |= STATUS_CAPACITY

    def erase(self, keys):
        self._m.erase(_np(keys.to(torch.int32)))

    def clear(self):
        self._m.clear()

    def load_states(self, states):
        self._m.load_states(
            _np(states["active_keys"]), _np(states["active_indices"]), _np(states["heap"]).copy()
        )

    def items(self):
        k, i = self._m.items()
        return torch.from_numpy(k), torch.from_numpy(i)

    def size(self):
        return self._m.size()

    def device(self):
        return self._device


def query_forward(emb, off, gi, ci, masks, g2g, c2c, c2g, grid_dim, interpolation):
    return torch.from_numpy(
        _o.query_forward(_np(emb), _np(off), _np(gi), _np(ci), _np(masks), _np(g2g), _np(c2c), _np(c2g), interpolation)
    )


def query_backward_forward(z, emb, off, gi, ci, masks, g2g, c2c, c2g, grid_dim, interpolation):
    ge, go = _o.query_backward_forward(
        _np(z), _np(emb), _np(off), _np(gi), _np(ci), _np(masks), _np(g2g), _np(c2c), _np(c2g), interpolation
    )
    return torch.from_numpy(ge), torch.from_numpy(go)


def query_backward_backward(gge, ggo, z, emb, off, gi, ci, masks, g2g, c2c, c2g, grid_dim, interpolation):
    gz, ge, go = _o.query_backward_backward(
        _np(ggo), _np(z), _np(emb), _np(off), _np(gi), _np(ci), _np(masks), _np(g2g), _np(c2c), _np(c2g), interpolation
    )
    return torch.from_numpy(gz), torch.from_numpy(ge), torch.from_numpy(go)


def convolution_forward(inputs, weights, masks, grid_indices, cell_indices, g2g, c2c, c2g, grid_dim):
    return torch.from_numpy(
        _o.convolution_forward(
            _np(inputs), _np(weights), _np(masks), _np(grid_indices), _np(cell_indices), _np(g2g), _np(c2c), _np(c2g)
        )
    )


def ray_find_near_far(hashmap, o, d, bbox_min, bbox_max, t_min, t_max, t_step, grid2cell):
    n, f = _o.ray_find_near_far(
        hashmap._m, _np(o), _np(d), _np(bbox_min), _np(bbox_max), t_min, t_max, t_step, grid2cell
    )
    return torch.from_numpy(n), torch.from_numpy(f)


def ray_sample(hashmap, o, d, nears, fars, bbox_min, bbox_max, max_samples_per_ray, grid2cell):
    nears = torch.as_tensor(nears, dtype=torch.float32).expand(len(o)) if not torch.is_tensor(nears) or nears.ndim == 0 else nears
    fars = torch.as_tensor(fars, dtype=torch.float32).expand(len(o)) if not torch.is_tensor(fars) or fars.ndim == 0 else fars
    r = _o.ray_sample(
        hashmap._m, _np(o), _np(d), _np(nears), _np(fars), _np(bbox_min), _np(bbox_max), max_samples_per_ray, grid2cell
    )
    return tuple(torch.from_numpy(x) for x in r)


def isosurface_extraction(sdfs, weights, grid_indices, grid_coords_table, g2g, cell_coords_table, c2c, c2g, grid_dim,
                          iso_value, weight_thr):
    return torch.from_numpy(
        _o.isosurface_extraction(_np(sdfs), _np(weights), _np(grid_indices), _np(grid_coords_table), _np(g2g),
                                 _np(cell_coords_table), _np(c2c), _np(c2g), grid_dim, iso_value, weight_thr))


def marching_cubes(sdfs, weights, grid_indices, grid_coords_table, g2g, cell_coords_table, c2c, c2g, grid_dim,
                   iso_value, weight_thr):
    tris, verts = _o.marching_cubes(_np(sdfs), _np(weights), _np(grid_indices), _np(grid_coords_table), _np(g2g),
                                    _np(cell_coords_table), _np(c2c), _np(c2g), grid_dim, iso_value, weight_thr)
    return torch.from_numpy(tris), torch.from_numpy(verts)
