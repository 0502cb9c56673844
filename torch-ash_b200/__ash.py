"""``__ash`` -- the native module of torch-ash, re-implemented for B200.

The reference builds a pybind11 extension of this name from ash/src
(ash/src/pybind.cpp:8-38) and its Python layer imports it through
``ash.common._get_c_extension``.  This module exports the same names with the
same arguments and return values, but every operation is a call into
``libashb200.so`` (hand-written sm_100a CUDA behind a C ABI, see
include/ashb200.h).  It is the only place where torch tensors meet the C ABI:
it allocates outputs with torch (caching allocator, current stream), passes raw
device pointers and turns non-zero status codes into ``RuntimeError``.

There is no CPU path: tensors must live on a CUDA device and the shared library
must have been built (``python torch-ash_b200/build.py``).
"""
import ctypes
import os
import warnings

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libashb200.so")

if not os.path.exists(_LIB_PATH):
    raise ImportError(
        f"{_LIB_PATH} is missing: build it with `python {os.path.join(_HERE, 'build.py')}` "
        "(needs nvcc; there is no CPU fallback)"
    )

_lib = ctypes.CDLL(_LIB_PATH)
_c = ctypes
_vp, _i64, _int = _c.c_void_p, _c.c_int64, _c.c_int

_lib.ashb_last_error_string.restype = _c.c_char_p
_lib.ashb_map_create.argtypes = [_int, _i64, _vp, _int, _c.POINTER(_vp)]
_lib.ashb_map_destroy.argtypes = [_vp]
_lib.ashb_map_clear.argtypes = [_vp, _vp]
_lib.ashb_map_size.argtypes = [_vp, _vp, _c.POINTER(_i64)]
_lib.ashb_map_status.argtypes = [_vp, _vp, _c.POINTER(_c.c_uint32)]
_lib.ashb_map_status_async.argtypes = [_vp, _vp, _vp]
_lib.ashb_map_find.argtypes = [_vp, _vp, _i64, _vp, _vp, _vp]
_lib.ashb_map_insert_keys.argtypes = [_vp, _vp, _i64, _vp]
_lib.ashb_map_insert_values.argtypes = [_vp, _vp, _i64, _int, _vp, _vp, _vp, _vp]
_lib.ashb_map_erase.argtypes = [_vp, _vp, _i64, _vp]
_lib.ashb_map_items.argtypes = [_vp, _vp, _vp, _i64, _c.POINTER(_i64), _vp]
_lib.ashb_map_load_states.argtypes = [_vp, _vp, _vp, _i64, _vp, _vp]
_lib.ashb_map_rehash.argtypes = [_vp, _vp]
_lib.ashb_query_forward.argtypes = [_int, _int] + [_vp] * 9 + [_i64] * 4 + [_vp]
_lib.ashb_query_backward_forward.argtypes = [_int, _int] + [_vp] * 11 + [_int] + [_i64] * 4 + [_vp]
_lib.ashb_query_backward_backward.argtypes = [_int, _int] + [_vp] * 12 + [_int] + [_i64] * 4 + [_vp]
_f32 = _c.c_float
_lib.ashb_conv_forward.argtypes = [_int] + [_vp] * 9 + [_int] + [_i64] * 6 + [_vp]
_lib.ashb_ray_find_near_far.argtypes = [_vp] * 7 + [_f32] * 4 + [_i64, _vp]
_lib.ashb_ray_sample_count.argtypes = [_vp] * 6 + [_i64, _f32, _i64, _vp]
_lib.ashb_ray_sample_fill.argtypes = [_vp] * 9 + [_i64, _f32, _i64, _vp]
_lib.ashb_tsdf_touch.argtypes = [_vp, _vp, _int, _int, _vp, _vp, _f32, _c.c_double, _vp, _int, _int, _vp, _vp, _vp, _vp,
                                 _c.c_uint32, _vp, _vp, _vp]
_lib.ashb_tsdf_integrate.argtypes = [_vp, _i64, _int, _i64, _vp, _vp, _c.c_uint32, _vp, _vp, _int, _int, _vp, _vp,
                                     _f32, _c.c_double, _vp, _f32, _int, _int, _int, _vp, _vp, _vp, _vp]
_lib.ashb_tsdf_fuse_frame.argtypes = [_vp, _vp, _i64, _int, _i64, _vp, _vp, _int, _int, _vp, _vp, _vp, _f32, _c.c_double, _vp,
                                      _int, _vp, _vp, _f32, _int, _int, _int, _vp, _vp, _c.c_uint32, _vp, _vp, _vp, _vp]
_lib.ashb_tsdf_fuse_frames.argtypes = [_vp, _vp, _i64, _int, _i64, _int, _vp, _vp, _int, _int, _vp, _vp, _vp, _f32, _c.c_double,
                                       _vp, _int, _vp, _vp, _f32, _int, _int, _int, _vp, _vp, _c.c_uint32, _vp, _vp, _int, _vp, _vp]
_lib.ashb_tsdf_fuse_frame_static.argtypes = [_vp, _vp, _i64, _int, _i64, _vp, _vp, _int, _int, _vp, _vp, _vp, _f32, _c.c_double,
                                             _vp, _int, _vp, _vp, _f32, _int, _int, _int, _vp]
_lib.ashb_tsdf_copy_timeouts.argtypes = [_vp]
_lib.ashb_grid_build_neighbor_lut.argtypes = [_vp, _vp, _vp, _i64, _vp]
_lib.ashb_grid_query_forward.argtypes = [_vp, _int, _int, _vp, _vp, _c.c_double, _vp, _int, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]
_lib.ashb_grid_query_backward.argtypes = [_vp, _int, _int, _vp, _vp, _vp, _c.c_double, _vp, _int, _vp, _vp, _vp, _vp, _int,
                                          _i64, _i64, _i64, _vp]
_lib.ashb_grid_query_backward_backward.argtypes = [_vp, _int, _int, _vp, _vp, _vp, _vp, _c.c_double, _vp, _int, _vp, _vp, _vp,
                                                   _vp, _int, _i64, _i64, _i64, _vp]
_lib.ashb_conv_forward_tiled.argtypes = [_vp, _vp, _vp, _vp, _vp, _int, _i64, _i64, _int, _int, _i64, _vp]
_lib.ashb_conv_forward_separable.argtypes = [_vp, _vp, _vp, _vp, _vp, _int, _i64, _i64, _int, _int, _i64, _vp]
_lib.ashb_grid_spatial_init.argtypes = [_vp, _vp, _i64, _c.c_double, _vp, _int, _int, _int, _vp, _vp, _vp, _vp, _c.c_uint32,
                                        _vp, _vp, _vp]
_lib.ashb_route_by_owner.argtypes = [_vp, _i64, _int, _int, _vp, _vp, _vp, _vp, _vp]
_lib.ashb_render_segments.argtypes = [_vp, _i64, _i64, _vp, _vp, _vp]
_lib.ashb_render_weights_forward.argtypes = [_vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp]
_lib.ashb_render_weights_backward.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp]
_lib.ashb_render_accumulate_forward.argtypes = [_vp, _vp, _int, _vp, _vp, _i64, _vp, _vp]
_lib.ashb_render_accumulate_backward.argtypes = [_vp, _vp, _vp, _vp, _i64, _i64, _int, _vp, _vp, _vp]
_lib.ashb_isosurface_extraction.argtypes = [_vp] * 9 + [_i64, _c.POINTER(_i64), _vp, _f32, _f32, _int, _i64, _i64, _i64, _vp]
_lib.ashb_set_find_cooperative.argtypes = [_int]
_lib.ashb_set_scatter_aggregation.argtypes = [_int]
_lib.ashb_peer_route_keys.argtypes = [_vp, _i64, _int, _int, _int, _vp] + [_i64] * 6 + [_vp, _vp, _vp, _vp]
_lib.ashb_peer_unpack_answers.argtypes = [_vp, _i64, _int, _int, _vp] + [_i64] * 6 + [_vp, _vp, _vp]
_lib.ashb_peer_find_answer.argtypes = [_vp, _int, _int, _vp] + [_i64] * 6 + [_vp]
_lib.ashb_peer_update.argtypes = [_vp, _int, _int, _int, _vp] + [_i64] * 6 + [_vp]
_lib.ashb_grid_query_forward_sharded.argtypes = [_vp, _int, _vp, _int, _vp, _c.c_double, _vp, _int, _vp, _vp, _vp, _vp,
                                                 _vp, _i64, _i64, _i64, _vp]
_lib.ashb_grid_query_backward_backward_sharded.argtypes = [_vp, _int, _vp, _vp, _vp, _vp, _int, _vp, _c.c_double, _vp, _int,
                                                           _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]
_lib.ashb_grid_query_backward_sharded.argtypes = [_vp, _int, _vp, _vp, _vp, _int, _vp, _c.c_double, _vp, _int, _vp, _vp,
                                                  _vp, _int, _vp, _i64, _i64, _i64, _vp]
_lib.ashb_measure_random_reads.argtypes = [_vp, _i64, _i64, _int, _c.c_uint32, _vp, _vp]
_lib.ashb_marching_cubes_count.argtypes = [_vp] * 9 + [_f32, _f32, _i64, _i64, _i64, _c.POINTER(_i64), _c.POINTER(_i64), _vp]
_lib.ashb_marching_cubes_fill.argtypes = [_vp] * 11 + [_i64, _vp, _i64, _f32, _int, _i64, _i64, _i64, _vp]
_RAY_ARGS = [_vp, _int, _vp, _i64, _int, _int, _vp, _c.c_double, _vp, _vp, _vp, _vp, _vp, _vp, _f32, _f32, _i64, _int, _vp]
_lib.ashb_render_rays_forward.argtypes = _RAY_ARGS + [_vp, _i64, _vp]
_lib.ashb_render_rays_backward.argtypes = _RAY_ARGS + [_vp, _vp, _vp, _vp, _i64, _vp]
_RAY_GRID = [_vp, _int, _vp, _i64, _int, _int, _vp, _c.c_double, _vp]
_lib.ashb_render_rays_intervals.argtypes = _RAY_GRID + [_vp, _vp, _vp, _vp, _f32, _f32, _i64, _int, _vp, _vp, _vp, _i64, _i64,
                                                        _vp]
_lib.ashb_render_intervals_forward.argtypes = _RAY_GRID + [_vp] * 6 + [_i64, _vp, _i64, _vp]
_lib.ashb_render_intervals_backward.argtypes = _RAY_GRID + [_vp] * 5 + [_i64, _vp, _vp, _vp, _vp, _i64, _vp]
_lib.ashb_grid_query_backward_rows.argtypes = [_vp, _int, _int, _int, _vp, _vp, _vp, _vp, _c.c_double, _vp, _int, _vp, _vp,
                                               _vp, _vp, _vp, _i64, _i64, _i64, _vp]
_lib.ashb_rows_scatter_add.argtypes = [_int, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _c.c_double, _vp]
_lib.ashb_set_find_filter.argtypes = [_int]
_lib.ashb_set_erase_cooperative.argtypes = [_int]
_lib.ashb_measure_random_reads_ilp.argtypes = [_vp, _i64, _i64, _int, _int, _c.c_uint32, _vp, _vp]
_ROUTED_LAYOUT = [_vp] + [_i64] * 8 + [_int, _int]
_lib.ashb_routed_route.argtypes = [_vp, _vp, _i64, _c.c_double, _vp, _int, _vp, _vp, _i64, _i64] + _ROUTED_LAYOUT + [_vp] * 4
_lib.ashb_routed_forward.argtypes = [_vp, _int, _vp, _c.c_double, _vp, _int, _vp, _vp, _i64, _i64] + _ROUTED_LAYOUT + [_vp]
_lib.ashb_routed_unpack_y.argtypes = [_vp, _i64, _vp, _vp, _i64] + _ROUTED_LAYOUT + [_vp]
_lib.ashb_routed_send_z.argtypes = [_vp, _i64, _vp, _i64] + _ROUTED_LAYOUT + [_vp]
_lib.ashb_routed_backward.argtypes = [_vp, _int, _vp, _vp, _int, _int, _c.c_double, _vp, _int, _vp, _vp, _i64, _i64] + _ROUTED_LAYOUT + [_vp]
_lib.ashb_routed_send_g.argtypes = [_vp, _i64, _vp, _i64] + _ROUTED_LAYOUT + [_vp]
_lib.ashb_routed_backward_backward.argtypes = [_vp, _int, _vp, _vp, _c.c_double, _vp, _int, _vp, _vp, _i64, _i64] + _ROUTED_LAYOUT + [_vp]
_lib.ashb_routed_unpack_grad_x.argtypes = [_vp, _i64, _vp, _i64] + _ROUTED_LAYOUT + [_vp]
_lib.ashb_grid_zero_rows.argtypes = [_vp, _int, _vp, _vp, _c.c_double, _vp, _int, _vp, _vp, _i64, _i64, _i64, _vp]

STATUS_CAPACITY, STATUS_PROBE, STATUS_SPIN, STATUS_DUPLICATE = 1, 2, 4, 8
_DTYPES = {torch.float32: 0, torch.float64: 1}
_INTERP = {"linear": 0, "smooth_step": 1}


def _check(rc: int):
    if rc != 0:
        raise RuntimeError(f"libashb200: {_lib.ashb_last_error_string().decode()} (status {rc})")


def measure_random_reads(buffer: torch.Tensor, n_reads: int, fetch_bytes: int = 64, seed: int = 1,
                         reads_per_thread: int = 1) -> None:
    """Launch ``n_reads`` scattered 16-byte reads over ``buffer`` (a large CUDA tensor), ``reads_per_thread``
    (1, 2, 4, 8) of them in flight per thread; time it from outside.  The reads per second reached are
    the ceiling for the probe / gather kernels."""
    buf = _cuda(buffer, "buffer")
    sink = torch.zeros(1, dtype=torch.int64, device=buf.device)
    with torch.cuda.device(buf.device):
        _check(_lib.ashb_measure_random_reads_ilp(buf.data_ptr(), buf.numel() * buf.element_size(), int(n_reads),
                                                  int(fetch_bytes), int(reads_per_thread), int(seed) & 0xFFFFFFFF,
                                                  sink.data_ptr(), _stream(buf.device)))


def set_erase_cooperative(enable: bool) -> None:
    """Process-wide choice of the erase kernel for key_dim <= 3: one thread per key (default) or
    eight lanes per key reading whole 128-byte lines of slots."""
    _check(_lib.ashb_set_erase_cooperative(int(bool(enable))))


def set_find_filter(mode: int) -> None:
    """Process-wide use of the one-bit-per-slot occupancy map in ``HashMap.find`` (key_dim <= 3):
    -1 automatic (tables of 64 MB and more), 0 never, 1 always.  Same answers in every mode."""
    _check(_lib.ashb_set_find_filter(int(mode)))


def set_scatter_aggregation(enable: bool) -> None:
    """Process-wide: combine, inside a warp, the gradient contributions of queries that share a
    corner row before the atomic reduction (helps batches whose neighbours in memory are
    neighbours in space, such as samples in marching order; costs a little on scattered batches)."""
    _check(_lib.ashb_set_scatter_aggregation(int(bool(enable))))


def set_find_cooperative(enable: bool) -> None:
    """Process-wide choice of the find kernel for key_dim <= 3: one thread per key (default, the
    faster one for tables beyond L2) or eight lanes per key reading whole 128-byte lines of slots."""
    _check(_lib.ashb_set_find_cooperative(int(bool(enable))))


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _cuda(t: torch.Tensor, name: str, dtype=None) -> torch.Tensor:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (there is no CPU implementation), got {t.device}")
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError(f"{name} must be {dtype}, got {t.dtype}")
    return t.contiguous()


def _interp_code(name: str) -> int:
    try:
        return _INTERP[name]
    except KeyError:
        raise RuntimeError(f"Unknown interpolation functor: {name}") from None  # ash/src/grid.cu:61


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise RuntimeError(f"embeddings must be float32 or float64, got {t.dtype}") from None


class HashMap:
    """Key (int32 x key_dim) -> index map; replaces ash/src/hashmap.h:18-61.

    ``heap`` is the caller's int32 free-index stack; it is aliased and mutated
    in place for the life of the map (it is part of the checkpoint,
    ash/core.py:72-74).
    """

    def __init__(self, key_dim: int, capacity: int, heap: torch.Tensor, device):
        device = torch.device(device)
        if device.type != "cuda":
            raise RuntimeError(f"HashMap needs a CUDA device (there is no CPU implementation), got {device}")
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        if heap.device != device or heap.dtype != torch.int32 or not heap.is_contiguous() or heap.numel() != capacity:
            raise RuntimeError("heap must be a contiguous int32 tensor of `capacity` elements on the map's device")
        self._device = device
        self._key_dim = int(key_dim)
        self._capacity = int(capacity)
        self._heap = heap
        handle = _vp()
        # make sure the heap's initial contents are complete before the library touches it
        torch.cuda.current_stream(device).synchronize()
        _check(_lib.ashb_map_create(self._key_dim, self._capacity, heap.data_ptr(), device.index, _c.byref(handle)))
        self._h = handle

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            self._h = None
            try:
                torch.cuda.synchronize(self._device)
            except Exception:  # interpreter shutdown
                pass
            if _lib is not None:  # None once the interpreter is tearing modules down
                _lib.ashb_map_destroy(h)

    # -- helpers
    def _keys(self, keys: torch.Tensor) -> torch.Tensor:
        if keys.dim() != 2 or keys.shape[1] != self._key_dim:
            raise RuntimeError(f"keys must be (N, {self._key_dim}), got {tuple(keys.shape)}")
        # erase() receives unconverted keys from the reference's engine (ash/core.py:256)
        return keys.to(self._device, torch.int32).contiguous()

    def _raise_status(self, where: str):
        st = _c.c_uint32()
        _check(_lib.ashb_map_status(self._h, _stream(self._device), _c.byref(st)))
        if st.value & STATUS_CAPACITY:
            warnings.warn(
                f"{where}: more distinct keys than the capacity {self._capacity}; the excess keys were dropped"
            )
        if st.value & (STATUS_PROBE | STATUS_SPIN | STATUS_DUPLICATE):
            raise RuntimeError(f"{where}: hash table status 0x{st.value:x}")

    # -- the reference's interface
    def find(self, keys: torch.Tensor):
        keys = self._keys(keys)
        n = keys.shape[0]
        indices = torch.empty(n, dtype=torch.int64, device=self._device)
        masks = torch.empty(n, dtype=torch.bool, device=self._device)
        _check(_lib.ashb_map_find(self._h, keys.data_ptr(), n, indices.data_ptr(), masks.data_ptr(), _stream(self._device)))
        return indices, masks

    def insert_keys(self, keys: torch.Tensor) -> None:
        keys = self._keys(keys)
        _check(_lib.ashb_map_insert_keys(self._h, keys.data_ptr(), keys.shape[0], _stream(self._device)))

    def insert(self, keys: torch.Tensor, values: dict, external_values: dict) -> None:
        keys = self._keys(keys)
        names = list(values.keys())
        k = len(names)
        src = (_vp * max(k, 1))()
        dst = (_vp * max(k, 1))()
        row = (_i64 * max(k, 1))()
        keep = []
        for j, name in enumerate(names):
            v = _cuda(values[name], f"values[{name!r}]")
            e = external_values[name]
            if not e.is_cuda or not e.is_contiguous() or e.dtype != v.dtype or e.shape[1:] != v.shape[1:]:
                raise RuntimeError(f"external_values[{name!r}] must be a contiguous CUDA tensor matching values")
            if v.shape[0] != keys.shape[0] or e.shape[0] != self._capacity:
                raise RuntimeError(f"value {name!r}: row counts do not match keys / capacity")
            keep.append(v)
            src[j], dst[j] = v.data_ptr(), e.data_ptr()
            row[j] = (v.numel() // max(v.shape[0], 1)) * v.element_size()
        _check(
            _lib.ashb_map_insert_values(self._h, keys.data_ptr(), keys.shape[0], k, src, dst, row, _stream(self._device))
        )

    def erase(self, keys: torch.Tensor) -> None:
        keys = self._keys(keys)
        _check(_lib.ashb_map_erase(self._h, keys.data_ptr(), keys.shape[0], _stream(self._device)))

    def clear(self) -> None:
        _check(_lib.ashb_map_clear(self._h, _stream(self._device)))

    def load_states(self, states: dict) -> None:
        keys = self._keys(states["active_keys"])
        indices = states["active_indices"].to(self._device, torch.int64).contiguous()
        heap = states["heap"].to(self._device, torch.int32).contiguous()
        if heap.numel() != self._capacity or indices.numel() != keys.shape[0]:
            raise RuntimeError("load_states: heap / indices sizes do not match the map")
        _check(
            _lib.ashb_map_load_states(
                self._h, keys.data_ptr(), indices.data_ptr(), keys.shape[0], heap.data_ptr(), _stream(self._device)
            )
        )
        self._raise_status("load_states")

    def items(self):
        n = self.size()
        keys = torch.empty((n, self._key_dim), dtype=torch.int32, device=self._device)
        indices = torch.empty(n, dtype=torch.int64, device=self._device)
        got = _i64()
        _check(
            _lib.ashb_map_items(self._h, keys.data_ptr(), indices.data_ptr(), n, _c.byref(got), _stream(self._device))
        )
        if got.value != n:
            raise RuntimeError(f"items(): enumerated {got.value} entries but size() is {n}")
        return keys, indices

    def size(self) -> int:
        out = _i64()
        _check(_lib.ashb_map_size(self._h, _stream(self._device), _c.byref(out)))
        return int(out.value)

    def device(self) -> torch.device:
        return self._device

    # -- additions (no counterpart in the reference)
    def status(self) -> int:
        """Read and clear the device status word (STATUS_* bits)."""
        st = _c.c_uint32()
        _check(_lib.ashb_map_status(self._h, _stream(self._device), _c.byref(st)))
        return int(st.value)

    def status_async(self, host_word: torch.Tensor) -> torch.cuda.Event:
        """Enqueue a copy of the status word into ``host_word`` (a pinned int32 CPU tensor of one
        element) and its clearing; returns the event after which ``host_word`` holds it."""
        if host_word.is_cuda or host_word.dtype != torch.int32 or host_word.numel() != 1 or not host_word.is_pinned():
            raise RuntimeError("host_word must be a pinned int32 CPU tensor of one element")
        _check(_lib.ashb_map_status_async(self._h, host_word.data_ptr(), _stream(self._device)))
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self._device))
        return ev

    def rehash(self) -> None:
        """Rebuild the table from its live entries, dropping erased slots (indices unchanged)."""
        _check(_lib.ashb_map_rehash(self._h, _stream(self._device)))

    @property
    def handle(self) -> int:
        return self._h.value


def _query_args(embeddings, offsets, grid_indices, cell_indices, masks, g2g, c2c, c2g):
    emb = _cuda(embeddings, "embeddings")
    if emb.dim() != 3:
        raise RuntimeError("embeddings must be (num_embeddings, cells_per_grid, embedding_dim)")
    dev = emb.device
    off = _cuda(offsets.to(dev), "offsets", torch.float32)  # ash/src/grid.cu:71: offsets are always float32
    gi = _cuda(grid_indices.to(dev), "grid_indices", torch.int64).view(-1)
    ci = _cuda(cell_indices.to(dev), "cell_indices", torch.int64).view(-1)
    mk = _cuda(masks.to(dev), "masks", torch.bool).view(-1)
    n = gi.shape[0]
    if off.shape != (n, 3) or ci.shape[0] != n or mk.shape[0] != n:
        raise RuntimeError("offsets / grid_indices / cell_indices / masks disagree on the number of queries")
    g2g = _cuda(g2g, "lut_grid_nb2grid_idx", torch.int64)
    c2c = _cuda(c2c, "lut_cell_nb2cell_idx", torch.int64)
    c2g = _cuda(c2g, "lut_cell_nb2grid_nb", torch.int64)
    if g2g.shape != (emb.shape[0], 8) or c2c.shape != (emb.shape[1], 8) or c2g.shape != (emb.shape[1], 8):
        raise RuntimeError("neighbour lookup tables must be (num_embeddings, 8) and (cells_per_grid, 8)")
    return emb, off, gi, ci, mk, g2g, c2c, c2g, n


def query_forward(embeddings, offsets, grid_indices, cell_indices, masks, lut_grid_nb2grid_idx,
                  lut_cell_nb2cell_idx, lut_cell_nb2grid_nb, grid_dim, interpolation):
    """ash/src/grid.cu:134-175."""
    emb, off, gi, ci, mk, g2g, c2c, c2g, n = _query_args(
        embeddings, offsets, grid_indices, cell_indices, masks, lut_grid_nb2grid_idx, lut_cell_nb2cell_idx,
        lut_cell_nb2grid_nb)
    out = torch.empty((n, emb.shape[2]), dtype=emb.dtype, device=emb.device)
    with torch.cuda.device(emb.device):
        _check(_lib.ashb_query_forward(
            _dtype_code(emb), _interp_code(interpolation), emb.data_ptr(), off.data_ptr(), gi.data_ptr(),
            ci.data_ptr(), mk.data_ptr(), g2g.data_ptr(), c2c.data_ptr(), c2g.data_ptr(), out.data_ptr(), n,
            emb.shape[0], emb.shape[1], emb.shape[2], _stream(emb.device)))
    return out


def query_backward_forward(z, embeddings, offsets, grid_indices, cell_indices, masks, lut_grid_nb2grid_idx,
                           lut_cell_nb2cell_idx, lut_cell_nb2grid_nb, grid_dim, interpolation,
                           grad_embeddings_out=None):
    """ash/src/grid.cu:257-307.  Returns (grad_embeddings, grad_offsets).

    ``grad_embeddings_out`` (an addition): accumulate into this existing tensor
    instead of allocating and zero-filling a fresh table-sized gradient.
    """
    emb, off, gi, ci, mk, g2g, c2c, c2g, n = _query_args(
        embeddings, offsets, grid_indices, cell_indices, masks, lut_grid_nb2grid_idx, lut_cell_nb2cell_idx,
        lut_cell_nb2grid_nb)
    z = _cuda(z, "z", emb.dtype)
    if z.shape != (n, emb.shape[2]):
        raise RuntimeError("z must be (num_queries, embedding_dim)")
    if grad_embeddings_out is None:
        grad_emb, zero = torch.empty_like(emb), 1
    else:
        grad_emb, zero = grad_embeddings_out, 0
        if grad_emb.shape != emb.shape or grad_emb.dtype != emb.dtype or not grad_emb.is_contiguous():
            raise RuntimeError("grad_embeddings_out must match embeddings")
    grad_off = torch.empty((n, 3), dtype=emb.dtype, device=emb.device)  # ash/src/grid.cu:277
    with torch.cuda.device(emb.device):
        _check(_lib.ashb_query_backward_forward(
            _dtype_code(emb), _interp_code(interpolation), z.data_ptr(), emb.data_ptr(), off.data_ptr(),
            gi.data_ptr(), ci.data_ptr(), mk.data_ptr(), g2g.data_ptr(), c2c.data_ptr(), c2g.data_ptr(),
            grad_emb.data_ptr(), grad_off.data_ptr(), zero, n, emb.shape[0], emb.shape[1], emb.shape[2],
            _stream(emb.device)))
    return grad_emb, grad_off


def query_backward_backward(grad_grad_embeddings, grad_grad_offsets, z, embeddings, offsets, grid_indices,
                            cell_indices, masks, lut_grid_nb2grid_idx, lut_cell_nb2cell_idx, lut_cell_nb2grid_nb,
                            grid_dim, interpolation, grad_embeddings_out=None):
    """ash/src/grid.cu:389-451.  Returns (grad_z, grad_embeddings, grad_offsets).

    ``grad_grad_embeddings`` is accepted and unused, and the returned
    grad_offsets is all zeros, exactly as in the reference (grid.cu:417-418, :426).
    """
    emb, off, gi, ci, mk, g2g, c2c, c2g, n = _query_args(
        embeddings, offsets, grid_indices, cell_indices, masks, lut_grid_nb2grid_idx, lut_cell_nb2cell_idx,
        lut_cell_nb2grid_nb)
    z = _cuda(z, "z", emb.dtype)
    ggo = _cuda(grad_grad_offsets, "grad_grad_offsets", emb.dtype)
    if z.shape != (n, emb.shape[2]) or ggo.shape != (n, 3):
        raise RuntimeError("z must be (num_queries, embedding_dim) and grad_grad_offsets (num_queries, 3)")
    if grad_embeddings_out is None:
        grad_emb, zero = torch.empty_like(emb), 1
    else:
        grad_emb, zero = grad_embeddings_out, 0
    grad_z = torch.empty_like(z)
    with torch.cuda.device(emb.device):
        _check(_lib.ashb_query_backward_backward(
            _dtype_code(emb), _interp_code(interpolation), ggo.data_ptr(), z.data_ptr(), emb.data_ptr(),
            off.data_ptr(), gi.data_ptr(), ci.data_ptr(), mk.data_ptr(), g2g.data_ptr(), c2c.data_ptr(),
            c2g.data_ptr(), grad_z.data_ptr(), grad_emb.data_ptr(), zero, n, emb.shape[0], emb.shape[1],
            emb.shape[2], _stream(emb.device)))
    grad_off = torch.zeros((n, 3), dtype=emb.dtype, device=emb.device)
    return grad_z, grad_emb, grad_off


def convolution_forward(inputs, weights, masks, grid_indices, cell_indices, lut_grid_nb2grid_idx,
                        lut_cell_nb2cell_idx, lut_cell_nb2grid_nb, grid_dim):
    """ash/src/grid.cu:1006-1043.  ``masks`` is indexed flat over (listed block, cell)."""
    inp = _cuda(inputs, "inputs")
    dev = inp.device
    w = _cuda(weights, "weights", inp.dtype)
    mk = _cuda(masks, "masks", torch.bool).view(-1)
    gi = _cuda(grid_indices, "grid_indices", torch.int64).view(-1)
    ci = _cuda(cell_indices, "cell_indices", torch.int64).view(-1)
    g2g = _cuda(lut_grid_nb2grid_idx, "lut_grid_nb2grid_idx", torch.int64)
    c2c = _cuda(lut_cell_nb2cell_idx, "lut_cell_nb2cell_idx", torch.int64)
    c2g = _cuda(lut_cell_nb2grid_nb, "lut_cell_nb2grid_nb", torch.int64)
    n_emb, cells, D = inp.shape
    if ci.shape[0] != cells or c2c.shape != c2g.shape or c2c.shape[0] != cells or g2g.shape[0] != n_emb:
        raise RuntimeError("convolution_forward: lookup table shapes do not match the inputs")
    if w.shape != (c2c.shape[1], D) or mk.numel() < gi.shape[0] * cells:
        raise RuntimeError("convolution_forward: weights must be (window taps, channels) and masks cover every cell")
    out = torch.empty_like(inp)
    with torch.cuda.device(dev):
        _check(_lib.ashb_conv_forward(
            _dtype_code(inp), inp.data_ptr(), w.data_ptr(), mk.data_ptr(), gi.data_ptr(), ci.data_ptr(),
            g2g.data_ptr(), c2c.data_ptr(), c2g.data_ptr(), out.data_ptr(), 1, gi.shape[0], n_emb, cells, D,
            c2c.shape[1], g2g.shape[1], _stream(dev)))
    return out


def _rays(hashmap, ray_origins, ray_directions):
    if not isinstance(hashmap, HashMap):
        raise RuntimeError("hashmap is not a GPU hashmap of type <int, 3>, ray sample not supported")
    dev = hashmap.device()
    o = _cuda(ray_origins.to(dev), "ray_origins", torch.float32)
    d = _cuda(ray_directions.to(dev), "ray_directions", torch.float32)
    if o.dim() != 2 or o.shape[1] != 3 or d.shape != o.shape:
        raise RuntimeError("ray origins and directions must both be (N, 3)")
    return dev, o, d


def _per_ray(v, n, dev, name):
    """A per-ray float32 tensor from a tensor or a scalar."""
    if not torch.is_tensor(v):
        return torch.full((n,), float(v), dtype=torch.float32, device=dev)
    v = v.to(dev, torch.float32)
    return (v.expand(n) if v.dim() == 0 else v.reshape(-1)).contiguous()


def ray_find_near_far(hashmap, ray_origins, ray_directions, bbox_min, bbox_max, t_min, t_max, t_step,
                      grid2cell_multiplier):
    """ash/src/sampler.cu:73-121.  Returns (ray_nears, ray_fars) float32 (N,)."""
    dev, o, d = _rays(hashmap, ray_origins, ray_directions)
    n = o.shape[0]
    lo = _cuda(bbox_min.to(dev, torch.float32), "bbox_min").view(-1)
    hi = _cuda(bbox_max.to(dev, torch.float32), "bbox_max").view(-1)
    nears = torch.empty(n, dtype=torch.float32, device=dev)
    fars = torch.empty(n, dtype=torch.float32, device=dev)
    _check(_lib.ashb_ray_find_near_far(
        hashmap._h, o.data_ptr(), d.data_ptr(), lo.data_ptr(), hi.data_ptr(), nears.data_ptr(), fars.data_ptr(),
        float(t_min), float(t_max), float(t_step), float(grid2cell_multiplier), n, _stream(dev)))
    return nears, fars


def ray_sample(hashmap, ray_origins, ray_directions, ray_nears, ray_fars, bbox_min, bbox_max,
               max_samples_per_ray, grid2cell_multiplier):
    """ash/src/sampler.cu:217-294.  Returns (ray_indices int64 (M,), t_nears (M,), t_fars (M,),
    inclusive prefix sum of samples per ray int64 (N,)).  The bbox is unused, as in the reference."""
    dev, o, d = _rays(hashmap, ray_origins, ray_directions)
    n = o.shape[0]
    nears = _per_ray(ray_nears, n, dev, "ray_nears")
    fars = _per_ray(ray_fars, n, dev, "ray_fars")
    counts = torch.empty(n, dtype=torch.int64, device=dev)
    st = _stream(dev)
    g2c = float(grid2cell_multiplier)
    _check(_lib.ashb_ray_sample_count(
        hashmap._h, o.data_ptr(), d.data_ptr(), nears.data_ptr(), fars.data_ptr(), counts.data_ptr(),
        int(max_samples_per_ray), g2c, n, st))
    prefix = torch.cumsum(counts, 0)
    total = int(prefix[-1].item()) if n else 0
    ray_indices = torch.empty(total, dtype=torch.int64, device=dev)
    t_nears = torch.empty(total, dtype=torch.float32, device=dev)
    t_fars = torch.empty(total, dtype=torch.float32, device=dev)
    if total:
        _check(_lib.ashb_ray_sample_fill(
            hashmap._h, o.data_ptr(), d.data_ptr(), nears.data_ptr(), fars.data_ptr(), prefix.data_ptr(),
            ray_indices.data_ptr(), t_nears.data_ptr(), t_fars.data_ptr(), int(max_samples_per_ray), g2c, n, st))
    return ray_indices, t_nears, t_fars, prefix


def _host_floats(values, n):
    """A C float[n] from a flat or nested sequence / array (row major)."""
    flat = []
    for v in values:
        flat.extend(v) if hasattr(v, "__len__") else flat.append(v)
    return (_f32 * n)(*[float(v) for v in flat[:n]])


def tsdf_touch(hashmap, depth, intrinsic, cam_to_world, depth_max, cell_size, origin, grid_dim, dilation,
               grid_coords, touched, stamp, bound_lo=None, bound_hi=None, touched_list=None, touched_count=None):
    """Allocate and stamp the blocks seen by a depth frame (no counterpart in the reference's
    native module; replaces the allocation half of demo/rgbd_fusion.py:199-224).
    ``intrinsic`` (3,3), ``cam_to_world`` (>=3,4) and ``origin`` (3,) are host values."""
    dev = hashmap.device()
    depth = _cuda(depth, "depth", torch.float32)
    if depth.dim() != 2 or grid_coords.dtype != torch.int32 or touched.dtype != torch.int32:
        raise RuntimeError("depth must be (H, W); grid_coords and touched must be int32")
    H, W = depth.shape
    K = _host_floats([intrinsic[i][j] for i in range(3) for j in range(3)], 9)
    Ei = _host_floats([cam_to_world[i][j] for i in range(3) for j in range(4)], 12)
    org = _host_floats(origin, 3)
    lo = (_c.c_int32 * 3)(*bound_lo) if bound_lo is not None else None
    hi = (_c.c_int32 * 3)(*bound_hi) if bound_hi is not None else None
    _check(_lib.ashb_tsdf_touch(
        hashmap._h, depth.data_ptr(), H, W, K, Ei, float(depth_max), float(cell_size), org, int(grid_dim),
        int(dilation), lo, hi, grid_coords.data_ptr(), touched.data_ptr(), int(stamp),
        touched_list.data_ptr() if touched_list is not None else None,
        touched_count.data_ptr() if touched_count is not None else None, _stream(dev)))


def tsdf_integrate(embeddings, grid_dim, grid_coords, touched, stamp, depth, color, intrinsic, world_to_cam,
                   depth_max, cell_size, origin, trunc, sdf_channel=0, rgb_channel=1, weight_channel=4,
                   counter=None, touched_list=None, touched_count=None):
    """Fuse a frame into every stamped block in place (replaces demo/rgbd_fusion.py:226-254)."""
    emb = embeddings
    if not emb.is_cuda or emb.dtype != torch.float32 or not emb.is_contiguous() or emb.dim() != 3:
        raise RuntimeError("embeddings must be a contiguous float32 CUDA tensor (blocks, cells, channels)")
    depth = _cuda(depth, "depth", torch.float32)
    color = _cuda(color, "color", torch.float32)
    H, W = depth.shape
    if color.shape != (H, W, 3):
        raise RuntimeError("color must be (H, W, 3)")
    K = _host_floats([intrinsic[i][j] for i in range(3) for j in range(3)], 9)
    E = _host_floats([world_to_cam[i][j] for i in range(3) for j in range(4)], 12)
    org = _host_floats(origin, 3)
    with torch.cuda.device(emb.device):
        _check(_lib.ashb_tsdf_integrate(
            emb.data_ptr(), emb.shape[0], int(grid_dim), emb.shape[2], grid_coords.data_ptr(), touched.data_ptr(),
            int(stamp), depth.data_ptr(), color.data_ptr(), H, W, K, E, float(depth_max), float(cell_size), org,
            float(trunc), int(sdf_channel), int(rgb_channel), int(weight_channel),
            counter.data_ptr() if counter is not None else None,
            touched_list.data_ptr() if touched_list is not None else None,
            touched_count.data_ptr() if touched_count is not None else None, _stream(emb.device)))


def tsdf_fuse_frame(hashmap, embeddings, grid_dim, depth, color, K9, E12, Ei12, depth_max, cell_size, origin3, dilation,
                    trunc, grid_coords, touched, stamp, touched_list, touched_count, lo3=None, hi3=None, counter=None,
                    sdf_channel=0, rgb_channel=1, weight_channel=4):
    """``tsdf_touch`` + ``tsdf_integrate`` as ONE native call.  The camera arrays are prepared by the
    caller as C float arrays (``K9`` intrinsic row major, ``E12`` / ``Ei12`` the top three rows of world ->
    camera and camera -> world, ``origin3``; ``lo3`` / ``hi3`` C int32[3] or None), so a frame costs
    one foreign call and no conversions here.  ``depth`` (H, W), ``color`` (H, W, 3): contiguous
    float32 CUDA tensors."""
    emb = embeddings
    H, W = depth.shape
    if not (emb.is_cuda and emb.dtype == torch.float32 and emb.is_contiguous() and emb.dim() == 3):
        raise RuntimeError("embeddings must be a contiguous float32 CUDA tensor (blocks, cells, channels)")
    if not (depth.is_cuda and depth.dtype == torch.float32 and depth.is_contiguous() and color.is_cuda
            and color.dtype == torch.float32 and color.is_contiguous() and color.shape == (H, W, 3)):
        raise RuntimeError("depth (H, W) and color (H, W, 3) must be contiguous float32 CUDA tensors")
    _check(_lib.ashb_tsdf_fuse_frame(
        hashmap._h, emb.data_ptr(), emb.shape[0], int(grid_dim), emb.shape[2], depth.data_ptr(), color.data_ptr(), H, W,
        K9, E12, Ei12, float(depth_max), float(cell_size), origin3, int(dilation), lo3, hi3, float(trunc),
        int(sdf_channel), int(rgb_channel), int(weight_channel), grid_coords.data_ptr(), touched.data_ptr(), int(stamp),
        touched_list.data_ptr(), touched_count.data_ptr(), counter.data_ptr() if counter is not None else None,
        _stream(emb.device)))


def tsdf_fuse_frames(hashmap, embeddings, grid_dim, depths, colors, K, E, Ei, depth_max, cell_size, origin3, dilation,
                     trunc, grid_coords, touched, first_stamp, touched_list, touched_count, lo3=None, hi3=None,
                     counter=None, sdf_channel=0, rgb_channel=1, weight_channel=4):
    """A sequence of equally sized frames in ONE native call: ``depths`` / ``colors`` lists of contiguous
    float32 CUDA tensors (H, W) / (H, W, 3); ``K`` (n, 3, 3), ``E`` and ``Ei`` (n, >=3, 4) float64 numpy arrays
    (intrinsics, world -> camera, camera -> world).  When ``touched_list`` holds two lists (2 x num_embeddings
    entries) and ``touched_count`` two counters, the allocation pass of every frame overlaps the fusion of
    the frame before it."""
    import numpy as np

    n = len(depths)
    if n == 0:
        return
    emb = embeddings
    H, W = depths[0].shape
    for d, c in zip(depths, colors):
        if not (d.is_cuda and d.dtype == torch.float32 and d.is_contiguous() and d.shape == (H, W) and c.is_cuda
                and c.dtype == torch.float32 and c.is_contiguous() and c.shape == (H, W, 3)):
            raise RuntimeError("every depth (H, W) / color (H, W, 3) must be a contiguous float32 CUDA tensor of one size")
    dp = (_vp * n)(*[d.data_ptr() for d in depths])
    cp = (_vp * n)(*[c.data_ptr() for c in colors])
    k = np.ascontiguousarray(np.asarray(K, np.float64).reshape(n, 9), dtype=np.float32)
    e = np.ascontiguousarray(np.asarray(E, np.float64)[:, :3, :].reshape(n, 12), dtype=np.float32)
    ei = np.ascontiguousarray(np.asarray(Ei, np.float64)[:, :3, :].reshape(n, 12), dtype=np.float32)
    _check(_lib.ashb_tsdf_fuse_frames(
        hashmap._h, emb.data_ptr(), emb.shape[0], int(grid_dim), emb.shape[2], n, dp, cp, H, W, k.ctypes.data,
        e.ctypes.data, ei.ctypes.data, float(depth_max), float(cell_size), origin3, int(dilation), lo3, hi3, float(trunc),
        int(sdf_channel), int(rgb_channel), int(weight_channel), grid_coords.data_ptr(), touched.data_ptr(),
        int(first_stamp), touched_list.data_ptr(), touched_count.data_ptr(),
        int(touched_list.numel() >= 2 * emb.shape[0] and touched_count.numel() >= 2),
        counter.data_ptr() if counter is not None else None, _stream(emb.device)))


def tsdf_copy_timeouts(device=None) -> int:
    """Waits of the fusion kernel's bulk copies that ran out on ``device`` since the library was loaded
    (0 in any healthy run).  Synchronises with the device."""
    out = _c.c_uint(0)
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        _check(_lib.ashb_tsdf_copy_timeouts(_c.byref(out)))
    return int(out.value)


def tsdf_fuse_frame_static(hashmap, embeddings, grid_dim, depth, color, intrinsic, world_to_cam, cam_to_world,
                           depth_max, cell_size, origin, dilation, trunc, bound_lo=None, bound_hi=None,
                           sdf_channel=0, rgb_channel=1, weight_channel=4):
    """One fusion step without any allocation, on this side or in the library.

    For callers that cannot allocate device memory while running (all memory reserved up
    front, or an allocation would stall the device): the per-block scratch that
    ``tsdf_touch`` / ``tsdf_integrate`` take as tensors lives in a fixed array inside the
    library instead, so grids are limited to ``_lib.ashb_tsdf_static_max_blocks()`` blocks.
    ``depth`` (H, W) and ``color`` (H, W, 3) must already be contiguous float32 CUDA tensors:
    nothing is copied or converted here.  Calls share the library's array; do not let two of
    them overlap on the GPU.  Make the first call on a device outside stream capture.
    """
    emb = embeddings
    if not (emb.is_cuda and emb.dtype == torch.float32 and emb.is_contiguous() and emb.dim() == 3):
        raise RuntimeError("embeddings must be a contiguous float32 CUDA tensor (blocks, cells, channels)")
    for name, t in (("depth", depth), ("color", color)):
        if not (t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()):
            raise RuntimeError(f"{name} must be a contiguous float32 CUDA tensor (nothing is converted here)")
    H, W = depth.shape
    if color.shape != (H, W, 3):
        raise RuntimeError("color must be (H, W, 3)")
    K = _host_floats([intrinsic[i][j] for i in range(3) for j in range(3)], 9)
    E = _host_floats([world_to_cam[i][j] for i in range(3) for j in range(4)], 12)
    Ei = _host_floats([cam_to_world[i][j] for i in range(3) for j in range(4)], 12)
    org = _host_floats(origin, 3)
    lo = (_c.c_int32 * 3)(*bound_lo) if bound_lo is not None else None
    hi = (_c.c_int32 * 3)(*bound_hi) if bound_hi is not None else None
    _check(_lib.ashb_tsdf_fuse_frame_static(
        hashmap._h, emb.data_ptr(), emb.shape[0], int(grid_dim), emb.shape[2], depth.data_ptr(), color.data_ptr(),
        H, W, K, E, Ei, float(depth_max), float(cell_size), org, int(dilation), lo, hi, float(trunc),
        int(sdf_channel), int(rgb_channel), int(weight_channel), _stream(hashmap.device())))


# ---------------------------------------------------------------------------------------------
# Fused grid query: additions with no counterpart in the reference's native module.  They do in
# one launch what SparseDenseGrid.forward does with ~15 torch launches + find + query_forward.

def grid_build_neighbor_lut(hashmap, num_embeddings, with_coords=False):
    """int32 (num_embeddings, 8) block-neighbour table (and optionally the (num_embeddings, 3)
    block coordinates), -1 for absent; the content of ash/grid.py:566-617 for radius 1, one-sided."""
    dev = hashmap.device()
    lut = torch.empty((num_embeddings, 8), dtype=torch.int32, device=dev)
    coords = torch.empty((num_embeddings, 3), dtype=torch.int32, device=dev) if with_coords else None
    _check(_lib.ashb_grid_build_neighbor_lut(
        hashmap._h, lut.data_ptr(), coords.data_ptr() if with_coords else None, num_embeddings, _stream(dev)))
    return (lut, coords) if with_coords else lut


def _fused_args(hashmap, embeddings, x, nb_lut):
    emb = _cuda(embeddings, "embeddings")
    if emb.dim() != 3 or emb.device != hashmap.device():
        raise RuntimeError("embeddings must be (num_embeddings, cells_per_grid, embedding_dim) on the map's device")
    x = _cuda(x, "x", torch.float32)
    if x.dim() != 2 or x.shape[1] != 3:
        raise RuntimeError("x must be (N, 3)")
    nb_lut = _cuda(nb_lut, "nb_lut", torch.int32)
    if nb_lut.shape != (emb.shape[0], 8):
        raise RuntimeError("nb_lut must be int32 (num_embeddings, 8)")
    return emb, x, nb_lut


def grid_query_forward(hashmap, embeddings, x, cell_size, origin, grid_dim, nb_lut, interpolation):
    """Returns (features (N, D), masks bool (N,), block_idx int32 (N,))."""
    emb, x, nb_lut = _fused_args(hashmap, embeddings, x, nb_lut)
    n, dev = x.shape[0], emb.device
    out = torch.empty((n, emb.shape[2]), dtype=emb.dtype, device=dev)
    masks = torch.empty(n, dtype=torch.bool, device=dev)
    bidx = torch.empty(n, dtype=torch.int32, device=dev)
    _check(_lib.ashb_grid_query_forward(
        hashmap._h, _dtype_code(emb), _interp_code(interpolation), emb.data_ptr(), x.data_ptr(), float(cell_size),
        _host_floats(origin, 3), int(grid_dim), nb_lut.data_ptr(), out.data_ptr(), masks.data_ptr(), bidx.data_ptr(),
        n, emb.shape[0], emb.shape[2], _stream(dev)))
    return out, masks, bidx


def grid_query_backward(hashmap, z, embeddings, x, cell_size, origin, grid_dim, nb_lut, block_idx, interpolation,
                        grad_embeddings_out=None, need_grad_x=True, need_grad_embeddings=True):
    """Returns (grad_embeddings, grad_x (N, 3) in the embeddings' dtype); either is None when not needed."""
    emb, x, nb_lut = _fused_args(hashmap, embeddings, x, nb_lut)
    n, dev = x.shape[0], emb.device
    z = _cuda(z, "z", emb.dtype)
    if z.shape != (n, emb.shape[2]):
        raise RuntimeError("z must be (num_queries, embedding_dim)")
    if not need_grad_embeddings:
        grad_emb, zero = None, 0
    elif grad_embeddings_out is None:
        grad_emb, zero = torch.empty_like(emb), 1
    else:
        grad_emb, zero = grad_embeddings_out, 0
        if grad_emb.shape != emb.shape or grad_emb.dtype != emb.dtype or not grad_emb.is_contiguous():
            raise RuntimeError("grad_embeddings_out must match embeddings")
    if grad_emb is None and not need_grad_x:
        return None, None
    grad_x = torch.empty((n, 3), dtype=emb.dtype, device=dev) if need_grad_x else None
    bidx = _cuda(block_idx, "block_idx", torch.int32) if block_idx is not None else None
    _check(_lib.ashb_grid_query_backward(
        hashmap._h, _dtype_code(emb), _interp_code(interpolation), z.data_ptr(), emb.data_ptr(), x.data_ptr(),
        float(cell_size), _host_floats(origin, 3), int(grid_dim), nb_lut.data_ptr(),
        bidx.data_ptr() if bidx is not None else None, grad_emb.data_ptr() if grad_emb is not None else None,
        grad_x.data_ptr() if need_grad_x else None, zero, n, emb.shape[0], emb.shape[2], _stream(dev)))
    return grad_emb, grad_x


def grid_query_backward_backward(hashmap, grad_grad_x, z, embeddings, x, cell_size, origin, grid_dim, nb_lut,
                                 block_idx, interpolation, grad_embeddings_out=None):
    """Returns (grad_z, grad_embeddings); the gradient w.r.t. x is dropped as in the reference."""
    emb, x, nb_lut = _fused_args(hashmap, embeddings, x, nb_lut)
    n, dev = x.shape[0], emb.device
    z = _cuda(z, "z", emb.dtype)
    ggx = _cuda(grad_grad_x, "grad_grad_x", emb.dtype)
    if z.shape != (n, emb.shape[2]) or ggx.shape != (n, 3):
        raise RuntimeError("z must be (num_queries, embedding_dim) and grad_grad_x (num_queries, 3)")
    if grad_embeddings_out is None:
        grad_emb, zero = torch.empty_like(emb), 1
    else:
        grad_emb, zero = grad_embeddings_out, 0
    grad_z = torch.empty_like(z)
    bidx = _cuda(block_idx, "block_idx", torch.int32) if block_idx is not None else None
    _check(_lib.ashb_grid_query_backward_backward(
        hashmap._h, _dtype_code(emb), _interp_code(interpolation), ggx.data_ptr(), z.data_ptr(), emb.data_ptr(),
        x.data_ptr(), float(cell_size), _host_floats(origin, 3), int(grid_dim), nb_lut.data_ptr(),
        bidx.data_ptr() if bidx is not None else None, grad_z.data_ptr(), grad_emb.data_ptr(), zero, n, emb.shape[0],
        emb.shape[2], _stream(dev)))
    return grad_z, grad_emb


def grid_query_backward_rows(hashmap, z, embeddings, x, cell_size, origin, grid_dim, nb_lut, block_idx, interpolation,
                             need_grad_x=True, grad_grad_x=None):
    """The backward passes with the embedding gradient as a ROW LIST: returns ``(idx int64 (2, 8N),
    rows (8N, D), side)``; record ``8 q + c`` is corner ``c`` of query ``q``, ``idx[0]`` its block
    index, ``idx[1]`` its cell index.  ``side`` is grad_x (N, 3) (None unless ``need_grad_x``) for the
    first-order pass, or grad_z (N, D) when ``grad_grad_x`` is given (the double backward)."""
    emb, x, nb_lut = _fused_args(hashmap, embeddings, x, nb_lut)
    n, dev, D = x.shape[0], emb.device, emb.shape[2]
    z = _cuda(z, "z", emb.dtype)
    if z.shape != (n, D):
        raise RuntimeError("z must be (num_queries, embedding_dim)")
    second = grad_grad_x is not None
    ggx = None
    if second:
        ggx = _cuda(grad_grad_x, "grad_grad_x", emb.dtype)
        if ggx.shape != (n, 3):
            raise RuntimeError("grad_grad_x must be (num_queries, 3)")
        side = torch.empty_like(z)
    else:
        side = torch.empty((n, 3), dtype=emb.dtype, device=dev) if need_grad_x else None
    idx = torch.empty((2, 8 * n), dtype=torch.int64, device=dev)
    rows = torch.empty((8 * n, D), dtype=emb.dtype, device=dev)
    bidx = _cuda(block_idx, "block_idx", torch.int32) if block_idx is not None else None
    _check(_lib.ashb_grid_query_backward_rows(
        hashmap._h, _dtype_code(emb), _interp_code(interpolation), int(second), ggx.data_ptr() if second else None,
        z.data_ptr(), emb.data_ptr(), x.data_ptr(), float(cell_size), _host_floats(origin, 3), int(grid_dim),
        nb_lut.data_ptr(), bidx.data_ptr() if bidx is not None else None, idx.data_ptr(), rows.data_ptr(),
        side.data_ptr() if side is not None else None, n, emb.shape[0], D, _stream(dev)))
    return idx, rows, side


def rows_scatter_add(dst, idx, rows, alpha=1.0):
    """``dst[idx[0][r], idx[1][r], :] += alpha * rows[r]`` for a row list; ``dst`` is a contiguous
    (num_embeddings, cells_per_grid, D) tensor: a gradient buffer, or the parameters with ``alpha =
    -learning_rate``."""
    dst = _cuda(dst, "dst")
    if dst.dim() != 3 or not dst.is_contiguous():
        raise RuntimeError("dst must be a contiguous (num_embeddings, cells_per_grid, embedding_dim) tensor")
    idx = _cuda(idx, "idx", torch.int64)
    rows = _cuda(rows, "rows", dst.dtype)
    m = rows.shape[0]
    if idx.shape != (2, m) or rows.shape != (m, dst.shape[2]):
        raise RuntimeError("idx must be (2, m) and rows (m, embedding_dim)")
    with torch.cuda.device(dst.device):
        _check(_lib.ashb_rows_scatter_add(_dtype_code(dst), dst.data_ptr(), idx.data_ptr(), rows.data_ptr(), m,
                                          dst.shape[0], dst.shape[1], dst.shape[2], float(alpha), _stream(dst.device)))


def convolution_forward_tiled(inputs, weights, grid_indices, lut_grid_nb27, grid_dim, radius):
    """Shared-memory tiled form of ``convolution_forward`` for a two-sided window of ``radius`` <=
    ``grid_dim`` cells (float32).  ``weights`` ((2R+1)^3, D), ``lut_grid_nb27`` int64
    (num_embeddings, 27); the per-cell tables are implied.  No counterpart in the reference."""
    inp = _cuda(inputs, "inputs", torch.float32)
    w = _cuda(weights, "weights", torch.float32)
    gi = _cuda(grid_indices, "grid_indices", torch.int64).view(-1)
    g27 = _cuda(lut_grid_nb27, "lut_grid_nb27", torch.int64)
    n_emb, cells, D = inp.shape
    S = 2 * int(radius) + 1
    if cells != int(grid_dim) ** 3 or w.shape != (S**3, D) or g27.shape != (n_emb, 27):
        raise RuntimeError("convolution_forward_tiled: shapes do not match (grid_dim, radius)")
    out = torch.empty_like(inp)
    with torch.cuda.device(inp.device):
        _check(_lib.ashb_conv_forward_tiled(
            inp.data_ptr(), w.data_ptr(), gi.data_ptr(), g27.data_ptr(), out.data_ptr(), 1, gi.shape[0], n_emb,
            int(grid_dim), int(radius), D, _stream(inp.device)))
    return out


def convolution_forward_separable(inputs, weights_1d, grid_indices, lut_grid_nb27, grid_dim, radius):
    """``convolution_forward_tiled`` for a separable window: ``weights_1d`` (3, 2R+1, D) float32 holds
    the x, y and z factors per channel.  No counterpart in the reference."""
    inp = _cuda(inputs, "inputs", torch.float32)
    w = _cuda(weights_1d, "weights_1d", torch.float32)
    gi = _cuda(grid_indices, "grid_indices", torch.int64).view(-1)
    g27 = _cuda(lut_grid_nb27, "lut_grid_nb27", torch.int64)
    n_emb, cells, D = inp.shape
    S = 2 * int(radius) + 1
    if cells != int(grid_dim) ** 3 or w.shape != (3, S, D) or g27.shape != (n_emb, 27):
        raise RuntimeError("convolution_forward_separable: shapes do not match (grid_dim, radius)")
    out = torch.empty_like(inp)
    with torch.cuda.device(inp.device):
        _check(_lib.ashb_conv_forward_separable(
            inp.data_ptr(), w.data_ptr(), gi.data_ptr(), g27.data_ptr(), out.data_ptr(), 1, gi.shape[0], n_emb,
            int(grid_dim), int(radius), D, _stream(inp.device)))
    return out


def grid_spatial_init(hashmap, points, cell_size, origin, grid_dim, dilation, bidirectional, grid_coords, touched,
                      stamp, touched_list, touched_count, bound_lo=None, bound_hi=None):
    """Allocate the blocks around ``points`` (N, 3) float32 world positions in one launch and
    leave their compact list in ``touched_list[:touched_count]``; replaces the temporary hash
    set + insert + find sequence of ash/grid.py:121-159.  No counterpart in the reference's
    native module."""
    dev = hashmap.device()
    pts = _cuda(points, "points", torch.float32)
    if pts.dim() != 2 or pts.shape[1] != 3:
        raise RuntimeError("points must be (N, 3)")
    lo = (_c.c_int32 * 3)(*bound_lo) if bound_lo is not None else None
    hi = (_c.c_int32 * 3)(*bound_hi) if bound_hi is not None else None
    _check(_lib.ashb_grid_spatial_init(
        hashmap._h, pts.data_ptr(), pts.shape[0], float(cell_size), _host_floats(origin, 3), int(grid_dim),
        int(dilation), int(bool(bidirectional)), lo, hi, grid_coords.data_ptr(), touched.data_ptr(), int(stamp),
        touched_list.data_ptr(), touched_count.data_ptr(), _stream(dev)))


def route_by_owner(keys, world):
    """Group ``keys`` int32 (N, dim) by owner rank for the key-hash-partitioned map: returns
    (keys grouped by owner, perm int64 (N,) = source row of every grouped row, send counts list).
    No counterpart in the reference (single-GPU)."""
    keys = _cuda(keys, "keys", torch.int32)
    n, dim = keys.shape
    out = torch.empty_like(keys)
    perm = torch.empty(n, dtype=torch.int64, device=keys.device)
    scratch = torch.empty(128, dtype=torch.int64, device=keys.device)
    counts = (_i64 * int(world))()
    with torch.cuda.device(keys.device):
        _check(_lib.ashb_route_by_owner(keys.data_ptr(), n, dim, int(world), out.data_ptr(), perm.data_ptr(), counts,
                                        scratch.data_ptr(), _stream(keys.device)))
    return out, perm, list(counts)


# ---------------------------------------------------------------------------------------------
# Volume-rendering accumulation over packed ray samples (no counterpart in the reference's native
# module: its demo calls a third-party package for this step).

def render_segments(ray_indices, n_rays):
    """(seg_start, seg_end) int64 (n_rays,): sample range of every ray; ray_indices non-decreasing."""
    ri = _cuda(ray_indices, "ray_indices", torch.int64).view(-1)
    start = torch.empty(n_rays, dtype=torch.int64, device=ri.device)
    end = torch.empty(n_rays, dtype=torch.int64, device=ri.device)
    with torch.cuda.device(ri.device):
        _check(_lib.ashb_render_segments(ri.data_ptr(), ri.shape[0], n_rays, start.data_ptr(), end.data_ptr(),
                                         _stream(ri.device)))
    return start, end


def _f32_flat(t, name):
    return _cuda(t, name, torch.float32).reshape(-1)


def _samples_by_channels(values, m):
    """values as (m, C) float32, or None."""
    if values is None:
        return None
    v = _cuda(values, "values", torch.float32)
    channels = v.shape[-1] if v.dim() > 1 else 1
    return v.reshape(m, channels)


def render_weights_forward(t_starts, t_ends, sigmas, seg_start, seg_end):
    ts, te, sg = _f32_flat(t_starts, "t_starts"), _f32_flat(t_ends, "t_ends"), _f32_flat(sigmas, "sigmas")
    if not (ts.shape == te.shape == sg.shape):
        raise RuntimeError("t_starts, t_ends and sigmas must have one value per sample")
    w = torch.empty_like(sg)
    with torch.cuda.device(sg.device):
        _check(_lib.ashb_render_weights_forward(ts.data_ptr(), te.data_ptr(), sg.data_ptr(), seg_start.data_ptr(),
                                                seg_end.data_ptr(), seg_start.shape[0], w.data_ptr(), _stream(sg.device)))
    return w


def render_weights_backward(t_starts, t_ends, sigmas, weights, grad_weights, seg_start, seg_end):
    ts, te, sg = _f32_flat(t_starts, "t_starts"), _f32_flat(t_ends, "t_ends"), _f32_flat(sigmas, "sigmas")
    w, gw = _f32_flat(weights, "weights"), _f32_flat(grad_weights, "grad_weights")
    gs = torch.empty_like(sg)
    with torch.cuda.device(sg.device):
        _check(_lib.ashb_render_weights_backward(
            ts.data_ptr(), te.data_ptr(), sg.data_ptr(), w.data_ptr(), gw.data_ptr(), seg_start.data_ptr(),
            seg_end.data_ptr(), seg_start.shape[0], gs.data_ptr(), _stream(sg.device)))
    return gs


def render_accumulate_forward(weights, values, seg_start, seg_end):
    w = _f32_flat(weights, "weights")
    v = _samples_by_channels(values, w.shape[0])
    C = v.shape[1] if v is not None else 1
    out = torch.empty((seg_start.shape[0], C), dtype=torch.float32, device=w.device)
    with torch.cuda.device(w.device):
        _check(_lib.ashb_render_accumulate_forward(
            w.data_ptr(), v.data_ptr() if v is not None else None, C, seg_start.data_ptr(), seg_end.data_ptr(),
            seg_start.shape[0], out.data_ptr(), _stream(w.device)))
    return out


def render_accumulate_backward(weights, values, grad_out, ray_indices, n_rays, need_weights=True, need_values=True):
    w = _f32_flat(weights, "weights")
    m = w.shape[0]
    v = _samples_by_channels(values, m)
    C = v.shape[1] if v is not None else 1
    go = _cuda(grad_out, "grad_out", torch.float32).reshape(n_rays, C)
    ri = _cuda(ray_indices, "ray_indices", torch.int64).view(-1)
    gw = torch.empty(m, dtype=torch.float32, device=w.device) if need_weights else None
    gv = torch.empty((m, C), dtype=torch.float32, device=w.device) if (need_values and v is not None) else None
    with torch.cuda.device(w.device):
        _check(_lib.ashb_render_accumulate_backward(
            w.data_ptr(), v.data_ptr() if v is not None else None, go.data_ptr(), ri.data_ptr(), m, n_rays, C,
            gw.data_ptr() if gw is not None else None, gv.data_ptr() if gv is not None else None, _stream(w.device)))
    return gw, gv


def isosurface_extraction(sdfs, weights, grid_indices, grid_coords_table, lut_grid_nb2grid_idx, cell_coords_table,
                          lut_cell_nb2cell_idx, lut_cell_nb2grid_nb, grid_dim, iso_value, weight_thr):
    """ash/src/grid.cu:534-604: (n, 3) float32 zero crossings along +x/+y/+z cell edges, in cell units."""
    sd = _cuda(sdfs, "sdfs", torch.float32)
    n_emb = lut_grid_nb2grid_idx.shape[0]
    sd = sd.reshape(n_emb, -1)
    wt = _cuda(weights, "weights", torch.float32).reshape(sd.shape)
    dev = sd.device
    gi = _cuda(grid_indices, "grid_indices", torch.int64).view(-1)
    gct = _cuda(grid_coords_table, "grid_coords_table", torch.int32)
    cct = _cuda(cell_coords_table, "cell_coords_table", torch.int32)
    g2g = _cuda(lut_grid_nb2grid_idx, "lut_grid_nb2grid_idx", torch.int64)
    c2c = _cuda(lut_cell_nb2cell_idx, "lut_cell_nb2cell_idx", torch.int64)
    c2g = _cuda(lut_cell_nb2grid_nb, "lut_cell_nb2grid_nb", torch.int64)
    cells = sd.shape[1]
    if gct.shape != (n_emb, 3) or cct.shape != (cells, 3) or c2c.shape != (cells, 8) or c2g.shape != (cells, 8):
        raise RuntimeError("isosurface_extraction: table shapes do not match sdfs")
    cursor = torch.empty(1, dtype=torch.int64, device=dev)
    n = _i64()

    def run(out, max_out):
        with torch.cuda.device(dev):
            _check(_lib.ashb_isosurface_extraction(
                sd.data_ptr(), wt.data_ptr(), gi.data_ptr(), gct.data_ptr(), g2g.data_ptr(), cct.data_ptr(),
                c2c.data_ptr(), c2g.data_ptr(), out.data_ptr() if out is not None else None, max_out, _c.byref(n),
                cursor.data_ptr(), float(iso_value), float(weight_thr), int(grid_dim), cells, n_emb, gi.shape[0],
                _stream(dev)))

    run(None, 0)
    positions = torch.empty((n.value, 3), dtype=torch.float32, device=dev)
    if n.value:
        run(positions, n.value)
    return positions


def marching_cubes(sdfs, weights, grid_indices, grid_coords_table, lut_grid_nb2grid_idx, cell_coords_table,
                   lut_cell_nb2cell_idx, lut_cell_nb2grid_nb, grid_dim, iso_value, weight_thr):
    """ash/src/grid.cu:840-946: (triangles (T, 3) int32 vertex ids, vertices (V, 3) float32 in cell
    units).  Triangle normals point towards increasing sdf; the triangulation table is this
    library's own."""
    sd = _cuda(sdfs, "sdfs", torch.float32)
    n_emb = lut_grid_nb2grid_idx.shape[0]
    sd = sd.reshape(n_emb, -1)
    wt = _cuda(weights, "weights", torch.float32).reshape(sd.shape)
    dev = sd.device
    gi = _cuda(grid_indices, "grid_indices", torch.int64).view(-1)
    gct = _cuda(grid_coords_table, "grid_coords_table", torch.int32)
    cct = _cuda(cell_coords_table, "cell_coords_table", torch.int32)
    g2g = _cuda(lut_grid_nb2grid_idx, "lut_grid_nb2grid_idx", torch.int64)
    c2c = _cuda(lut_cell_nb2cell_idx, "lut_cell_nb2cell_idx", torch.int64)
    c2g = _cuda(lut_cell_nb2grid_nb, "lut_cell_nb2grid_nb", torch.int64)
    cells = sd.shape[1]
    if gct.shape != (n_emb, 3) or cct.shape != (cells, 3) or c2c.shape != (cells, 8) or c2g.shape != (cells, 8):
        raise RuntimeError("marching_cubes: table shapes do not match sdfs")
    codes = torch.empty(max(gi.shape[0] * cells, 1), dtype=torch.uint8, device=dev)
    edge_vertex = torch.empty(n_emb * cells * 3, dtype=torch.int32, device=dev)
    counters = torch.empty(2, dtype=torch.int64, device=dev)
    nv, nt = _i64(), _i64()
    with torch.cuda.device(dev):
        _check(_lib.ashb_marching_cubes_count(
            sd.data_ptr(), wt.data_ptr(), gi.data_ptr(), g2g.data_ptr(), c2c.data_ptr(), c2g.data_ptr(), codes.data_ptr(),
            edge_vertex.data_ptr(), counters.data_ptr(), float(iso_value), float(weight_thr), cells, n_emb, gi.shape[0],
            _c.byref(nv), _c.byref(nt), _stream(dev)))
        vertices = torch.empty((nv.value, 3), dtype=torch.float32, device=dev)
        triangles = torch.empty((nt.value, 3), dtype=torch.int32, device=dev)
        _check(_lib.ashb_marching_cubes_fill(
            sd.data_ptr(), gi.data_ptr(), gct.data_ptr(), g2g.data_ptr(), cct.data_ptr(), c2c.data_ptr(), c2g.data_ptr(),
            codes.data_ptr(), edge_vertex.data_ptr(), counters.data_ptr(), vertices.data_ptr() if nv.value else None,
            nv.value, triangles.data_ptr() if nt.value else None, nt.value, float(iso_value), int(grid_dim), cells, n_emb,
            gi.shape[0], _stream(dev)))
    return triangles, vertices


def grid_zero_rows(hashmap, grad_embeddings, x, cell_size, origin, grid_dim, nb_lut, block_idx=None):
    """Zero, in ``grad_embeddings``, the corner rows the batch ``x`` touches (in place)."""
    g, x, nb_lut = _fused_args(hashmap, grad_embeddings, x, nb_lut)
    if g.data_ptr() != grad_embeddings.data_ptr():
        raise RuntimeError("grad_embeddings must be contiguous (it is modified in place)")
    bidx = _cuda(block_idx, "block_idx", torch.int32) if block_idx is not None else None
    _check(_lib.ashb_grid_zero_rows(
        hashmap._h, _dtype_code(g), g.data_ptr(), x.data_ptr(), float(cell_size), _host_floats(origin, 3),
        int(grid_dim), nb_lut.data_ptr(), bidx.data_ptr() if bidx is not None else None, x.shape[0], g.shape[0],
        g.shape[2], _stream(g.device)))


# ---------------------------------------------------------------------------------------------
# Fused ray renderer (no counterpart in the reference's native module: its demo composes this
# from ray_find_near_far, ray_sample, the grid query, autograd.grad and a third-party package).

def _ray_args(hashmap, embeddings, nb_lut, cell_size, origin, ray_o_world, ray_o_cell, ray_d, bbox_min_cell,
              bbox_max_cell, t_min_cell, t_max_cell, max_samples_per_ray, skip_missed, beta, interpolation):
    emb = _cuda(embeddings, "embeddings", torch.float32)
    if emb.dim() != 3 or emb.shape[2] < 4:
        raise RuntimeError("ray rendering needs embeddings (num_embeddings, G^3, D >= 4): signed distance + colour")
    G = round(emb.shape[1] ** (1.0 / 3.0))
    if G ** 3 != emb.shape[1]:
        raise RuntimeError("embeddings.shape[1] is not a cube")
    lut = _cuda(nb_lut, "nb_lut", torch.int32)
    ow = _cuda(ray_o_world, "ray_o_world", torch.float32)
    oc = _cuda(ray_o_cell, "ray_o_cell", torch.float32)
    d = _cuda(ray_d, "ray_d", torch.float32)
    if not (ow.shape == oc.shape == d.shape and ow.dim() == 2 and ow.shape[1] == 3):
        raise RuntimeError("ray origins and directions must be (n_rays, 3)")
    lo = _cuda(bbox_min_cell, "bbox_min", torch.float32).view(-1)
    hi = _cuda(bbox_max_cell, "bbox_max", torch.float32).view(-1)
    b = _cuda(beta, "beta", torch.float32).view(-1)
    org = (_f32 * 3)(*[float(v) for v in origin]) if origin is not None else None
    keep = (emb, lut, ow, oc, d, lo, hi, b, org)
    args = [hashmap._h, _INTERP[interpolation], emb.data_ptr(), emb.shape[0], G, emb.shape[2], lut.data_ptr(),
            float(cell_size), org, ow.data_ptr(), oc.data_ptr(), d.data_ptr(), lo.data_ptr(), hi.data_ptr(),
            float(t_min_cell), float(t_max_cell), int(max_samples_per_ray), int(bool(skip_missed)), b.data_ptr()]
    return args, keep, emb, ow.shape[0]


def render_rays_forward(hashmap, embeddings, nb_lut, cell_size, origin, ray_o_world, ray_o_cell, ray_d, bbox_min_cell,
                        bbox_max_cell, t_min_cell, t_max_cell, max_samples_per_ray, skip_missed, beta,
                        interpolation="linear"):
    """(n_rays, 16) float32 rows: rgb, depth, normal, accumulated weight, the two eikonal sums,
    sample count, near, far (columns as documented for ashb_render_rays_forward)."""
    args, keep, emb, n = _ray_args(hashmap, embeddings, nb_lut, cell_size, origin, ray_o_world, ray_o_cell, ray_d,
                                   bbox_min_cell, bbox_max_cell, t_min_cell, t_max_cell, max_samples_per_ray,
                                   skip_missed, beta, interpolation)
    out = torch.empty((n, 16), dtype=torch.float32, device=emb.device)
    with torch.cuda.device(emb.device):
        _check(_lib.ashb_render_rays_forward(*args, out.data_ptr(), n, _stream(emb.device)))
    return out


def render_rays_backward(hashmap, embeddings, nb_lut, cell_size, origin, ray_o_world, ray_o_cell, ray_d, bbox_min_cell,
                         bbox_max_cell, t_min_cell, t_max_cell, max_samples_per_ray, skip_missed, beta, out, grad_out,
                         interpolation="linear", grad_embeddings_out=None):
    """(grad_embeddings, grad_beta (1,)); adds into ``grad_embeddings_out`` when given, else into
    a fresh zero-filled tensor shaped like ``embeddings``."""
    args, keep, emb, n = _ray_args(hashmap, embeddings, nb_lut, cell_size, origin, ray_o_world, ray_o_cell, ray_d,
                                   bbox_min_cell, bbox_max_cell, t_min_cell, t_max_cell, max_samples_per_ray,
                                   skip_missed, beta, interpolation)
    out = _cuda(out, "out", torch.float32)
    go = _cuda(grad_out, "grad_out", torch.float32)
    if out.shape != (n, 16) or go.shape != (n, 16):
        raise RuntimeError("out and grad_out must be (n_rays, 16)")
    if grad_embeddings_out is None:
        ge = torch.zeros_like(emb)
    else:
        ge = grad_embeddings_out
        if not (ge.is_cuda and ge.is_contiguous() and ge.shape == emb.shape and ge.dtype == emb.dtype):
            raise RuntimeError("grad_embeddings_out must be a contiguous CUDA tensor shaped like embeddings")
    gb = torch.zeros(1, dtype=torch.float32, device=emb.device)
    with torch.cuda.device(emb.device):
        _check(_lib.ashb_render_rays_backward(*args, out.data_ptr(), go.data_ptr(), ge.data_ptr(), gb.data_ptr(), n,
                                              _stream(emb.device)))
    return ge, gb


# ---------------------------------------------------------------------------------------------
# Peer-memory transport of the partitioned map (no counterpart in the reference).  ``layout`` =
# (peer_bases_dev: address of the device array of mailbox addresses, mailbox_bytes, inbox_offset,
# counts_offset, answers_offset, region_capacity, answer_capacity).

def peer_route_keys(keys, world, rank, layout, cursor, status, where=None):
    keys = _cuda(keys, "keys", torch.int32)
    n, dim = keys.shape
    with torch.cuda.device(keys.device):
        _check(_lib.ashb_peer_route_keys(keys.data_ptr(), n, dim, int(world), int(rank), *[int(v) for v in layout],
                                         cursor.data_ptr(), where.data_ptr() if where is not None else None,
                                         status.data_ptr(), _stream(keys.device)))


def peer_unpack_answers(where, n, world, rank, layout):
    """(indices int64 (n,), masks bool (n,)) gathered from this rank's own answers section."""
    dev = where.device
    indices = torch.empty(n, dtype=torch.int64, device=dev)
    masks = torch.empty(n, dtype=torch.bool, device=dev)
    with torch.cuda.device(dev):
        _check(_lib.ashb_peer_unpack_answers(where.data_ptr(), int(n), int(world), int(rank), *[int(v) for v in layout],
                                             indices.data_ptr(), masks.data_ptr(), _stream(dev)))
    return indices, masks


def peer_find_answer(hashmap, world, rank, layout):
    dev = hashmap._device
    with torch.cuda.device(dev):
        _check(_lib.ashb_peer_find_answer(hashmap._h, int(world), int(rank), *[int(v) for v in layout], _stream(dev)))


def peer_update(hashmap, erase, world, rank, layout):
    """Insert-if-absent (or erase) the keys other ranks routed into this rank's inbox."""
    dev = hashmap._device
    with torch.cuda.device(dev):
        _check(_lib.ashb_peer_update(hashmap._h, int(bool(erase)), int(world), int(rank), *[int(v) for v in layout],
                                     _stream(dev)))


# ---------------------------------------------------------------------------------------------
# Grid query over an embedding table sharded by block over the GPUs of one box (peer memory).
# ``emb_bases`` / ``grad_bases``: addresses of device arrays [world] holding every shard's address
# as mapped into this GPU.  No counterpart in the reference.

def grid_query_forward_sharded(hashmap, emb_bases, world, n_emb, embedding_dim, x, cell_size, origin, grid_dim, nb_lut,
                               interpolation, keep_rows=False):
    """Returns (features (N, D) float32, masks bool (N,), block_idx int32 (N,), rows): ``rows`` is
    the local copy (N, 8, D) of the fetched corner rows when ``keep_rows``, else None."""
    x = _cuda(x, "x", torch.float32)
    nb_lut = _cuda(nb_lut, "nb_lut", torch.int32)
    if x.dim() != 2 or x.shape[1] != 3 or nb_lut.shape != (n_emb, 8):
        raise RuntimeError("x must be (N, 3) and nb_lut int32 (num_embeddings, 8)")
    n, dev = x.shape[0], x.device
    out = torch.empty((n, embedding_dim), dtype=torch.float32, device=dev)
    masks = torch.empty(n, dtype=torch.bool, device=dev)
    bidx = torch.empty(n, dtype=torch.int32, device=dev)
    # rows of queries that resolve to nothing are never written -- and never read back either
    rows = torch.empty((n, 8, embedding_dim), dtype=torch.float32, device=dev) if keep_rows else None
    with torch.cuda.device(dev):
        _check(_lib.ashb_grid_query_forward_sharded(
            hashmap._h, _interp_code(interpolation), int(emb_bases), int(world), x.data_ptr(), float(cell_size),
            _host_floats(origin, 3), int(grid_dim), nb_lut.data_ptr(), out.data_ptr(), masks.data_ptr(), bidx.data_ptr(),
            rows.data_ptr() if keep_rows else None, n, int(n_emb), int(embedding_dim), _stream(dev)))
    return out, masks, bidx, rows


def grid_query_backward_sharded(hashmap, z, emb_bases, grad_bases, world, n_emb, x, cell_size, origin, grid_dim, nb_lut,
                                block_idx, interpolation, need_grad_x=True, need_grad_embeddings=True, rows=None):
    """Adds the embedding gradient into the owners' gradient shards (unless not needed); returns
    grad_x (N, 3) or None."""
    x = _cuda(x, "x", torch.float32)
    z = _cuda(z, "z", torch.float32)
    nb_lut = _cuda(nb_lut, "nb_lut", torch.int32)
    bidx = _cuda(block_idx, "block_idx", torch.int32)
    n, dev = x.shape[0], x.device
    if z.dim() != 2 or z.shape[0] != n or bidx.shape != (n,) or nb_lut.shape != (n_emb, 8):
        raise RuntimeError("z must be (N, D), block_idx (N,), nb_lut int32 (num_embeddings, 8)")
    if not need_grad_x and not need_grad_embeddings:
        return None
    grad_x = torch.empty((n, 3), dtype=torch.float32, device=dev) if need_grad_x else None
    with torch.cuda.device(dev):
        _check(_lib.ashb_grid_query_backward_sharded(
            hashmap._h, _interp_code(interpolation), z.data_ptr(), int(emb_bases), int(grad_bases), int(world),
            x.data_ptr(), float(cell_size), _host_floats(origin, 3), int(grid_dim), nb_lut.data_ptr(), bidx.data_ptr(),
            grad_x.data_ptr() if need_grad_x else None, int(bool(need_grad_embeddings)),
            rows.data_ptr() if rows is not None else None, n, int(n_emb), z.shape[1], _stream(dev)))
    return grad_x


def grid_query_backward_backward_sharded(hashmap, grad_grad_x, z, emb_bases, grad_bases, world, n_emb, x, cell_size,
                                         origin, grid_dim, nb_lut, block_idx, interpolation, rows=None):
    """Adds the second-order embedding gradient into the owners' gradient shards; returns grad_z (N, D)."""
    x = _cuda(x, "x", torch.float32)
    z = _cuda(z, "z", torch.float32)
    ggx = _cuda(grad_grad_x, "grad_grad_x", torch.float32)
    nb_lut = _cuda(nb_lut, "nb_lut", torch.int32)
    bidx = _cuda(block_idx, "block_idx", torch.int32)
    n, dev = x.shape[0], x.device
    if z.dim() != 2 or z.shape[0] != n or ggx.shape != (n, 3) or bidx.shape != (n,) or nb_lut.shape != (n_emb, 8):
        raise RuntimeError("z must be (N, D), grad_grad_x (N, 3), block_idx (N,), nb_lut int32 (num_embeddings, 8)")
    grad_z = torch.empty_like(z)
    with torch.cuda.device(dev):
        _check(_lib.ashb_grid_query_backward_backward_sharded(
            hashmap._h, _interp_code(interpolation), ggx.data_ptr(), z.data_ptr(), int(emb_bases), int(grad_bases),
            int(world), x.data_ptr(), float(cell_size), _host_floats(origin, 3), int(grid_dim), nb_lut.data_ptr(),
            bidx.data_ptr(), grad_z.data_ptr(), rows.data_ptr() if rows is not None else None, n, int(n_emb), z.shape[1],
            _stream(dev)))
    return grad_z


def _ray_grid_args(hashmap, embeddings, nb_lut, cell_size, origin, interpolation):
    emb = _cuda(embeddings, "embeddings", torch.float32)
    if emb.dim() != 3 or emb.shape[2] < 4:
        raise RuntimeError("ray rendering needs embeddings (num_embeddings, G^3, D >= 4): signed distance + colour")
    G = round(emb.shape[1] ** (1.0 / 3.0))
    if G ** 3 != emb.shape[1]:
        raise RuntimeError("embeddings.shape[1] is not a cube")
    lut = _cuda(nb_lut, "nb_lut", torch.int32)
    org = (_f32 * 3)(*[float(v) for v in origin]) if origin is not None else None
    args = [hashmap._h, _INTERP[interpolation], emb.data_ptr(), emb.shape[0], G, emb.shape[2], lut.data_ptr(),
            float(cell_size), org]
    return args, (emb, lut, org)


def render_rays_intervals(hashmap, embeddings, nb_lut, cell_size, origin, ray_o_cell, ray_d, bbox_min_cell,
                          bbox_max_cell, t_min_cell, t_max_cell, max_samples_per_ray, skip_missed,
                          interpolation="linear"):
    """March every ray once: (intervals (n, stride, 2) float32 in cell units, counts int32 (n,),
    near_far float32 (n, 2) in world units)."""
    args, keep = _ray_grid_args(hashmap, embeddings, nb_lut, cell_size, origin, interpolation)
    oc = _cuda(ray_o_cell, "ray_o_cell", torch.float32)
    d = _cuda(ray_d, "ray_d", torch.float32)
    lo = _cuda(bbox_min_cell, "bbox_min", torch.float32).view(-1)
    hi = _cuda(bbox_max_cell, "bbox_max", torch.float32).view(-1)
    n, dev = oc.shape[0], oc.device
    stride = int(max_samples_per_ray) + 2
    intervals = torch.empty((n, stride, 2), dtype=torch.float32, device=dev)
    counts = torch.empty(n, dtype=torch.int32, device=dev)
    near_far = torch.empty((n, 2), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _check(_lib.ashb_render_rays_intervals(*args, oc.data_ptr(), d.data_ptr(), lo.data_ptr(), hi.data_ptr(),
                                               float(t_min_cell), float(t_max_cell), int(max_samples_per_ray),
                                               int(bool(skip_missed)), intervals.data_ptr(), counts.data_ptr(),
                                               near_far.data_ptr(), stride, n, _stream(dev)))
    return intervals, counts, near_far


def render_intervals_forward(hashmap, embeddings, nb_lut, cell_size, origin, ray_o_world, ray_d, beta, intervals, counts,
                             near_far, interpolation="linear"):
    """(n_rays, 16) rows as ``render_rays_forward``, one warp per ray over the listed intervals."""
    args, keep = _ray_grid_args(hashmap, embeddings, nb_lut, cell_size, origin, interpolation)
    ow = _cuda(ray_o_world, "ray_o_world", torch.float32)
    d = _cuda(ray_d, "ray_d", torch.float32)
    b = _cuda(beta, "beta", torch.float32).view(-1)
    n, dev = ow.shape[0], ow.device
    out = torch.empty((n, 16), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _check(_lib.ashb_render_intervals_forward(*args, ow.data_ptr(), d.data_ptr(), b.data_ptr(), intervals.data_ptr(),
                                                  counts.data_ptr(), near_far.data_ptr(), intervals.shape[1],
                                                  out.data_ptr(), n, _stream(dev)))
    return out


def render_intervals_backward(hashmap, embeddings, nb_lut, cell_size, origin, ray_o_world, ray_d, beta, intervals, counts,
                              out, grad_out, interpolation="linear", grad_embeddings_out=None):
    """(grad_embeddings, grad_beta (1,)) as ``render_rays_backward``, without marching again."""
    args, keep = _ray_grid_args(hashmap, embeddings, nb_lut, cell_size, origin, interpolation)
    emb = keep[0]
    ow = _cuda(ray_o_world, "ray_o_world", torch.float32)
    d = _cuda(ray_d, "ray_d", torch.float32)
    b = _cuda(beta, "beta", torch.float32).view(-1)
    out = _cuda(out, "out", torch.float32)
    go = _cuda(grad_out, "grad_out", torch.float32)
    n, dev = ow.shape[0], ow.device
    if out.shape != (n, 16) or go.shape != (n, 16):
        raise RuntimeError("out and grad_out must be (n_rays, 16)")
    if grad_embeddings_out is None:
        ge = torch.zeros_like(emb)
    else:
        ge = grad_embeddings_out
        if not (ge.is_cuda and ge.is_contiguous() and ge.shape == emb.shape and ge.dtype == emb.dtype):
            raise RuntimeError("grad_embeddings_out must be a contiguous CUDA tensor shaped like embeddings")
    gb = torch.zeros(1, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _check(_lib.ashb_render_intervals_backward(*args, ow.data_ptr(), d.data_ptr(), b.data_ptr(), intervals.data_ptr(),
                                                   counts.data_ptr(), intervals.shape[1], out.data_ptr(), go.data_ptr(),
                                                   ge.data_ptr(), gb.data_ptr(), n, _stream(dev)))
    return ge, gb


# ---- table sharded over the ranks, queries routed to the owners -----------------------------------
# ``layout`` = (peer_bases_dev, mailbox_bytes, inbox_x, counts, inbox_z, out_y, out_gx, inbox_g, region_capacity, world, rank);
# ``geom`` = (cell_size, origin, grid_dim, nb_lut int32, row_of int32 viewed as uint32, n_emb, D).
def _routed_geom(geom):
    cell_size, origin, grid_dim, nb_lut, row_of, n_emb, D = geom
    return (float(cell_size), _host_floats(origin, 3), int(grid_dim), nb_lut.data_ptr(), row_of.data_ptr(), int(n_emb), int(D))


def routed_route(hashmap, x, geom, layout, cursor, where, status):
    """Send every position of ``x`` (N, 3) float32 to the owner of its block; ``where`` int32 (N,)
    receives owner << 26 | slot (-1: no block there)."""
    x = _cuda(x, "x", torch.float32)
    _check(_lib.ashb_routed_route(hashmap._h, x.data_ptr(), x.shape[0], *_routed_geom(geom), *layout, cursor.data_ptr(),
                                  where.data_ptr(), status.data_ptr(), _stream(x.device)))


def routed_forward(hashmap, emb_bases, geom, layout, interpolation):
    _check(_lib.ashb_routed_forward(hashmap._h, _interp_code(interpolation), emb_bases, *_routed_geom(geom), *layout,
                                    _stream(hashmap.device())))


def routed_unpack_y(where, n, D, layout, with_masks=True):
    dev = where.device
    y = torch.empty((n, D), dtype=torch.float32, device=dev)
    masks = torch.empty(n, dtype=torch.bool, device=dev) if with_masks else None
    with torch.cuda.device(dev):
        _check(_lib.ashb_routed_unpack_y(where.data_ptr(), n, y.data_ptr(), masks.data_ptr() if with_masks else None, D,
                                         *layout, _stream(dev)))
    return y, masks


def routed_send_z(where, z, layout):
    z = _cuda(z, "z", torch.float32)
    with torch.cuda.device(z.device):
        _check(_lib.ashb_routed_send_z(where.data_ptr(), z.shape[0], z.data_ptr(), z.shape[1], *layout, _stream(z.device)))


def routed_backward(hashmap, emb_bases, grad_bases, geom, layout, interpolation, need_grad_x, need_grad_embeddings=True):
    _check(_lib.ashb_routed_backward(hashmap._h, _interp_code(interpolation), emb_bases, grad_bases, int(bool(need_grad_x)),
                                     int(bool(need_grad_embeddings)), *_routed_geom(geom), *layout,
                                     _stream(hashmap.device())))


def routed_send_g(where, grad_grad_x, D, layout):
    g = _cuda(grad_grad_x, "grad_grad_x", torch.float32)
    with torch.cuda.device(g.device):
        _check(_lib.ashb_routed_send_g(where.data_ptr(), g.shape[0], g.data_ptr(), int(D), *layout, _stream(g.device)))


def routed_backward_backward(hashmap, emb_bases, grad_bases, geom, layout, interpolation):
    _check(_lib.ashb_routed_backward_backward(hashmap._h, _interp_code(interpolation), emb_bases, grad_bases,
                                              *_routed_geom(geom), *layout, _stream(hashmap.device())))


def routed_unpack_grad_x(where, n, D, layout):
    dev = where.device
    gx = torch.empty((n, 3), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _check(_lib.ashb_routed_unpack_grad_x(where.data_ptr(), n, gx.data_ptr(), D, *layout, _stream(dev)))
    return gx
