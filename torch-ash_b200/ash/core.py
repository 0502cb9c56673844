"""ASHEngine: the key -> index hash engine behind every container (API of ash/core.py).

The engine keeps the minimal state of a collision-free hash map: the native
table (``backend``, a ``__ash.HashMap``) and the free-index stack ``_heap``.
Values / embeddings live outside, in rows addressed by the indices it hands
out.  Class, method, argument and state_dict key names follow ash/core.py:39-371
so that code and checkpoints written for the reference keep working.
"""
import warnings
from typing import Dict, Optional, Tuple, Union

import torch
import torch.nn as nn

from .common import _get_c_extension

backend = _get_c_extension()


def _as_device(device) -> torch.device:
    device = torch.device(device) if not isinstance(device, torch.device) else device
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return device


class ASHEngine(nn.Module):
    """Hash map core: keys (int32, ``dim`` columns) -> row indices in ``[0, capacity)``."""

    def __init__(self, dim: int, capacity: int, device: Union[str, torch.device] = torch.device("cpu")):
        super().__init__()
        assert dim > 0, "dim must be positive"
        assert capacity > 0, "capacity must be positive"
        self.dim = dim
        self.capacity = capacity
        self.device = _as_device(device)
        self._register_buffers()
        self.backend = backend.HashMap(self.dim, self.capacity, self._heap, self.device)
        # Host-side upper bound on the number of live keys: lets inserts that
        # cannot overflow skip the device round trip the reference pays twice
        # per call (ash/core.py:203-205).
        self._size_bound = 0
        # Upper bound on the erased slots (tombstones) the open-addressing table carries.  When it
        # passes half the capacity the table is rebuilt from its live entries, so that long
        # insert / erase histories (fusion with pruning) do not lengthen every probe.
        self._erased_bound = 0
        self.auto_rehash = True
        self.register_load_state_dict_post_hook(ASHEngine._post_load_state_dict_hook)

    # ------------------------------------------------------------------ state
    def _register_buffers(self) -> None:
        """(Re)create the checkpointed buffers (ash/core.py:69-90): the live heap plus
        ``_keys/_indices/_size``, which are only filled in by ``state_dict()``."""
        dev = self.device
        self.register_buffer("_heap", torch.arange(self.capacity, dtype=torch.int32, device=dev))
        self.register_buffer("_keys", torch.zeros((self.capacity, self.dim), dtype=torch.int32, device=dev))
        self.register_buffer("_indices", torch.zeros(self.capacity, dtype=torch.long, device=dev))
        self.register_buffer("_size", torch.zeros(1, dtype=torch.int32, device=dev))

    def state_dict(self, *args, **kwargs):
        """Snapshot the active (key, index) pairs into the buffers, then defer to nn.Module
        (ash/core.py:92-114)."""
        keys, indices = self.items()
        n = keys.shape[0]
        self._size.fill_(n)
        if n > 0:
            self._keys[:n] = keys
            self._indices[:n] = indices
        return super().state_dict(*args, **kwargs)

    def _post_load_state_dict_hook(self, incompatible_keys) -> None:
        """Rebuild the native table from the loaded buffers (ash/core.py:116-135)."""
        n = int(self._size.item())
        assert self._heap.numel() == self.capacity
        active_keys = self._keys[:n]
        self._key_check(active_keys)
        # Loading replaces the contents: an engine that already holds keys (a replica being
        # re-aligned with another rank) must not keep its old key -> index pairs.  clear() resets the
        # aliased free-index stack, so the loaded one is set aside first.
        heap = self._heap.clone()
        self.backend.clear()
        self.backend.load_states({"active_keys": active_keys, "active_indices": self._indices[:n], "heap": heap})
        self._size_bound = n
        self._erased_bound = 0

    # ------------------------------------------------------------------ checks
    def _key_check(self, keys: torch.Tensor) -> None:
        assert keys.dim() == 2 and keys.shape[1] == self.dim, "keys shape mismatch"
        if keys.dtype != torch.int32:
            warnings.warn("keys are not int32, conversion might reduce precision.")

    def _value_check(self, values: Dict[str, torch.Tensor], external_values: Dict[str, torch.Tensor]) -> None:
        assert values.keys() == external_values.keys()
        for name, v in values.items():
            ext = external_values[name]
            assert v.is_contiguous() and ext.is_contiguous()
            assert v.dim() == ext.dim() and v.dtype == ext.dtype and v.shape[1:] == ext.shape[1:]
            assert ext.shape[0] == self.capacity

    def _prepare(self, keys: torch.Tensor) -> Optional[torch.Tensor]:
        self._key_check(keys)
        if keys.shape[0] == 0:
            warnings.warn("empty keys")
            return None
        return keys.to(self.device, torch.int32).contiguous()

    def _after_insert(self, n_new: int) -> None:
        """Overflow check of ash/core.py:206-211, paid for only when the batch could overflow."""
        self._size_bound += n_new
        if self._size_bound <= self.capacity:
            return
        self._report_status(f"Insertion of {n_new} keys")
        self._size_bound = self.backend.size()

    def _report_status(self, what: str) -> None:
        """Read and clear the native status word: capacity exhausted -> the reference's warning
        (ash/core.py:206-211); a probe or wait that gave up (the key was NOT stored) -> error.  Called
        where the host synchronises with the device anyway (a batch that could overflow, size(),
        items(), state_dict()), so that no such bit stays unseen."""
        if not hasattr(self.backend, "status"):
            return
        st = self.backend.status()
        if st & backend.STATUS_CAPACITY:
            warnings.warn(
                f"{what} exceeds the hash map capacity {self.capacity}; the keys beyond "
                "capacity were dropped. Please resize the hash map or the behavior could be unexpected."
            )
        if st & ~backend.STATUS_CAPACITY:
            raise RuntimeError(f"hash table status 0x{st:x}")

    # ------------------------------------------------------------------ operations
    def find(self, keys: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """(indices int64 (N,), masks bool (N,)); a miss has index 0 and mask False."""
        k = self._prepare(keys)
        if k is None:
            return (
                torch.empty((0,), dtype=torch.long, device=self.device),
                torch.empty((0,), dtype=torch.bool, device=self.device),
            )
        return self.backend.find(k)

    def insert_keys(self, keys: torch.Tensor) -> None:
        """Insert-if-absent without values; each new key takes the next free index."""
        k = self._prepare(keys)
        if k is None:
            return
        self.backend.insert_keys(k)
        self._after_insert(k.shape[0])

    def insert(self, keys: torch.Tensor, values: Dict[str, torch.Tensor],
               external_values: Dict[str, torch.Tensor]) -> None:
        """Insert-if-absent; the row of every new key is copied into ``external_values``."""
        k = self._prepare(keys)
        if k is None:
            return
        self._value_check(values, external_values)
        for v in values.values():
            assert v.shape[0] == k.shape[0]
        self.backend.insert(k, values, external_values)
        self._after_insert(k.shape[0])

    def erase(self, keys: torch.Tensor) -> None:
        self._key_check(keys)
        if keys.shape[0] == 0:
            warnings.warn("empty keys")
            return
        self.backend.erase(keys)
        self._erased_bound += keys.shape[0]
        # auto_rehash: rebuild the table once the erased keys may fill half of it (tombstones lengthen every
        # probe).  The rebuild allocates a second table and waits for the stream, so it cannot run inside
        # stream capture nor while another stream still probes this map: set auto_rehash = False there and
        # call backend.rehash() at a point of your choosing.
        if self.auto_rehash and self._erased_bound > self.capacity // 2 and hasattr(self.backend, "rehash"):
            self.backend.rehash()
            self._erased_bound = 0

    def clear(self) -> None:
        self.backend.clear()
        self._size_bound = 0
        self._erased_bound = 0

    def size(self) -> int:
        self._size_bound = self.backend.size()
        self._report_status("An earlier insertion")
        return self._size_bound

    def resize(self, capacity: int, old_external_values: Dict[str, torch.Tensor] = None,
               new_external_values: Dict[str, torch.Tensor] = None) -> None:
        """Change the capacity, keeping every key -> value association (ash/core.py:266-302).

        Growing keeps every live key at ITS index: a table of the new size is loaded with the
        (key, index) pairs as a checkpoint would be, the free-index stack is carried over with the
        new indices appended, and value rows move as one straight copy of the old buffers into the
        head of the new ones -- no re-insertion, no gather by index.  Shrinking re-inserts the
        active keys and moves their rows by index, as the reference always does."""
        active_keys, old_indices = self.items()
        n = active_keys.shape[0]
        assert capacity >= n, "new capacity is smaller than the current size"
        assert capacity > 0, "new capacity is 0"
        old_heap, old_capacity = self._heap, self.capacity
        in_place = capacity >= old_capacity
        del self.backend
        self.capacity = capacity
        self._register_buffers()
        if in_place:
            self._heap[:old_capacity] = old_heap   # entries n .. old_capacity-1 are the old free indices; the new ones follow
        self.backend = backend.HashMap(self.dim, self.capacity, self._heap, self.device)
        self._size_bound = n
        self._erased_bound = 0
        if in_place:
            if n:
                self.backend.load_states({"active_keys": active_keys, "active_indices": old_indices, "heap": self._heap})
            if old_external_values is not None and new_external_values is not None:
                for name, v in old_external_values.items():
                    new_external_values[name][:old_capacity] = v
            return
        if n == 0:
            return
        if old_external_values is not None and new_external_values is not None:
            moved = {name: v[old_indices].contiguous() for name, v in old_external_values.items()}
            self.backend.insert(active_keys, moved, new_external_values)
        else:
            self.backend.insert_keys(active_keys)

    def keys(self) -> torch.Tensor:
        return self.items()[0]

    def items(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """(active_keys int32 (n, dim), active_indices int64 (n,)), order unspecified."""
        self._report_status("An earlier insertion")
        return self.backend.items()

    # ------------------------------------------------------------------ device moves
    def to(self, device: Union[str, torch.device]):
        """Engine on ``device``.  The reference returns a fresh EMPTY engine here
        (ash/core.py:325-329, marked TODO); this one carries its contents along."""
        device = _as_device(device)
        if device == self.device:
            return self
        moved = ASHEngine(self.dim, self.capacity, device)
        keys, indices = self.items()
        moved._heap.copy_(self._heap)
        moved.backend.load_states(
            {"active_keys": keys.to(device), "active_indices": indices.to(device), "heap": moved._heap}
        )
        moved._size_bound = keys.shape[0]
        return moved

    def cpu(self):
        return self.to("cpu")

    def cuda(self, device: Optional[Union[str, torch.device]] = None):
        return self.to("cuda" if device is None else device)

    def __repr__(self) -> str:
        return f"ASHEngine (dim={self.dim}, capacity={self.capacity}, size={self.size()}) at {self.device}"


class ASHModule(nn.Module):
    """Base of HashSet / HashMap / HashEmbedding / grids: moves the engine with the module
    (ash/core.py:349-371)."""

    def __init__(self):
        super().__init__()
        self.engine = None

    def to(self, device):
        assert self.engine is not None, "engine is not initialized"
        module = super().to(device)
        module.engine = module.engine.to(device)
        return module

    def cpu(self):
        return self.to(torch.device("cpu"))

    def cuda(self, device: Optional[Union[str, torch.device]] = None):
        return self.to(torch.device("cuda") if device is None else device)
