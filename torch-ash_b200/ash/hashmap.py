"""HashMap and HashSet containers over ASHEngine (API of ash/hashmap.py)."""
from typing import Dict, List, Union

import torch

from .core import ASHEngine, ASHModule

Values = Union[torch.Tensor, List[torch.Tensor], Dict[str, torch.Tensor]]


def _value_names(value_dims) -> Dict[str, int]:
    """Naming rule of ash/hashmap.py:24-37: int -> "default", list -> "default_i", dict as given."""
    if isinstance(value_dims, int):
        return {"default": value_dims}
    if isinstance(value_dims, list):
        return {f"default_{i}": d for i, d in enumerate(value_dims)}
    if isinstance(value_dims, dict):
        return dict(value_dims)
    raise ValueError("value_dims must be int, list or dict")


class HashMap(ASHModule):
    """Hash map with values stored in registered buffers of ``capacity`` rows."""

    def __init__(self, key_dim: int, value_dims: Union[int, List[int], Dict[str, int]], capacity: int,
                 device: Union[str, torch.device] = torch.device("cpu")):
        super().__init__()
        self.engine = ASHEngine(key_dim, capacity, device)
        self.value_dims = value_dims
        self.values = {}
        self._set_values(
            {name: torch.zeros(capacity, d, device=self.engine.device) for name, d in _value_names(value_dims).items()}
        )

    def _set_values(self, new_values: Dict[str, torch.Tensor]) -> None:
        for name in self.values:
            delattr(self, name)
        self.values = new_values
        for name, v in new_values.items():
            self.register_buffer(name, v)

    def _as_dict(self, values: Values) -> Dict[str, torch.Tensor]:
        if isinstance(values, torch.Tensor):
            assert isinstance(self.value_dims, int)
            return {"default": values}
        if isinstance(values, list):
            assert isinstance(self.value_dims, list)
            return {f"default_{i}": v for i, v in enumerate(values)}
        if isinstance(values, dict):
            assert isinstance(self.value_dims, dict)
            return values
        raise ValueError("values must be Tensor, list, or dict")

    def reinterpret_value_dict(self, values: Dict[str, torch.Tensor]) -> Values:
        """Give values back in the form ``value_dims`` was declared in."""
        if isinstance(self.value_dims, int):
            return values["default"]
        if isinstance(self.value_dims, list):
            return [values[f"default_{i}"] for i in range(len(self.value_dims))]
        if isinstance(self.value_dims, dict):
            return values
        raise ValueError("values must be Tensor, list, or dict")

    def _gather(self, indices: torch.Tensor) -> Values:
        return self.reinterpret_value_dict({name: v[indices] for name, v in self.values.items()})

    def insert(self, keys: torch.Tensor, values: Values) -> None:
        self.engine.insert(keys, self._as_dict(values), self.values)

    def find(self, keys: torch.Tensor, return_indices: bool = True, return_values: bool = False):
        """(masks[, indices][, values]) -- masks first, as ash/hashmap.py:72-95."""
        assert return_indices or return_values, "Must return at least one of indices or values"
        indices, masks = self.engine.find(keys)
        ans = (masks,)
        if return_indices:
            ans += (indices,)
        if return_values:
            ans += (self._gather(indices),)
        return ans

    def erase(self, keys: torch.Tensor) -> None:
        self.engine.erase(keys)

    def clear(self) -> None:
        for v in self.values.values():
            v.zero_()
        self.engine.clear()

    def size(self) -> int:
        return self.engine.size()

    def resize(self, new_capacity: int) -> None:
        new_values = {
            name: torch.zeros(new_capacity, *v.shape[1:], dtype=v.dtype, device=self.engine.device)
            for name, v in self.values.items()
        }
        self.engine.resize(new_capacity, self.values, new_values)
        self._set_values(new_values)

    def keys(self) -> torch.Tensor:
        return self.engine.keys()

    def items(self, return_indices: bool = True, return_values: bool = False):
        """(keys[, indices][, values]) of the active entries (ash/hashmap.py:129-150)."""
        assert return_indices or return_values, "Must return at least one of indices or values"
        active_keys, active_indices = self.engine.items()
        ans = (active_keys,)
        if return_indices:
            ans += (active_indices,)
        if return_values:
            ans += (self._gather(active_indices),)
        return ans


class HashSet(ASHModule):
    """Hash set: keys only (ash/hashmap.py:153-178)."""

    def __init__(self, key_dim: int, capacity: int, device: Union[str, torch.device]):
        super().__init__()
        self.engine = ASHEngine(key_dim, capacity, device)

    def insert(self, keys: torch.Tensor) -> None:
        self.engine.insert_keys(keys)

    def find(self, keys: torch.Tensor) -> torch.Tensor:
        return self.engine.find(keys)[1]

    def erase(self, keys: torch.Tensor) -> None:
        self.engine.erase(keys)

    def clear(self) -> None:
        self.engine.clear()

    def size(self) -> int:
        return self.engine.size()

    def resize(self, new_capacity: int) -> None:
        self.engine.resize(new_capacity)

    def keys(self) -> torch.Tensor:
        return self.engine.keys()
