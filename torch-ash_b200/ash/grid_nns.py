"""Neighbourhood enumeration shared by the grid lookup tables (API of ash/grid_nns.py)."""
from typing import Callable, Tuple

import torch


def enumerate_neighbor_coord_offsets(
    dim: int, radius: int, bidirectional: bool, device: torch.device
) -> Tuple[torch.Tensor, Callable[[torch.Tensor], torch.Tensor]]:
    """All integer offsets of a (one- or two-sided) radius-``radius`` window.

    Same contract as ash/grid_nns.py:5-47: the returned table has
    ``window ** dim`` rows with ``window = 2 * radius + 1`` (two-sided, offsets
    ``-radius..radius``) or ``radius + 1`` (one-sided, ``0..radius``); column 0
    (x) varies fastest, so for radius 1 one-sided row ``c`` is the corner whose
    bit ``d`` is the offset along axis ``d``.  The second return value maps
    offsets (N, dim) back to row numbers (N,).
    """
    lo = -radius if bidirectional else 0
    window = radius - lo + 1
    rows = torch.arange(window**dim, device=device)
    # digit d of the row number in base `window` is the offset along axis d
    digits = [(rows // window**d) % window + lo for d in range(dim)]
    idx2offset = torch.stack(digits, dim=1).contiguous()

    def fn_offset2idx(offset: torch.Tensor) -> torch.Tensor:
        assert offset.dim() == 2
        idx = torch.zeros_like(offset[:, 0])
        for d in reversed(range(dim)):
            idx = idx * window + (offset[:, d] - lo)
        return idx

    return idx2offset, fn_offset2idx
