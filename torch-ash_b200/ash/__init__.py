"""ash -- torch-ash's Python API on hand-written sm_100a CUDA (B200).

Same public names as the reference package (ash/__init__.py:1-14) minus the
dense MLP helpers, which are not part of the sparse hot path.
"""
from .common import DotDict
from .core import ASHEngine, ASHModule
from .embedding import HashEmbedding
from .grid import (
    BoundedSparseDenseGrid,
    SparseDenseGrid,
    UnBoundedSparseDenseGrid,
    UnboundedSparseDenseGrid,
)
from .grid_nns import enumerate_neighbor_coord_offsets
from .grid_query import SparseDenseGridQuery, SparseDenseGridQueryBackward
from .hashmap import HashMap, HashSet

__all__ = [
    "ASHEngine", "ASHModule", "BoundedSparseDenseGrid", "DotDict", "HashEmbedding", "HashMap", "HashSet",
    "SparseDenseGrid", "SparseDenseGridQuery", "SparseDenseGridQueryBackward", "UnBoundedSparseDenseGrid",
    "UnboundedSparseDenseGrid", "enumerate_neighbor_coord_offsets",
]
