"""HashEmbedding: a trainable row per inserted key (API of ash/embedding.py)."""
from typing import Union

import torch
import torch.nn as nn

from .core import ASHEngine, ASHModule


class HashEmbedding(ASHModule):
    """Static-capacity embedding table addressed through the hash engine.

    ``forward`` returns the stored row for inserted keys and zeros for the rest
    (ash/embedding.py:31-38); gradients flow to ``embedding`` through plain
    indexing.
    """

    def __init__(self, in_dim: int, num_embeddings: int, embedding_dim: int,
                 device: Union[str, torch.device] = "cpu"):
        super().__init__()
        self.engine = ASHEngine(in_dim, num_embeddings, device)
        self.embedding = nn.Parameter(torch.randn(num_embeddings, embedding_dim, device=self.engine.device))

    def spatial_init_(self, keys: torch.Tensor) -> None:
        self.engine.insert_keys(keys)

    def forward(self, keys: torch.Tensor) -> torch.Tensor:
        indices, masks = self.engine.find(keys)
        return self.embedding[indices] * masks.unsqueeze(-1)
