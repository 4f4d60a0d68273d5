"""The small encoder model the reference's README trains (README.md:64-77): embedding,
``nn.TransformerEncoderLayer`` stack (post-LN, ReLU, dropout 0.1, batch_first) and a vocabulary
projection. It is the "plumbing" model of the CPU configuration: any ``nn.Module`` goes through the
same Trainer / Scheduler path."""
from __future__ import annotations

import torch
import torch.nn as nn


class SimpleTransformer(nn.Module):
    def __init__(self, vocab_size: int = 10000, d_model: int = 768, num_layers: int = 12, nhead: int = 12,
                 dim_feedforward: int = 2048, dropout: float = 0.1):
        super().__init__()
        self.embedding = nn.Embedding(vocab_size, d_model)
        self.layers = nn.ModuleList([
            nn.TransformerEncoderLayer(d_model=d_model, nhead=nhead, dim_feedforward=dim_feedforward, dropout=dropout,
                                       batch_first=True)
            for _ in range(num_layers)
        ])
        self.output = nn.Linear(d_model, vocab_size)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = self.embedding(x)
        for layer in self.layers:
            h = layer(h)
        return self.output(h)
