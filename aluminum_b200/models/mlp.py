"""A small MLP used by tests and the smoke run of the data-parallel trainer."""
import torch
from torch import nn


class MLP(nn.Module):
    def __init__(self, d_in: int = 64, d_hidden: int = 128, d_out: int = 10, depth: int = 2):
        super().__init__()
        layers, d = [], d_in
        for _ in range(depth):
            layers += [nn.Linear(d, d_hidden), nn.ReLU()]
            d = d_hidden
        layers.append(nn.Linear(d, d_out))
        self.net = nn.Sequential(*layers)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.net(x)
