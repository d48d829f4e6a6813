"""Models used by the end-to-end benchmarks and tests."""
from .mlp import MLP
from .resnet import ResNet, resnet50

__all__ = ["ResNet", "resnet50", "MLP"]
