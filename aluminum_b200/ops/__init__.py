"""Element-wise and halo kernels exposed as functions on PyTorch tensors."""
from .elementwise import fill_u32, scale_cast, sgd_momentum_step
from .halo import HaloExchange, halo_pack, halo_unpack

__all__ = ["scale_cast", "sgd_momentum_step", "fill_u32", "HaloExchange", "halo_pack", "halo_unpack"]
