"""Halo exchange for spatially partitioned 3-D convolutions.

A global tensor (N, C, D, H, W) is split along D; every rank stores its slab
with ``depth`` extra planes on both sides.  :class:`HaloExchange` allocates the
slab in symmetric memory and fills the halo planes of both neighbours with one
fused kernel (direct peer stores, no pack / unpack buffers).  This is the
pattern the reference exercises with Put / Sync in
``test/test_rma_halo_exchange.cpp:79-241``.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib
from .._lib import check


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def halo_pack(tensor: torch.Tensor, d_first: int, depth: int, out: torch.Tensor = None) -> torch.Tensor:
    """Gather planes [d_first, d_first+depth) of every channel of a (N, C, D, H, W) fp32 tensor into a packed buffer."""
    n, c, d, h, w = tensor.shape
    if out is None:
        out = torch.empty(n * c * depth * h * w, device=tensor.device, dtype=torch.float32)
    check(_lib.load().al_halo_pack(C.c_void_p(out.data_ptr()), C.c_void_p(tensor.data_ptr()), n * c, d, h * w, d_first,
                                   depth, 0, _stream()))
    return out


def halo_unpack(tensor: torch.Tensor, packed: torch.Tensor, d_first: int, depth: int) -> None:
    n, c, d, h, w = tensor.shape
    check(_lib.load().al_halo_pack(C.c_void_p(packed.data_ptr()), C.c_void_p(tensor.data_ptr()), n * c, d, h * w, d_first,
                                   depth, 1, _stream()))


class HaloExchange:
    """Owns the symmetric slab(s) of one D-split tensor and exchanges halos on demand."""

    def __init__(self, comm, n: int, c: int, d_local: int, h: int, w: int, depth: int = 1, periodic: bool = False):
        self.comm, self.depth, self.periodic = comm, depth, periodic
        shape = (n, c, d_local + 2 * depth, h, w)
        slabs = comm.symm_empty(shape, torch.float32)
        if comm.nlocal > 1:
            self.tensors = slabs            # emulation: every rank's slab
            self.local = slabs
        else:
            self.local = slabs
            self.tensors = [None] * comm.size
            self.tensors[comm.rank] = slabs
            p = comm.size
            for nb in {comm.rank - 1, comm.rank + 1}:
                if periodic:
                    nb %= p
                if 0 <= nb < p and nb != comm.rank:
                    self.tensors[nb] = comm.peer_ptr(slabs, nb)

    def exchange(self, ctas: int = 0) -> None:
        """Fill the neighbours' halo planes from this rank's boundary planes and wait for theirs."""
        self.comm.halo_exchange(self.tensors, self.depth, self.periodic, ctas)
