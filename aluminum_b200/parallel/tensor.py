"""Tensor parallelism: column- and row-parallel linear layers (Megatron style).

Built on the device communicator's allgather / allreduce; the reference offers only those
primitives (include/Al.hpp:119-207, 551-633 of the reference).
"""
from __future__ import annotations

import torch

from ._util import call, unwrap, wrap


def column_parallel_linear(comm, x, w_shard, gather_output: bool = True):
    """y = x @ W^T with W split by output features: every rank computes its slice of the outputs;
    with ``gather_output`` the slices are allgathered (feature-major, then transposed back)."""
    xs, ws = wrap(comm, x), wrap(comm, w_shard)
    ys = [xi @ wi.t() for xi, wi in zip(xs, ws)]
    if not gather_output:
        return unwrap(comm, ys, x)
    p = comm.size
    # allgather wants each rank's contribution contiguous: send the transposed slice (f_local, batch)
    send = [y.t().contiguous() for y in ys]
    recv = [torch.empty((p * s.shape[0], s.shape[1]), device=s.device, dtype=s.dtype) for s in send]
    call(comm, comm.allgather, [s.view(-1) for s in send], [r.view(-1) for r in recv])
    return unwrap(comm, [r.t().contiguous() for r in recv], x)


def row_parallel_linear(comm, x_shard, w_shard):
    """y = x @ W^T with W split by input features: partial products are summed with an allreduce."""
    xs, ws = wrap(comm, x_shard), wrap(comm, w_shard)
    ys = [(xi @ wi.t()).contiguous() for xi, wi in zip(xs, ws)]
    call(comm, comm.allreduce, [y.view(-1) for y in ys])
    return unwrap(comm, ys, x_shard)
