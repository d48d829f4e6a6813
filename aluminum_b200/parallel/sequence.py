"""Sequence parallelism (Megatron style): activations are sharded along the sequence dimension
outside the tensor-parallel blocks.  Entering a block allgathers the sequence, leaving it
reduce-scatters the partial sums - both on the library's kernels, with the optional dtype cast
fused into the allgather's publish step (fp32 shards gathered as bf16)."""
from __future__ import annotations

import torch

from ._util import call, unwrap, wrap


def gather_sequence(comm, x_shard, out_dtype=None):
    """(s/p, ...) on every rank -> (s, ...) on every rank."""
    xs = [x.contiguous() for x in wrap(comm, x_shard)]
    p = comm.size
    dt = out_dtype or xs[0].dtype
    outs = [torch.empty((p * x.shape[0],) + tuple(x.shape[1:]), device=x.device, dtype=dt) for x in xs]
    kw = {"wire_dtype": dt} if dt != xs[0].dtype else {}
    call(comm, comm.allgather, [x.view(-1) for x in xs], [o.view(-1) for o in outs], **kw)
    return unwrap(comm, outs, x_shard)


def scatter_sequence(comm, x_partial):
    """Partial sums (s, ...) on every rank -> reduced shard (s/p, ...) on every rank."""
    xs = [x.contiguous() for x in wrap(comm, x_partial)]
    p = comm.size
    outs = [torch.empty((x.shape[0] // p,) + tuple(x.shape[1:]), device=x.device, dtype=x.dtype) for x in xs]
    call(comm, comm.reduce_scatter, [x.view(-1) for x in xs], [o.view(-1) for o in outs])
    return unwrap(comm, outs, x_partial)
