"""Differentiable collectives and the tensor- / sequence-parallel layers built from them.

Each function is a :class:`torch.autograd.Function` whose backward is the conjugate collective, so models
sharded across the ranks of a :class:`~aluminum_b200.device.DeviceComm` (one process and one GPU per rank)
train with plain ``loss.backward()``:

==================  ================================  =================================
function            forward                           backward
==================  ================================  =================================
``copy_to_ranks``   identity                          allreduce (sum)
``reduce_from``     allreduce (sum)                   identity
``gather_seq``      allgather along dim 0             reduce_scatter (sum) along dim 0
``scatter_seq``     reduce_scatter (sum) along dim 0  allgather along dim 0
``seq_to_head``     row exchange (s/p,h,d)->(s,h/p,d) row exchange back
``head_to_seq``     row exchange (s,h/p,d)->(s/p,h,d) row exchange back
==================  ================================  =================================

The reference offers only the collectives themselves (include/Al.hpp:119-925 of the reference); these are the
consumers' layers (Megatron-style tensor + sequence parallelism, DeepSpeed-Ulysses) on this library's kernels.
"""
from __future__ import annotations

import math

import torch
from torch import nn


class _Copy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, comm, x):
        ctx.comm = comm
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        ctx.comm.allreduce(g.view(-1))
        return None, g


class _Reduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, comm, x):
        y = x.contiguous().clone()
        comm.allreduce(y.view(-1))
        return y

    @staticmethod
    def backward(ctx, g):
        return None, g


class _GatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, comm, x):
        ctx.comm = comm
        x = x.contiguous()
        out = torch.empty((x.shape[0] * comm.size,) + tuple(x.shape[1:]), device=x.device, dtype=x.dtype)
        comm.allgather(x.view(-1), out.view(-1))
        return out

    @staticmethod
    def backward(ctx, g):
        comm = ctx.comm
        g = g.contiguous()
        out = torch.empty((g.shape[0] // comm.size,) + tuple(g.shape[1:]), device=g.device, dtype=g.dtype)
        comm.reduce_scatter(g.view(-1), out.view(-1))
        return None, out


class _ScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, comm, x):
        ctx.comm = comm
        x = x.contiguous()
        out = torch.empty((x.shape[0] // comm.size,) + tuple(x.shape[1:]), device=x.device, dtype=x.dtype)
        comm.reduce_scatter(x.view(-1), out.view(-1))
        return out

    @staticmethod
    def backward(ctx, g):
        comm = ctx.comm
        g = g.contiguous()
        out = torch.empty((g.shape[0] * comm.size,) + tuple(g.shape[1:]), device=g.device, dtype=g.dtype)
        comm.allgather(g.view(-1), out.view(-1))
        return None, out


def _seq_to_head_raw(comm, x):
    """(s_local, h, d) -> (s_local * p, h / p, d): one kernel, the transposition happens in its publish step."""
    p = comm.size
    s, h, d = x.shape
    esz = x.element_size()
    rb = (h // p) * d * esz
    out = torch.empty((s * p, h // p, d), device=x.device, dtype=x.dtype)
    comm.exchange_rows(x, out, rb, h * d * esz, rb,
                       send_rows=[s] * p, send_first=[0] * p, send_peer_off=[j * rb for j in range(p)],
                       recv_rows=[s] * p, recv_first=[j * s for j in range(p)], recv_peer_off=[0] * p)
    return out


def _head_to_seq_raw(comm, x):
    """(s, h_local, d) -> (s / p, h_local * p, d): the inverse; the transposition happens in the consume step."""
    p = comm.size
    s, hl, d = x.shape
    esz = x.element_size()
    rb = hl * d * esz
    out = torch.empty((s // p, hl * p, d), device=x.device, dtype=x.dtype)
    comm.exchange_rows(x, out, rb, rb, p * rb,
                       send_rows=[s // p] * p, send_first=[j * (s // p) for j in range(p)], send_peer_off=[0] * p,
                       recv_rows=[s // p] * p, recv_first=[0] * p, recv_peer_off=[j * rb for j in range(p)])
    return out


class _SeqToHead(torch.autograd.Function):
    @staticmethod
    def forward(ctx, comm, x):
        ctx.comm = comm
        return _seq_to_head_raw(comm, x.contiguous())

    @staticmethod
    def backward(ctx, g):
        return None, _head_to_seq_raw(ctx.comm, g.contiguous())


class _HeadToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, comm, x):
        ctx.comm = comm
        return _head_to_seq_raw(comm, x.contiguous())

    @staticmethod
    def backward(ctx, g):
        return None, _seq_to_head_raw(ctx.comm, g.contiguous())


def copy_to_ranks(comm, x):
    return _Copy.apply(comm, x)


def reduce_from_ranks(comm, x):
    return _Reduce.apply(comm, x)


def gather_seq(comm, x):
    return _GatherSeq.apply(comm, x)


def scatter_seq(comm, x):
    return _ScatterSeq.apply(comm, x)


def seq_to_head(comm, x):
    return _SeqToHead.apply(comm, x)


def head_to_seq(comm, x):
    return _HeadToSeq.apply(comm, x)


def _full_weight(out_f: int, in_f: int, seed: int, device, dtype):
    """The unsharded weight every rank can reproduce (same seed): shards of it equal a single-device layer."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    w = torch.empty(out_f, in_f, dtype=torch.float32)
    bound = 1.0 / math.sqrt(in_f)
    w.uniform_(-bound, bound, generator=g)
    b = torch.empty(out_f, dtype=torch.float32).uniform_(-bound, bound, generator=g)
    return w.to(device=device, dtype=dtype), b.to(device=device, dtype=dtype)


class ColumnParallelLinear(nn.Module):
    """y = x W^T + b with W split by output features.  ``sequence_parallel``: the input arrives sharded along
    dim 0 and is allgathered on entry (backward: reduce-scatter); otherwise it is replicated (backward: allreduce).
    The output stays split by features unless ``gather_output``."""

    def __init__(self, comm, in_features: int, out_features: int, bias: bool = True, sequence_parallel: bool = False,
                 seed: int = 0, device="cuda", dtype=torch.float32):
        super().__init__()
        p, r = comm.size, comm.rank
        assert out_features % p == 0
        self.comm, self.sequence_parallel = comm, sequence_parallel
        w, b = _full_weight(out_features, in_features, seed, device, dtype)
        n = out_features // p
        self.weight = nn.Parameter(w[r * n:(r + 1) * n].clone())
        self.bias = nn.Parameter(b[r * n:(r + 1) * n].clone()) if bias else None

    def forward(self, x):
        x = gather_seq(self.comm, x) if self.sequence_parallel else copy_to_ranks(self.comm, x)
        return nn.functional.linear(x, self.weight, self.bias)


class RowParallelLinear(nn.Module):
    """y = x W^T + b with W split by input features (the input is the feature-split output of a column-parallel
    layer).  The partial products are allreduced, or reduce-scattered along dim 0 with ``sequence_parallel``.
    The bias is replicated and added after the reduction; with sequence parallelism its gradient has to be
    summed over the ranks (:func:`sync_replicated_grads`)."""

    def __init__(self, comm, in_features: int, out_features: int, bias: bool = True, sequence_parallel: bool = False,
                 seed: int = 1, device="cuda", dtype=torch.float32):
        super().__init__()
        p, r = comm.size, comm.rank
        assert in_features % p == 0
        self.comm, self.sequence_parallel = comm, sequence_parallel
        w, b = _full_weight(out_features, in_features, seed, device, dtype)
        n = in_features // p
        self.weight = nn.Parameter(w[:, r * n:(r + 1) * n].clone())
        self.bias = nn.Parameter(b.clone()) if bias else None
        if self.bias is not None:
            self.bias.replicated = True

    def forward(self, x):
        y = nn.functional.linear(x, self.weight)
        y = scatter_seq(self.comm, y) if self.sequence_parallel else reduce_from_ranks(self.comm, y)
        return y if self.bias is None else y + self.bias


def sync_replicated_grads(comm, module: nn.Module) -> None:
    """Sum the gradients of parameters that are replicated while the activations they see are sharded along the
    sequence (biases and norms outside the tensor-parallel blocks)."""
    for prm in module.parameters():
        if getattr(prm, "replicated", False) and prm.grad is not None:
            comm.allreduce(prm.grad.view(-1))
