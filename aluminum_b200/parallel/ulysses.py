"""DeepSpeed-Ulysses style sequence parallelism: one row exchange turns a sequence-sharded tensor
(s/p, h, d) into a head-sharded one (s, h/p, d) before attention, and one turns it back.

The head slices a rank sends are strided in its tensor and the blocks it receives interleave in the
result; both transpositions happen inside the exchange kernel (kernels/rows.cu: one warp per row reads
the strided source and writes the packed slot, or reads the slot and writes the strided destination), so
no ``permute().contiguous()`` copy runs before or after the alltoall.  Differentiable forms for one rank
per process: :func:`aluminum_b200.parallel.autograd.seq_to_head` / ``head_to_seq``.
"""
from __future__ import annotations

import torch

from ._util import unwrap, wrap


def _tables(comm, rows, first, off):
    one = comm.nlocal == 1
    return (rows if one else [rows] * comm.size, first if one else [first] * comm.size, off if one else [off] * comm.size)


def seq_to_head(comm, x):
    """(s_local, h, d) -> (s_local * p, h / p, d)."""
    p = comm.size
    xs = [t.contiguous() for t in wrap(comm, x)]
    s, h, d = xs[0].shape
    esz = xs[0].element_size()
    rb = (h // p) * d * esz
    outs = [torch.empty((s * p, h // p, d), device=t.device, dtype=t.dtype) for t in xs]
    sr, sf, so = _tables(comm, [s] * p, [0] * p, [j * rb for j in range(p)])
    rr, rf, ro = _tables(comm, [s] * p, [j * s for j in range(p)], [0] * p)
    one = comm.nlocal == 1
    comm.exchange_rows(xs[0] if one else xs, outs[0] if one else outs, rb, h * d * esz, rb, sr, sf, so, rr, rf, ro)
    return unwrap(comm, outs, x)


def head_to_seq(comm, x):
    """(s, h_local, d) -> (s / p, h_local * p, d); inverse of :func:`seq_to_head`."""
    p = comm.size
    xs = [t.contiguous() for t in wrap(comm, x)]
    s, hl, d = xs[0].shape
    esz = xs[0].element_size()
    rb = hl * d * esz
    outs = [torch.empty((s // p, hl * p, d), device=t.device, dtype=t.dtype) for t in xs]
    sr, sf, so = _tables(comm, [s // p] * p, [j * (s // p) for j in range(p)], [0] * p)
    rr, rf, ro = _tables(comm, [s // p] * p, [0] * p, [j * rb for j in range(p)])
    one = comm.nlocal == 1
    comm.exchange_rows(xs[0] if one else xs, outs[0] if one else outs, rb, rb, p * rb, sr, sf, so, rr, rf, ro)
    return unwrap(comm, outs, x)
