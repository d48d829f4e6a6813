"""DeepSpeed-Ulysses style sequence parallelism: one alltoall turns a sequence-sharded tensor
(s/p, h, d) into a head-sharded one (s, h/p, d) before attention, and one turns it back."""
from __future__ import annotations

import torch

from ._util import call, unwrap, wrap


def seq_to_head(comm, x):
    """(s_local, h, d) -> (s_local * p, h / p, d)."""
    p = comm.size
    xs = wrap(comm, x)
    sends, outs = [], []
    for t in xs:
        s, h, d = t.shape
        # slice for peer j = heads [j*h/p, (j+1)*h/p): make it contiguous per peer
        sends.append(t.view(s, p, h // p, d).permute(1, 0, 2, 3).contiguous())
        outs.append(torch.empty((p, s, h // p, d), device=t.device, dtype=t.dtype))
    call(comm, comm.alltoall, [s.view(-1) for s in sends], [o.view(-1) for o in outs])
    res = [o.view(p * o.shape[1], o.shape[2], o.shape[3]) for o in outs]
    return unwrap(comm, res, x)


def head_to_seq(comm, x):
    """(s, h_local, d) -> (s / p, h_local * p, d); inverse of :func:`seq_to_head`."""
    p = comm.size
    xs = wrap(comm, x)
    sends, outs = [], []
    for t in xs:
        s, hl, d = t.shape
        sends.append(t.view(p, s // p, hl, d).contiguous())
        outs.append(torch.empty((p, s // p, hl, d), device=t.device, dtype=t.dtype))
    call(comm, comm.alltoall, [s.view(-1) for s in sends], [o.view(-1) for o in outs])
    res = [o.permute(1, 0, 2, 3).contiguous().view(o.shape[1], p * o.shape[2], o.shape[3]) for o in outs]
    return unwrap(comm, res, x)
