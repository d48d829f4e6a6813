"""Expert parallelism: token dispatch to the rank that owns the chosen expert and the inverse
combine, on alltoallv (counts are exchanged with a small alltoall first)."""
from __future__ import annotations

import torch

from ._util import call, local_ranks, unwrap, wrap


def dispatch(comm, tokens, dest_rank):
    """Send every token (row of ``tokens``) to ``dest_rank[i]``.

    Returns (received tokens grouped by source rank, state for :func:`combine`)."""
    p = comm.size
    toks, dests = wrap(comm, tokens), wrap(comm, dest_rank)
    order = [torch.argsort(d, stable=True) for d in dests]
    sorted_toks = [t[o].contiguous() for t, o in zip(toks, order)]
    send_counts = [torch.bincount(d, minlength=p).to(torch.int64) for d in dests]
    recv_counts = [torch.empty(p, device=c.device, dtype=torch.int64) for c in send_counts]
    call(comm, comm.alltoall, send_counts, recv_counts)
    width = toks[0].shape[1]
    sc = [[int(v) * width for v in c.tolist()] for c in send_counts]
    rc = [[int(v) * width for v in c.tolist()] for c in recv_counts]
    sd = [[sum(r[:i]) for i in range(p)] for r in sc]
    rd = [[sum(r[:i]) for i in range(p)] for r in rc]
    outs = [torch.empty((sum(r) // width, width), device=toks[0].device, dtype=toks[0].dtype) for r in rc]
    one = comm.nlocal == 1
    call(comm, comm.alltoallv, [t.view(-1) for t in sorted_toks], sc[0] if one else sc, sd[0] if one else sd,
         [o.view(-1) for o in outs], rc[0] if one else rc, rd[0] if one else rd)
    state = {"order": order, "sc": sc, "sd": sd, "rc": rc, "rd": rd, "width": width, "like": tokens}
    return unwrap(comm, outs, tokens), state


def combine(comm, expert_out, state):
    """Return processed tokens to the ranks (and positions) they came from."""
    outs_in = wrap(comm, expert_out)
    width = state["width"]
    one = comm.nlocal == 1
    sc, sd, rc, rd = state["rc"], state["rd"], state["sc"], state["sd"]  # directions swap
    back = [torch.empty((sum(r) // width, width), device=outs_in[0].device, dtype=outs_in[0].dtype) for r in rc]
    call(comm, comm.alltoallv, [t.contiguous().view(-1) for t in outs_in], sc[0] if one else sc, sd[0] if one else sd,
         [b.view(-1) for b in back], rc[0] if one else rc, rd[0] if one else rd)
    res = []
    for b, o in zip(back, state["order"]):
        r = torch.empty_like(b)
        r[o] = b
        res.append(r)
    return unwrap(comm, res, state["like"])
