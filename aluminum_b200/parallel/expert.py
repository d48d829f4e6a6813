"""Expert parallelism: token dispatch to the rank that owns the chosen expert and the inverse combine.

Both directions are one row exchange (kernels/rows.cu): dispatch reads the tokens through the sort
permutation inside the kernel's publish step (no gather into a packed send buffer) and combine writes the
returning tokens through the same permutation in its consume step (no scatter afterwards).  The per-peer
token counts are exchanged with a small alltoall and read back with ONE device-to-host copy (the sizes of
the receive buffer have to be known on the host to allocate it).
"""
from __future__ import annotations

import torch

from ._util import call, unwrap, wrap


def _prefix(counts):
    out, run = [], 0
    for c in counts:
        out.append(run)
        run += c
    return out


def dispatch(comm, tokens, dest_rank):
    """Send every token (row of ``tokens``) to ``dest_rank[i]``.

    Returns (received tokens grouped by source rank, state for :func:`combine`)."""
    p = comm.size
    toks = [t.contiguous() for t in wrap(comm, tokens)]
    dests = wrap(comm, dest_rank)
    order = [torch.argsort(d, stable=True).contiguous() for d in dests]   # int64: token i of the sorted order
    send_counts = [torch.bincount(d, minlength=p).to(torch.int64) for d in dests]
    recv_counts = [torch.empty(p, device=c.device, dtype=torch.int64) for c in send_counts]
    call(comm, comm.alltoall, send_counts, recv_counts)
    both = torch.stack([torch.stack(send_counts), torch.stack(recv_counts)]).cpu()   # the one host read
    sc = [[int(v) for v in row] for row in both[0].tolist()]
    rc = [[int(v) for v in row] for row in both[1].tolist()]
    width = toks[0].shape[1]
    rb = width * toks[0].element_size()
    outs = [torch.empty((sum(r), width), device=toks[0].device, dtype=toks[0].dtype) for r in rc]
    one = comm.nlocal == 1
    zeros = [[0] * p for _ in sc]
    sf = [_prefix(r) for r in sc]
    rf = [_prefix(r) for r in rc]
    pick = (lambda t: t[0]) if one else (lambda t: t)
    comm.exchange_rows(pick(toks), pick(outs), rb, rb, rb, pick(sc), pick(sf), pick(zeros), pick(rc), pick(rf),
                       pick(zeros), send_idx=pick(order))
    state = {"order": order, "sc": sc, "sf": sf, "rc": rc, "rf": rf, "width": width, "like": tokens}
    return unwrap(comm, outs, tokens), state


def combine(comm, expert_out, state):
    """Return processed tokens to the ranks (and positions) they came from."""
    p = comm.size
    outs_in = [t.contiguous() for t in wrap(comm, expert_out)]
    width = state["width"]
    rb = width * outs_in[0].element_size()
    one = comm.nlocal == 1
    # directions swap: what was received is sent back, and lands through the sort permutation
    sc, sf, rc, rf = state["rc"], state["rf"], state["sc"], state["sf"]
    back = [torch.empty((sum(r), width), device=outs_in[0].device, dtype=outs_in[0].dtype) for r in rc]
    zeros = [[0] * p for _ in sc]
    pick = (lambda t: t[0]) if one else (lambda t: t)
    comm.exchange_rows(pick(outs_in), pick(back), rb, rb, rb, pick(sc), pick(sf), pick(zeros), pick(rc), pick(rf),
                       pick(zeros), recv_idx=pick(state["order"]))
    return unwrap(comm, back, state["like"])
