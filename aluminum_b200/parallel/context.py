"""Context parallelism / ring attention: the sequence is sharded, every rank keeps its queries
and the key / value blocks travel around the ring (SendRecv to the next rank, from the previous
one) while partial attention is accumulated with a running log-sum-exp.  The reference exercises
the same ring pattern with Put / SendRecv (test/test_rma_ring.cpp:38-108)."""
from __future__ import annotations

import math

import torch

from ._util import local_ranks, unwrap, wrap


def ring_pass(comm, bufs_send, bufs_recv, nonblocking: bool = False):
    """Every rank sends its buffer to rank+1 and receives rank-1's (one fused kernel launch).  With
    ``nonblocking`` the transfer runs on the communicator's internal stream and a request is returned."""
    p = comm.size
    sends, recvs = wrap(comm, bufs_send), wrap(comm, bufs_recv)
    items = []
    for i, r in enumerate(local_ranks(comm)):
        items.append((True, (r + 1) % p, sends[i], r))
        items.append((False, (r - 1) % p, recvs[i], r))
    return comm.p2p(items, nonblocking=nonblocking)


def ring_attention(comm, q, k, v):
    """Non-causal attention over the full (sharded) sequence.  q, k, v: (s_local, h, d) per rank."""
    p = comm.size
    qs, ks, vs = wrap(comm, q), wrap(comm, k), wrap(comm, v)
    scale = 1.0 / math.sqrt(qs[0].shape[-1])
    acc = [torch.zeros_like(x, dtype=torch.float32) for x in qs]
    lse = [torch.full(x.shape[:2], -float("inf"), device=x.device, dtype=torch.float32) for x in qs]
    kv = [torch.stack([a, b]).contiguous() for a, b in zip(ks, vs)]
    nxt = [torch.empty_like(t) for t in kv]
    for step in range(p):
        # Double buffering: the next key / value block travels (internal stream) while this one is used.
        req = ring_pass(comm, kv, nxt, nonblocking=True) if step + 1 < p else None
        for i in range(len(qs)):
            kk, vv = kv[i][0].float(), kv[i][1].float()
            s = torch.einsum("qhd,khd->qhk", qs[i].float(), kk) * scale
            blk_lse = torch.logsumexp(s, dim=-1)
            new_lse = torch.logaddexp(lse[i], blk_lse)
            acc[i] = acc[i] * torch.exp(lse[i] - new_lse).unsqueeze(-1) + \
                torch.einsum("qhk,khd->qhd", torch.exp(s - new_lse.unsqueeze(-1)), vv)
            lse[i] = new_lse
        if req is not None:
            req.wait()  # the compute stream waits for the transfer; the host does not
            kv, nxt = nxt, kv
    return unwrap(comm, [a.to(qs[0].dtype) for a in acc], q)
