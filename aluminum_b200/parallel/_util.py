"""Helpers shared by the parallelism modules.

Every helper works on "rank lists": outside emulation a list with the one local tensor, in
emulation (all ranks in one process, used by the single-GPU tests) one tensor per rank.  ``wrap``
and ``unwrap`` convert between what the caller passed and that list form.
"""
from __future__ import annotations

import torch


def wrap(comm, x):
    if isinstance(x, (list, tuple)):
        return list(x)
    return [x]


def unwrap(comm, xs, like):
    if isinstance(like, (list, tuple)):
        return xs
    return xs[0]


def local_ranks(comm):
    """Ranks executed by this process: all of them in emulation, otherwise just this rank."""
    return list(range(comm.size)) if comm.nlocal > 1 else [comm.rank]


def call(comm, fn, *lists, **kw):
    """Invoke a communicator method with rank lists (emulation) or single tensors."""
    if comm.nlocal > 1:
        return fn(*lists, **kw)
    return fn(*[(l[0] if (isinstance(l, list) and len(l) == 1 and torch.is_tensor(l[0])) else l) for l in lists], **kw)
