"""Data-parallel training on the host communicator (CPU tensors).

The original use of the reference library: while backward is still running on
the caller's thread, the progress thread averages the gradient buckets that are
already complete (``NonblockingAllreduce`` + ``Wait``, include/Al.hpp:196 and
include/aluminum/mpi_impl.hpp of the reference).  Same layout as the GPU
:class:`~aluminum_b200.parallel.ddp.DataParallel`: flat fp32 parameter,
gradient and momentum buffers, gradients bucketed in reverse parameter order,
every ``param.grad`` a view into its bucket.  Works over shared memory inside a
node and over sockets between nodes, so a cluster without GPUs (or the CPU part
of a hybrid job) trains through the same code.
"""
from __future__ import annotations

from typing import List

import numpy as np
import torch
from torch import nn


class _Bucket:
    __slots__ = ("lo", "hi", "pending", "total", "req", "view")

    def __init__(self, lo: int):
        self.lo = self.hi = lo
        self.pending = self.total = 0
        self.req = None
        self.view = None


class HostDataParallel:
    """Flat buffers, bucketed overlapped gradient averaging, momentum SGD - all on CPU tensors."""

    def __init__(self, module: nn.Module, comm=None, bucket_bytes: int = 25 * 1024 * 1024, lr: float = 0.1,
                 momentum: float = 0.9, weight_decay: float = 0.0):
        self.module, self.comm = module, comm
        self.world = comm.size if comm is not None else 1
        self.lr, self.momentum, self.weight_decay = lr, momentum, weight_decay
        self.steps = 0
        params = [p for p in module.parameters() if p.requires_grad]
        assert all(p.dtype == torch.float32 and not p.is_cuda for p in params), "fp32 CPU parameters expected"
        order = list(reversed(params))  # the gradients backward produces first fill the first bucket
        offsets, total = [], 0
        for p in order:
            offsets.append(total)
            total += p.numel()
        self.flat_param = torch.zeros(total)
        self.flat_grad = torch.zeros(total)
        self.flat_mom = torch.zeros(total)
        per = max(1, bucket_bytes // 4)
        self.buckets: List[_Bucket] = []
        self._bucket_of = {}
        cur = _Bucket(0)
        for p, off in zip(order, offsets):
            end = off + p.numel()
            if cur.hi > cur.lo and end - cur.lo > per:
                self.buckets.append(cur)
                cur = _Bucket(off)
            cur.hi = end
            cur.total += 1
            self._bucket_of[p] = cur
        self.buckets.append(cur)
        for b in self.buckets:
            b.view = self.flat_grad[b.lo:b.hi].numpy()  # shares memory with the gradients
            b.pending = b.total
        with torch.no_grad():
            for p, off in zip(order, offsets):
                n = p.numel()
                self.flat_param[off:off + n].copy_(p.reshape(-1))
                p.data = self.flat_param[off:off + n].view(p.shape)
                p.grad = self.flat_grad[off:off + n].view(p.shape)
        if self.world > 1:
            for p in order:
                p.register_post_accumulate_grad_hook(self._on_grad)
            self.broadcast_parameters()

    def broadcast_parameters(self, root: int = 0) -> None:
        if self.world == 1:
            return
        self.comm.bcast(self.flat_param.numpy(), root=root)
        for b in self.module.buffers():
            if b.is_floating_point() and b.numel():
                t = b.contiguous()
                self.comm.bcast(t.numpy(), root=root)
                if t.data_ptr() != b.data_ptr():
                    b.copy_(t)

    def _on_grad(self, p: torch.Tensor) -> None:
        b = self._bucket_of[p]
        b.pending -= 1
        if b.pending == 0:
            b.req = self.comm.allreduce(b.view, op="avg", nonblocking=True)  # the progress thread takes over

    def __call__(self, *a, **kw):
        return self.module(*a, **kw)

    def finish_gradients(self) -> None:
        for b in self.buckets:
            if b.req is not None:
                b.req.wait()
                b.req = None
            b.pending = b.total

    def step(self) -> None:
        self.finish_gradients()
        g = self.flat_grad
        if self.weight_decay:
            g = g.add(self.flat_param, alpha=self.weight_decay)
        if self.steps == 0:
            self.flat_mom.copy_(g)
        else:
            self.flat_mom.mul_(self.momentum).add_(g)
        self.flat_param.add_(self.flat_mom, alpha=-self.lr)
        self.flat_grad.zero_()
        self.steps += 1

    def rebuild(self, comm, root: int = 0) -> None:
        """Continue on another communicator, typically the survivors' after a rank was lost
        (``HostComm.from_ranks(al.alive_ranks())``).  Collective over the new communicator.  Whatever the
        failed step left behind is dropped: unfinished requests, partly averaged gradients.  Parameters,
        buffers and momentum are taken from `root` of the new communicator, so the replicas are equal again
        whichever of them had got how far."""
        for b in self.buckets:
            b.req = None
            b.pending = b.total
        self.flat_grad.zero_()
        had_hooks = self.world > 1
        self.comm, self.world = comm, comm.size
        if self.world > 1:
            if not had_hooks:
                for p in self._bucket_of:
                    p.register_post_accumulate_grad_hook(self._on_grad)
            self.broadcast_parameters(root)
            self.comm.bcast(self.flat_mom.numpy(), root=root)
            steps = np.array([self.steps], dtype=np.int64)
            self.comm.bcast(steps, root=root)
            self.steps = int(steps[0])

    def state_dict(self) -> dict:
        return {"model": self.module.state_dict(), "momentum": self.flat_mom.clone(), "steps": self.steps}

    def load_state_dict(self, sd: dict) -> None:
        self.module.load_state_dict(sd["model"])
        self.flat_mom.copy_(sd["momentum"])
        self.steps = int(sd["steps"])
