"""Data-parallel training on the device communicator.

The pattern is the one Aluminum was written for: start a non-blocking
allreduce for a bucket of gradients as soon as backward has produced it, on a
communicator bound to the compute stream, and join with ``Wait`` before the
optimizer (include/Al.hpp:196 + nccl_impl.hpp:331-347,1421-1429 of the
reference).  Differences from a stock DDP:

* parameters, gradients and momentum live in three flat fp32 buffers;
  gradients are bucketed (25 MB by default) in reverse parameter order and each
  ``param.grad`` is a view into its bucket, so no gather/scatter copies exist;
* the flat gradient buffer is allocated from the communicator's symmetric
  memory: with NVLS the allreduce runs zero-copy on it (multimem.ld_reduce /
  multimem.st), otherwise it is staged by the two-shot kernel;
* the 1/world scale is fused into the allreduce kernel and the optimizer is one
  fused momentum-SGD launch over the whole model that also re-zeroes the
  gradients.
"""
from __future__ import annotations

from typing import List, Optional

import torch
from torch import nn

from ..ops.elementwise import sgd_momentum_step


class _Bucket:
    __slots__ = ("lo", "hi", "pending", "total", "req", "view")

    def __init__(self, lo: int, hi: int):
        self.lo, self.hi = lo, hi
        self.pending = self.total = 0
        self.req = None
        self.view = None


class DataParallel:
    """Wraps a module: flat buffers, bucketed overlapped gradient allreduce, fused SGD."""

    def __init__(self, module: nn.Module, comm=None, bucket_bytes: int = 25 * 1024 * 1024, lr: float = 0.1,
                 momentum: float = 0.9, weight_decay: float = 0.0, wire_dtype: Optional[torch.dtype] = None,
                 symmetric_grads: bool = True, timeline: bool = False):
        self.module = module
        self.comm = comm
        self.world = comm.size if comm is not None else 1
        self.lr, self.momentum, self.weight_decay = lr, momentum, weight_decay
        self.wire_dtype = wire_dtype
        self.steps = 0
        self.launches = 0  # kernels of this library launched so far (allreduces + optimizer steps)
        # Optional per-step timeline (CUDA events on the compute stream): when each bucket became ready, when
        # backward ended, when each bucket's averaged gradients were available to the optimizer.
        self.timeline = timeline
        self._tl_ready, self._tl_avail = {}, {}
        self._tl_bwd_end = self._tl_done = self._tl_start = None
        self.timeline_log: List[dict] = []

        params = [p for p in module.parameters() if p.requires_grad]
        assert all(p.dtype == torch.float32 and p.is_cuda for p in params), "fp32 CUDA parameters expected"
        # Reverse order: the gradients produced first by backward fill the first bucket.
        order = list(reversed(params))
        offsets, total = [], 0
        for p in order:
            offsets.append(total)
            total += (p.numel() + 3) // 4 * 4  # keep every tensor 16-byte aligned inside the flat buffers
        self.numel = total
        dev = params[0].device
        self.flat_param = torch.zeros(total, device=dev, dtype=torch.float32)
        self.flat_mom = torch.zeros(total, device=dev, dtype=torch.float32)
        if self.world > 1 and symmetric_grads and comm is not None and not comm.emulated:
            self.flat_grad = comm.symm_empty((total,), torch.float32)
            self.flat_grad.zero_()
        else:
            self.flat_grad = torch.zeros(total, device=dev, dtype=torch.float32)

        # Buckets over the flat gradient buffer.
        per = max(1, bucket_bytes // 4)
        self.buckets: List[_Bucket] = []
        self._bucket_of = {}
        cur = _Bucket(0, 0)
        for p, off in zip(order, offsets):
            end = off + (p.numel() + 3) // 4 * 4
            if cur.hi > cur.lo and end - cur.lo > per:
                self.buckets.append(cur)
                cur = _Bucket(off, off)
            cur.hi = end
            cur.total += 1
            self._bucket_of[p] = cur
        self.buckets.append(cur)
        for b in self.buckets:
            b.view = self.flat_grad[b.lo:b.hi]
            b.pending = b.total

        # Re-point parameters and gradients at the flat buffers.
        with torch.no_grad():
            for p, off in zip(order, offsets):
                n = p.numel()
                self.flat_param[off:off + n].copy_(p.reshape(-1))
                fmt = torch.channels_last if (p.dim() == 4 and p.is_contiguous(memory_format=torch.channels_last)
                                              and not p.is_contiguous()) else None
                if fmt is not None:
                    # keep channels-last weights physically channels-last inside the flat buffer
                    view = self.flat_param[off:off + n].view(p.shape[0], p.shape[2], p.shape[3], p.shape[1]).permute(0, 3, 1, 2)
                    view.copy_(p)
                    gview = self.flat_grad[off:off + n].view(p.shape[0], p.shape[2], p.shape[3], p.shape[1]).permute(0, 3, 1, 2)
                else:
                    view = self.flat_param[off:off + n].view(p.shape)
                    gview = self.flat_grad[off:off + n].view(p.shape)
                p.data = view
                p.grad = gview
        if self.world > 1:
            for p in order:
                p.register_post_accumulate_grad_hook(self._on_grad)
            self.broadcast_parameters()

    # ------------------------------------------------------------------------------------------
    def broadcast_parameters(self, root: int = 0) -> None:
        """Make every rank start from rank `root`'s parameters (and buffers)."""
        if self.world == 1:
            return
        self.comm.bcast(self.flat_param, root=root)
        for b in self.module.buffers():
            if b.is_floating_point() and b.numel():
                t = b.contiguous()
                self.comm.bcast(t, root=root)
                if t.data_ptr() != b.data_ptr():
                    b.copy_(t)

    def _on_grad(self, p: torch.Tensor) -> None:
        b = self._bucket_of[p]
        b.pending -= 1
        if b.pending == 0:
            if self.timeline:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                self._tl_ready[id(b)] = ev
            # Bucket complete: average it across ranks in the background.
            b.req = self.comm.allreduce(b.view, op="sum", scale=1.0 / self.world, nonblocking=True,
                                        wire_dtype=self.wire_dtype)
            self.launches += 1

    def __call__(self, *a, **kw):
        return self.module(*a, **kw)

    def finish_gradients(self) -> None:
        """Join every outstanding bucket allreduce on the compute stream (host does not block)."""
        if self.timeline:
            self._tl_bwd_end = torch.cuda.Event(enable_timing=True)
            self._tl_bwd_end.record()
        for b in self.buckets:
            if b.req is not None:
                b.req.wait()
                b.req = None
                if self.timeline:
                    ev = torch.cuda.Event(enable_timing=True)
                    ev.record()
                    self._tl_avail[id(b)] = ev
            b.pending = b.total

    def step(self) -> None:
        """Wait for the gradient allreduces, then one fused SGD launch that also zeroes the gradients."""
        self.finish_gradients()
        sgd_momentum_step(self.flat_param, self.flat_mom, self.flat_grad, self.lr, self.momentum, self.weight_decay,
                          1.0, first_step=(self.steps == 0), zero_grad=True)
        self.launches += 1
        self.steps += 1

    def mark_step_start(self) -> None:
        """Timeline mode: call at the start of a step (before forward)."""
        if self.timeline:
            self._tl_start = torch.cuda.Event(enable_timing=True)
            self._tl_start.record()

    def collect_timeline(self) -> Optional[dict]:
        """Timeline mode: synchronise and return this step's record (milliseconds relative to the end of backward):
        when each bucket was handed to the allreduce, when its result was available, and the exposed tail."""
        if not self.timeline or self._tl_bwd_end is None:
            return None
        torch.cuda.synchronize()
        end = self._tl_bwd_end
        rec = {"buckets": []}
        if self._tl_start is not None:
            rec["step_start_ms"] = -self._tl_start.elapsed_time(end)
        last = 0.0
        for i, b in enumerate(self.buckets):
            r, a = self._tl_ready.get(id(b)), self._tl_avail.get(id(b))
            if r is None or a is None:
                continue
            avail = end.elapsed_time(a)
            rec["buckets"].append({"bucket": i, "mbytes": (b.hi - b.lo) * 4 / 1e6, "ready_ms": -r.elapsed_time(end),
                                   "available_ms": avail})
            last = max(last, avail)
        rec["exposed_tail_ms"] = last
        self._tl_ready.clear(); self._tl_avail.clear()
        self.timeline_log.append(rec)
        return rec

    def state_dict(self) -> dict:
        return {"model": self.module.state_dict(), "momentum": self.flat_mom.clone(), "steps": self.steps}

    def load_state_dict(self, sd: dict) -> None:
        self.module.load_state_dict(sd["model"])
        self.flat_mom.copy_(sd["momentum"])
        self.steps = int(sd["steps"])
