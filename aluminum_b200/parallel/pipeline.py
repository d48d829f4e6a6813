"""Pipeline parallelism: activations (forward) and their gradients (backward) move between consecutive
stages with Send / Recv on the device communicator (the reference's primitives: include/Al.hpp:1565-1741).

:class:`PipelineStage` wraps the module of one stage and runs a GPipe-style schedule over micro-batches: all
forwards, then all backwards in reverse order.  Sends are non-blocking (they travel on the communicator's
internal stream while the next micro-batch computes); receives are stream-ordered.  Every stage keeps the
input / output tensors of its micro-batches so that ``backward`` can replay autograd with the gradient
received from the next stage.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
from torch import nn


def send_forward(comm, activation, to_stage: int, nonblocking: bool = True):
    return comm.send(activation.contiguous(), to_stage, nonblocking=nonblocking)


def recv_forward(comm, buffer, from_stage: int, nonblocking: bool = False):
    return comm.recv(buffer, from_stage, nonblocking=nonblocking)


class PipelineStage:
    """One stage of a linear pipeline over the ranks ``stages`` (in order) of ``comm``."""

    def __init__(self, comm, module: nn.Module, stages: Optional[Sequence[int]] = None):
        self.comm, self.module = comm, module
        self.stages = list(stages) if stages is not None else list(range(comm.size))
        self.index = self.stages.index(comm.rank)
        self.prev = self.stages[self.index - 1] if self.index > 0 else None
        self.next = self.stages[self.index + 1] if self.index + 1 < len(self.stages) else None

    @property
    def first(self) -> bool:
        return self.prev is None

    @property
    def last(self) -> bool:
        return self.next is None

    def run(self, microbatches: Sequence[torch.Tensor], act_shape, loss_fn: Optional[Callable] = None,
            targets: Optional[Sequence[torch.Tensor]] = None, out_shape=None, dtype=torch.float32) -> List[torch.Tensor]:
        """Forward all micro-batches, then backward all of them (gradients accumulate in the module's parameters).

        ``microbatches``: the inputs (used by the first stage; only their number matters elsewhere).
        ``act_shape``: shape of the activation this stage receives (ignored on the first stage);
        ``out_shape``: shape of what it sends on (defaults to what the module produces).
        The last stage applies ``loss_fn(output, target)`` and returns the losses; the others return their outputs."""
        comm = self.comm
        n = len(microbatches)
        inputs, outputs, pending = [], [], []
        results: List[torch.Tensor] = []
        # ---- forward ------------------------------------------------------------------------------------
        for i in range(n):
            if self.first:
                x = microbatches[i]
            else:
                x = torch.empty(act_shape, device="cuda", dtype=dtype)
                comm.recv(x, self.prev)
                x.requires_grad_(True)
            y = self.module(x)
            inputs.append(x)
            if self.last:
                y = loss_fn(y, targets[i]) if loss_fn is not None else y
                results.append(y.detach())
            else:
                pending.append(comm.send(y.detach().contiguous(), self.next, nonblocking=True))
                results.append(y.detach())
            outputs.append(y)
        for r in pending:
            r.wait()
        # ---- backward, last micro-batch first ----------------------------------------------------------------
        pending = []
        for i in reversed(range(n)):
            if self.last:
                outputs[i].backward()
            else:
                g = torch.empty_like(outputs[i])
                comm.recv(g, self.next)
                outputs[i].backward(g)
            if not self.first:
                pending.append(comm.send(inputs[i].grad.contiguous(), self.prev, nonblocking=True))
        for r in pending:
            r.wait()
        return results


def run_two_stage(comm, stage_module, microbatches, act_shape, dtype=torch.float32):
    """Forward-only schedule over two stages (ranks 0 and 1): stage 0 sends the activation of
    microbatch i while it computes microbatch i+1; stage 1 receives and finishes them in order."""
    outs = []
    if comm.rank == 0:
        pending = None
        for mb in microbatches:
            act = stage_module(mb)
            if pending is not None:
                pending.wait()
            pending = send_forward(comm, act, 1, nonblocking=True)
            outs.append(act)
        if pending is not None:
            pending.wait()
    elif comm.rank == 1:
        buf = torch.empty(act_shape, device="cuda", dtype=dtype)
        for _ in microbatches:
            recv_forward(comm, buf, 0)
            outs.append(stage_module(buf.clone()))
    return outs
