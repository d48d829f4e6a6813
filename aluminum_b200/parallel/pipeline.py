"""Pipeline parallelism: activations move between consecutive stages with Send / Recv on the
device communicator (the reference's primitives: include/Al.hpp:1565-1741)."""
from __future__ import annotations

import torch


def send_forward(comm, activation, to_stage: int, nonblocking: bool = True):
    return comm.send(activation.contiguous(), to_stage, nonblocking=nonblocking)


def recv_forward(comm, buffer, from_stage: int, nonblocking: bool = False):
    return comm.recv(buffer, from_stage, nonblocking=nonblocking)


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
