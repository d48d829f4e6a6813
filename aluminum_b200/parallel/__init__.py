"""Parallelism helpers built on the communicators.

``ddp``      data parallel: bucketed, overlapped gradient allreduce + fused SGD
``host_ddp`` the same on CPU tensors over the host communicator (shared memory or sockets)
``trainer``  end-to-end training loop (host batches in, losses out)
``tensor``   tensor parallel linear layers (column / row) on allgather / allreduce
``sequence`` Megatron-style sequence parallel: reduce-scatter / allgather along the sequence
``expert``   expert parallel token dispatch / combine on alltoall(v)
``context``  ring rotation of key / value blocks for blockwise (ring) attention
``ulysses``  sequence <-> head transposition on alltoall
``pipeline`` stage-to-stage activation transfer on send / recv
"""
from .ddp import DataParallel
from .trainer import Trainer

__all__ = ["DataParallel", "Trainer"]
