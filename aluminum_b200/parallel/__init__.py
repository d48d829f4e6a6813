"""Parallelism helpers built on the device communicator.

``ddp``      data parallel: bucketed, overlapped gradient allreduce + fused SGD
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
