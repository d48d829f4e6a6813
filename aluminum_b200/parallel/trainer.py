"""Training loop around :class:`DataParallel`: host batches in, losses out.

``Trainer.run`` is the end-to-end entry point: it takes an iterator of
``(inputs, labels)`` in pinned host memory, uploads each batch on a copy stream
while the previous step computes (two device slots), runs forward / backward
under bf16 autocast with the overlapped gradient allreduce, applies the fused
optimizer and yields the loss of every step as a Python float (a device-to-host
read per step).
"""
from __future__ import annotations

from typing import Iterable, Iterator, Tuple

import torch
from torch import nn

from .ddp import DataParallel


class Trainer:
    def __init__(self, dp: DataParallel, loss_fn: nn.Module | None = None, autocast_dtype=torch.bfloat16,
                 channels_last: bool = True):
        self.dp = dp
        self.loss_fn = loss_fn if loss_fn is not None else nn.CrossEntropyLoss()
        self.autocast_dtype = autocast_dtype
        self.channels_last = channels_last
        self.copy_stream = torch.cuda.Stream()
        self._slots = [None, None]
        self._slot_free = [None, None]   # event: the step that consumed the slot has been enqueued and finished
        self._slot_ready = [None, None]  # event: the upload into the slot finished
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    # ---- one optimisation step on device-resident data -------------------------------------------
    def step_device(self, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        if self.channels_last and x.dim() == 4:
            x = x.contiguous(memory_format=torch.channels_last)  # one device pass; the upload itself stays a plain copy
        with torch.autocast("cuda", dtype=self.autocast_dtype, enabled=self.autocast_dtype is not None):
            out = self.dp(x)
            loss = self.loss_fn(out.float(), y)
        loss.backward()
        self.dp.step()
        return loss.detach()

    # ---- host -> device staging ---------------------------------------------------------------------
    def _upload(self, slot: int, batch: Tuple[torch.Tensor, torch.Tensor]):
        xh, yh = batch
        with torch.cuda.stream(self.copy_stream):
            if self._slot_free[slot] is not None:
                self.copy_stream.wait_event(self._slot_free[slot])
            if self._slots[slot] is None or self._slots[slot][0].shape != xh.shape:
                xd = torch.empty(xh.shape, device="cuda", dtype=xh.dtype)
                yd = torch.empty(yh.shape, device="cuda", dtype=yh.dtype)
                self._slots[slot] = (xd, yd)
            xd, yd = self._slots[slot]
            xd.copy_(xh, non_blocking=True)
            yd.copy_(yh, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.copy_stream)
            self._slot_ready[slot] = ev
        self.h2d_bytes += xh.numel() * xh.element_size() + yh.numel() * yh.element_size()

    def run(self, batches: Iterable[Tuple[torch.Tensor, torch.Tensor]]) -> Iterator[float]:
        """Consume host batches; yield one loss value per step."""
        it = iter(batches)
        try:
            first = next(it)
        except StopIteration:
            return
        slot = 0
        self._upload(slot, first)
        while True:
            try:
                nxt = next(it)
            except StopIteration:
                nxt = None
            if nxt is not None:
                self._upload(1 - slot, nxt)  # overlaps with this step's compute
            torch.cuda.current_stream().wait_event(self._slot_ready[slot])
            xd, yd = self._slots[slot]
            loss = self.step_device(xd, yd)
            done = torch.cuda.Event()
            done.record(torch.cuda.current_stream())
            self._slot_free[slot] = done
            value = float(loss.item())  # device -> host read of the step's result
            self.d2h_bytes += 4
            yield value
            if nxt is None:
                return
            slot = 1 - slot
