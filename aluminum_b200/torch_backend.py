"""``torch.distributed`` backend "aluminum": PyTorch programs written against
``torch.distributed`` (DistributedDataParallel included) run on this library
without change::

    import aluminum_b200.torch_backend          # registers the backend
    torch.distributed.init_process_group("aluminum")

CPU tensors go through the host communicator (shared memory inside a node,
sockets between nodes), CUDA tensors through the device communicator (the
library's own NVLink kernels) on the current CUDA stream.  Ranks are taken from
the launcher's environment exactly as for the rest of the package (torchrun,
``alrun``, Open MPI, Slurm); the ``store`` PyTorch hands over is not needed.

The reference library has no PyTorch integration (its consumer, LBANN, is a C++
framework calling ``Al::`` directly); this module plays that role for PyTorch users.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from . import comm as _comm

_REDUCE_OPS = {
    dist.ReduceOp.SUM: "sum", dist.ReduceOp.PRODUCT: "prod", dist.ReduceOp.MIN: "min", dist.ReduceOp.MAX: "max",
    dist.ReduceOp.BAND: "band", dist.ReduceOp.BOR: "bor", dist.ReduceOp.BXOR: "bxor", dist.ReduceOp.AVG: "avg",
}


def _op_name(op) -> str:
    for k, v in _REDUCE_OPS.items():
        if op == k:
            return v
    raise _comm.AlError(f"reduction {op} is not supported by the aluminum backend")


def _tensors_in(x):
    if isinstance(x, torch.Tensor):
        yield x
    elif isinstance(x, (list, tuple)):
        for y in x:
            yield from _tensors_in(y)


class _Work(dist._Work):
    """Completed-on-return work handle.  Host operations have finished when the call returns; device
    operations are enqueued on the current CUDA stream, so later kernels on that stream are ordered
    after them, which is all ``wait()`` promises for CUDA tensors."""

    def __init__(self, result):
        super().__init__()
        self._result = result
        devices = sorted({t.device for t in _tensors_in(result) if t.is_cuda}, key=str)
        # a future that carries CUDA tensors has to know their devices; the values are ordered on the
        # current stream, which set_result records
        self._future = torch.futures.Future(devices=devices) if devices else torch.futures.Future()
        self._future.set_result(result)

    def wait(self, timeout=None):
        return True

    def is_completed(self):
        return True

    def is_success(self):
        return True

    def result(self):
        return self._result

    def get_future(self):
        return self._future


class AluminumProcessGroup(dist.ProcessGroup):
    """One process group = one host communicator plus, on first use with CUDA tensors, one device communicator."""

    def __init__(self, rank: int, size: int, global_ranks: Optional[List[int]] = None):
        super().__init__(rank, size)
        _comm.init()
        self._ranks = list(global_ranks) if global_ranks else list(range(size))
        if _comm.world_size() < size:
            raise _comm.AlError(f"the launcher started {_comm.world_size()} ranks, the process group wants {size}")
        self._host = _comm.HostComm.from_ranks(self._ranks)
        if self._host.rank != rank:
            raise _comm.AlError(f"rank mismatch: torch.distributed says {rank}, the library says {self._host.rank}")
        self._dev = None

    # ---- plumbing ---------------------------------------------------------------------------
    def getBackendName(self):
        return "aluminum"

    def _c(self, t: torch.Tensor):
        if t.is_cuda:
            if self._dev is None:
                from .device import DeviceComm
                self._dev = DeviceComm.from_ranks(self._ranks)
            return self._dev
        return self._host

    @staticmethod
    def _flat(t: torch.Tensor) -> torch.Tensor:
        return t if t.is_contiguous() else t.contiguous()

    @staticmethod
    def _one(tensors):
        if len(tensors) != 1:
            raise _comm.AlError("the aluminum backend takes one tensor per rank and call")
        return tensors[0]

    def _inplace(self, t: torch.Tensor, fn):
        """Run fn(buffer) on a contiguous view or copy of t and write the result back into t."""
        buf = self._flat(t)
        if buf.dtype == torch.bool:
            work = buf.to(torch.uint8)
            fn(work)
            t.copy_(work.to(torch.bool))
            return
        fn(buf)
        if buf is not t:
            t.copy_(buf)

    # ---- collectives ------------------------------------------------------------------------
    def allreduce(self, tensors, opts=None):
        t = self._one(tensors)
        op = _op_name(opts.reduceOp) if opts is not None else "sum"
        self._inplace(t, lambda b: self._c(b).allreduce(b.view(-1), op=op))
        return _Work(tensors)

    def allreduce_coalesced(self, tensors, opts=None):
        for t in tensors:
            self.allreduce([t], opts)
        return _Work(tensors)

    def broadcast(self, tensors, opts=None):
        t = self._one(tensors)
        root = opts.rootRank if opts is not None else 0
        self._inplace(t, lambda b: self._c(b).bcast(b.view(-1), root=root))
        return _Work(tensors)

    def reduce(self, tensors, opts=None):
        t = self._one(tensors)
        op = _op_name(opts.reduceOp) if opts is not None else "sum"
        root = opts.rootRank if opts is not None else 0
        if self.rank() == root:
            self._inplace(t, lambda b: self._c(b).reduce(b.view(-1), op=op, root=root))
        else:  # only the root's tensor changes
            b = self._flat(t).clone()
            self._c(b).reduce(b.view(-1), op=op, root=root)
        return _Work(tensors)

    def _allgather_flat(self, out: torch.Tensor, inp: torch.Tensor):
        self._c(inp).allgather(self._flat(inp).view(-1), out.view(-1))

    def allgather(self, output_tensors, input_tensors, opts=None):
        inp = self._one(input_tensors)
        outs = self._one(output_tensors)
        flat = torch.empty(self.size() * inp.numel(), dtype=inp.dtype, device=inp.device)
        self._allgather_flat(flat, inp)
        for r, o in enumerate(outs):
            o.copy_(flat[r * inp.numel():(r + 1) * inp.numel()].view_as(o))
        return _Work(output_tensors)

    def _allgather_base(self, output, input, opts=None):
        if output.is_contiguous():
            self._allgather_flat(output, input)
        else:
            flat = torch.empty(output.numel(), dtype=output.dtype, device=output.device)
            self._allgather_flat(flat, input)
            output.copy_(flat.view_as(output))
        return _Work(output)

    def allgather_coalesced(self, output_lists, input_tensors, opts=None):
        for outs, inp in zip(output_lists, input_tensors):
            self.allgather([outs], [inp], opts)
        return _Work(output_lists)

    def allgather_into_tensor_coalesced(self, outputs, inputs, opts=None):
        for o, i in zip(outputs, inputs):
            self._allgather_base(o, i, opts)
        return _Work(outputs)

    def _reduce_scatter_flat(self, out: torch.Tensor, inp: torch.Tensor, op: str):
        self._c(inp).reduce_scatter(self._flat(inp).view(-1), out.view(-1), op=op)

    def reduce_scatter(self, output_tensors, input_tensors, opts=None):
        out = self._one(output_tensors)
        ins = self._one(input_tensors)
        op = _op_name(opts.reduceOp) if opts is not None else "sum"
        flat = torch.cat([self._flat(t).view(-1) for t in ins])
        res = out if out.is_contiguous() else torch.empty_like(out, memory_format=torch.contiguous_format)
        self._reduce_scatter_flat(res, flat, op)
        if res is not out:
            out.copy_(res)
        return _Work(output_tensors)

    def _reduce_scatter_base(self, output, input, opts=None):
        op = _op_name(opts.reduceOp) if opts is not None else "sum"
        res = output if output.is_contiguous() else torch.empty_like(output, memory_format=torch.contiguous_format)
        self._reduce_scatter_flat(res, input, op)
        if res is not output:
            output.copy_(res)
        return _Work(output)

    def reduce_scatter_tensor_coalesced(self, outputs, inputs, opts=None):
        for o, i in zip(outputs, inputs):
            self._reduce_scatter_base(o, i, opts)
        return _Work(outputs)

    def alltoall_base(self, output, input, output_split_sizes, input_split_sizes, opts=None):
        c = self._c(input)
        inp = self._flat(input)
        res = output if output.is_contiguous() else torch.empty_like(output, memory_format=torch.contiguous_format)
        if not output_split_sizes and not input_split_sizes:
            c.alltoall(inp.view(-1), res.view(-1))
        else:
            p = self.size()
            row_in = inp.numel() // inp.shape[0] if inp.dim() > 1 and inp.shape[0] else 1
            row_out = res.numel() // res.shape[0] if res.dim() > 1 and res.shape[0] else 1
            ins = list(input_split_sizes) if input_split_sizes else [inp.shape[0] // p] * p
            outs = list(output_split_sizes) if output_split_sizes else [res.shape[0] // p] * p
            sc = [n * row_in for n in ins]
            rc = [n * row_out for n in outs]
            sd = [sum(sc[:i]) for i in range(p)]
            rd = [sum(rc[:i]) for i in range(p)]
            c.alltoallv(inp.view(-1), sc, sd, res.view(-1), rc, rd)
        if res is not output:
            output.copy_(res)
        return _Work(output)

    def alltoall(self, output_tensors, input_tensors, opts=None):
        p = self.size()
        sc = [t.numel() for t in input_tensors]
        rc = [t.numel() for t in output_tensors]
        send = torch.cat([self._flat(t).view(-1) for t in input_tensors])
        recv = torch.empty(sum(rc), dtype=send.dtype, device=send.device)
        sd = [sum(sc[:i]) for i in range(p)]
        rd = [sum(rc[:i]) for i in range(p)]
        self._c(send).alltoallv(send, sc, sd, recv, rc, rd)
        for r, o in enumerate(output_tensors):
            o.copy_(recv[rd[r]:rd[r] + rc[r]].view_as(o))
        return _Work(output_tensors)

    def gather(self, output_tensors, input_tensors, opts=None):
        inp = self._one(input_tensors)
        root = opts.rootRank if opts is not None else 0
        src = self._flat(inp).view(-1)
        if self.rank() == root:
            outs = self._one(output_tensors)
            flat = torch.empty(self.size() * inp.numel(), dtype=inp.dtype, device=inp.device)
            self._c(inp).gather(src, flat, root=root)
            for r, o in enumerate(outs):
                o.copy_(flat[r * inp.numel():(r + 1) * inp.numel()].view_as(o))
        else:
            self._c(inp).gather(src, None, root=root)
        return _Work(output_tensors)

    def scatter(self, output_tensors, input_tensors, opts=None):
        out = self._one(output_tensors)
        root = opts.rootRank if opts is not None else 0
        res = out if out.is_contiguous() else torch.empty_like(out, memory_format=torch.contiguous_format)
        if self.rank() == root:
            flat = torch.cat([self._flat(t).view(-1) for t in self._one(input_tensors)])
            self._c(out).scatter(flat, res.view(-1), root=root)
        else:
            self._c(out).scatter(None, res.view(-1), root=root)
        if res is not out:
            out.copy_(res)
        return _Work(output_tensors)

    def barrier(self, opts=None):
        self._host.barrier()
        return _Work(None)

    # ---- point to point ------------------------------------------------------------------------
    def send(self, tensors, dst, tag=0):
        t = self._flat(self._one(tensors))
        self._c(t).send(t.view(-1), dst)
        return _Work(tensors)

    def recv(self, tensors, src, tag=0):
        t = self._one(tensors)
        self._inplace(t, lambda b: self._c(b).recv(b.view(-1), src))
        return _Work(tensors)

    def __repr__(self):
        return f"AluminumProcessGroup(rank={self.rank()}, size={self.size()})"


def _create(dist_backend_opts, backend_options=None):
    ranks = list(getattr(dist_backend_opts, "global_ranks_in_group", []) or [])
    return AluminumProcessGroup(dist_backend_opts.group_rank, dist_backend_opts.group_size, ranks)


def register() -> None:
    """Idempotent registration with torch.distributed (done on import)."""
    if "ALUMINUM" not in getattr(dist.Backend, "_plugins", {}):
        dist.Backend.register_backend("aluminum", _create, extended_api=True, devices=["cpu", "cuda"])


register()
