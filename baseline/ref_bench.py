"""Reference arm of the benchmarks: the unmodified llnl/Aluminum, NCCL backend.

Everything communication-related here goes through ``baseline/_ref`` (the reference built by
``baseline/build_reference.py`` on the single-node MPI stand-in) via ``libref_driver.so``; nothing
of the ``aluminum_b200`` package is imported.  The reference ships no model and no trainer, so the
training loop around it is plain PyTorch written the way its consumers use it (LBANN's pattern,
README.md:9-17 and include/Al.hpp:196 of the reference): torchvision's ResNet-50, gradients in flat
25 MB fp32 buckets, ``Al::NonblockingAllreduce<Al::NCCLBackend>`` (operator ``avg``) per bucket as
soon as backward has filled it, ``Al::Wait`` on the compute stream before ``torch.optim.SGD``.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path
from typing import Iterable, Iterator, List, Tuple

HERE = Path(__file__).resolve().parent
DRIVER = HERE / "_ref" / "lib" / "libref_driver.so"

KINDS = {"allreduce": 0, "reduce_scatter": 1, "allgather": 2, "alltoall": 3}
OPS = {"sum": 0, "prod": 1, "min": 2, "max": 3, "avg": 4}


def unavailable_reason() -> str | None:
    """None when the reference arm can run; otherwise one line saying why not."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("al_build_reference", HERE / "build_reference.py")
    br = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(br)
    if br.driver_is_stale():
        # Only rank 0 of a node rebuilds; the others wait for the file.
        if int(os.environ.get("LOCAL_RANK", "0")) == 0:
            try:
                br.rebuild_driver_only()
            except Exception as e:  # noqa: BLE001
                return (f"{DRIVER.relative_to(HERE.parent)} is missing or older than baseline/ref_driver.cpp and could "
                        f"not be rebuilt ({str(e).splitlines()[-1][:200]}): run `python baseline/build_reference.py`")
        else:
            import time
            for _ in range(600):
                if not br.driver_is_stale():
                    break
                time.sleep(0.1)
    if not DRIVER.exists():
        return (f"{DRIVER.relative_to(HERE.parent)} is missing: run `python baseline/build_reference.py` "
                "(builds the MPI stand-in, the unmodified reference with its NCCL backend and the C driver)")
    return None


class RefAl:
    """ctypes view of libref_driver.so (the reference's public API behind C functions)."""

    def __init__(self, device: int):
        import torch  # loaded first so that the reference shares torch's CUDA runtime and NCCL
        self.torch = torch
        lib = C.CDLL(str(DRIVER), mode=C.RTLD_GLOBAL)
        lib.refal_last_error.restype = C.c_char_p
        lib.refal_version.restype = C.c_char_p
        lib.refal_comm_create.restype = C.c_void_p
        lib.refal_comm_create.argtypes = [C.c_void_p]
        lib.refal_comm_destroy.argtypes = [C.c_void_p]
        lib.refal_rank.argtypes = [C.c_void_p]
        lib.refal_size.argtypes = [C.c_void_p]
        lib.refal_nb_allreduce.restype = C.c_void_p
        lib.refal_nb_allreduce.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int]
        lib.refal_wait.argtypes = [C.c_void_p]
        lib.refal_collective.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int]
        lib.refal_time_collective.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int,
                                              C.c_int, C.c_int, C.POINTER(C.c_float)]
        lib.refal_host_barrier.argtypes = [C.c_void_p]
        lib.refal_host_max.restype = C.c_double
        lib.refal_host_max.argtypes = [C.c_void_p, C.c_double]
        self.lib = lib
        self._check(lib.refal_init(int(device)))
        self.version = lib.refal_version().decode()

    def _check(self, rc: int) -> None:
        if rc != 0:
            raise RuntimeError("reference: " + self.lib.refal_last_error().decode())

    def comm(self, stream) -> "RefComm":
        h = self.lib.refal_comm_create(C.c_void_p(stream.cuda_stream))
        if not h:
            raise RuntimeError("reference: " + self.lib.refal_last_error().decode())
        return RefComm(self, h)

    def finalize(self) -> None:
        self._check(self.lib.refal_finalize())


class RefComm:
    def __init__(self, al: RefAl, handle: int):
        self.al, self.h = al, C.c_void_p(handle)
        self.rank = al.lib.refal_rank(self.h)
        self.size = al.lib.refal_size(self.h)

    @staticmethod
    def _dt(t) -> int:
        name = str(t.dtype)
        if name == "torch.float32":
            return 0
        if name == "torch.bfloat16":
            return 1
        raise TypeError(f"reference driver: dtype {name} not wired")

    def nb_allreduce(self, t, op: str = "sum"):
        """Al::NonblockingAllreduce in place; returns a request for wait()."""
        r = self.al.lib.refal_nb_allreduce(self.h, C.c_void_p(t.data_ptr()), t.numel(), self._dt(t), OPS[op])
        if not r:
            raise RuntimeError("reference: " + self.al.lib.refal_last_error().decode())
        return r

    def wait(self, req) -> None:
        self.al._check(self.al.lib.refal_wait(C.c_void_p(req)))

    def collective(self, kind: str, send, recv, count: int, op: str = "sum") -> None:
        self.al._check(self.al.lib.refal_collective(self.h, KINDS[kind], C.c_void_p(send.data_ptr()),
                                                    C.c_void_p(recv.data_ptr()), count, self._dt(recv), OPS[op]))

    def time_collective(self, kind: str, send, recv, count: int, warmup: int, iters: int, op: str = "sum") -> List[float]:
        out = (C.c_float * iters)()
        self.al._check(self.al.lib.refal_time_collective(self.h, KINDS[kind], C.c_void_p(send.data_ptr()),
                                                         C.c_void_p(recv.data_ptr()), count, self._dt(recv), OPS[op],
                                                         warmup, iters, out))
        return [float(v) for v in out]

    def host_barrier(self) -> None:
        self.al._check(self.al.lib.refal_host_barrier(self.h))

    def host_max(self, v: float) -> float:
        return float(self.al.lib.refal_host_max(self.h, float(v)))

    def close(self) -> None:
        if self.h:
            self.al.lib.refal_comm_destroy(self.h)
            self.h = C.c_void_p(None)


class RefDataParallel:
    """Bucketed gradient averaging through the reference's non-blocking NCCL allreduce."""

    def __init__(self, module, comm: RefComm, bucket_bytes: int = 25 * 1024 * 1024):
        import torch
        self.module, self.comm = module, comm
        params = [p for p in module.parameters() if p.requires_grad]
        order = list(reversed(params))  # backward produces the last layers' gradients first
        offsets, total = [], 0
        for p in order:
            offsets.append(total)
            total += (p.numel() + 3) // 4 * 4
        self.flat_grad = torch.zeros(total, device=params[0].device, dtype=torch.float32)
        per = max(1, bucket_bytes // 4)
        self.buckets = []  # [lo, hi, total, pending, request]
        self._bucket_of = {}
        cur = [0, 0, 0, 0, None]
        for p, off in zip(order, offsets):
            end = off + (p.numel() + 3) // 4 * 4
            if cur[1] > cur[0] and end - cur[0] > per:
                self.buckets.append(cur)
                cur = [off, off, 0, 0, None]
            cur[1] = end
            cur[2] += 1
            self._bucket_of[p] = cur
        self.buckets.append(cur)
        for b in self.buckets:
            b[3] = b[2]
        for p, off in zip(order, offsets):
            n = p.numel()
            if p.dim() == 4 and p.is_contiguous(memory_format=torch.channels_last) and not p.is_contiguous():
                g = self.flat_grad[off:off + n].view(p.shape[0], p.shape[2], p.shape[3], p.shape[1]).permute(0, 3, 1, 2)
            else:
                g = self.flat_grad[off:off + n].view(p.shape)
            p.grad = g
            p.register_post_accumulate_grad_hook(self._on_grad)

    def _on_grad(self, p) -> None:
        b = self._bucket_of[p]
        b[3] -= 1
        if b[3] == 0:
            b[4] = self.comm.nb_allreduce(self.flat_grad[b[0]:b[1]], op="avg")

    def finish_gradients(self) -> None:
        for b in self.buckets:
            if b[4] is not None:
                self.comm.wait(b[4])
                b[4] = None
            b[3] = b[2]


class RefTrainer:
    """forward / backward under bf16 autocast, overlapped gradient averaging, torch.optim.SGD."""

    def __init__(self, model, comm: RefComm, lr: float = 0.1, momentum: float = 0.9):
        import torch
        self.torch = torch
        self.model = model
        self.dp = RefDataParallel(model, comm)
        self.opt = torch.optim.SGD(model.parameters(), lr=lr, momentum=momentum)
        self.loss_fn = torch.nn.CrossEntropyLoss()
        self.copy_stream = torch.cuda.Stream()
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def step_device(self, x, y):
        torch = self.torch
        x = x.contiguous(memory_format=torch.channels_last)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = self.loss_fn(self.model(x).float(), y)
        loss.backward()
        self.dp.finish_gradients()
        self.opt.step()
        self.opt.zero_grad(set_to_none=False)  # gradients are views into the buckets: zero them in place
        return loss.detach()

    def run(self, batches: Iterable[Tuple]) -> Iterator[float]:
        """Pinned host batches in (uploaded on a copy stream, two device slots), one loss value out per step."""
        torch = self.torch
        slots, ready, free = [None, None], [None, None], [None, None]

        def upload(i, batch):
            xh, yh = batch
            with torch.cuda.stream(self.copy_stream):
                if free[i] is not None:
                    self.copy_stream.wait_event(free[i])
                if slots[i] is None:
                    slots[i] = (torch.empty(xh.shape, device="cuda", dtype=xh.dtype),
                                torch.empty(yh.shape, device="cuda", dtype=yh.dtype))
                slots[i][0].copy_(xh, non_blocking=True)
                slots[i][1].copy_(yh, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.copy_stream)
                ready[i] = ev
            self.h2d_bytes += xh.numel() * xh.element_size() + yh.numel() * yh.element_size()

        it = iter(batches)
        try:
            first = next(it)
        except StopIteration:
            return
        i = 0
        upload(i, first)
        while True:
            nxt = next(it, None)
            if nxt is not None:
                upload(1 - i, nxt)
            torch.cuda.current_stream().wait_event(ready[i])
            loss = self.step_device(*slots[i])
            done = torch.cuda.Event()
            done.record(torch.cuda.current_stream())
            free[i] = done
            value = float(loss.item())
            self.d2h_bytes += 4
            yield value
            if nxt is None:
                return
            i = 1 - i
