"""``DeviceComm``: the GPU communicator for PyTorch tensors.

Each call launches one of the library's sm_100a kernels on the current PyTorch
CUDA stream (or on an internal high-priority stream with ``nonblocking=True``).
Outside emulation every argument is one tensor; in emulation (all ranks in one
process on one GPU) every argument is a list with one tensor per rank.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

from . import _lib
from ._lib import ALGOS, DTYPES, KINDS, OPS, PATHS, AlError, check, check_ptr, size_array
from .comm import Request, init


def _code(t) -> int:
    name = str(t.dtype).replace("torch.", "")
    if name not in DTYPES:
        raise AlError(f"unsupported dtype {t.dtype}")
    return DTYPES[name]


def _dtype_code(dtype) -> int:
    return DTYPES[str(dtype).replace("torch.", "")]


class _CudaBlob:
    """Exposes a raw device allocation through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self._owner = owner
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


class DeviceComm:
    def __init__(self, emulate: int = 0, stream=None, _handle=None):
        import torch
        init()
        lib = _lib.load()
        if not lib.al_cuda_available():
            raise AlError("DeviceComm needs a CUDA device")
        self._lib = lib
        self._torch = torch
        s = C.c_void_p(stream.cuda_stream if stream is not None else 0)
        if _handle:
            self._h = C.c_void_p(_handle)
        elif emulate:
            self._h = C.c_void_p(check_ptr(lib.al_dev_comm_create_emulated(int(emulate), s)))
        else:
            self._h = C.c_void_p(check_ptr(lib.al_dev_comm_create(s)))
        self.rank = lib.al_dev_comm_rank(self._h)
        self.size = lib.al_dev_comm_size(self._h)
        self.nlocal = lib.al_dev_comm_nlocal(self._h)
        self.emulated = self.nlocal > 1 or bool(emulate)
        self._symm = {}

    @classmethod
    def from_ranks(cls, world_ranks, stream=None) -> "DeviceComm":
        """Communicator over the listed world ranks, in that order.  Collective over those ranks only."""
        init()
        lib = _lib.load()
        arr = (C.c_int * len(world_ranks))(*[int(r) for r in world_ranks])
        s = C.c_void_p(stream.cuda_stream if stream is not None else 0)
        return cls(stream=stream, _handle=check_ptr(lib.al_dev_comm_create_group(arr, len(world_ranks), s)))

    # ---- properties / diagnostics -----------------------------------------------------
    @property
    def has_multicast(self) -> bool:
        return bool(self._lib.al_dev_comm_has_multicast(self._h))

    @property
    def backing(self) -> str:
        return self._lib.al_dev_comm_backing(self._h).decode()

    def set_timeout_ms(self, ms: float) -> None:
        check(self._lib.al_dev_comm_set_timeout_ms(self._h, float(ms)))

    def abort(self, why: str = "aborted by the caller") -> None:
        """Make every later call on this communicator raise; recovery is a new communicator."""
        check(self._lib.al_dev_comm_abort(self._h, why.encode()))

    def stats(self) -> dict:
        out = (C.c_uint64 * 16)()
        check(self._lib.al_dev_comm_stats(self._h, out))
        names = ["ops", "bytes", "kernels", "timeouts", "one_shot", "two_shot", "nvls", "nvls_zero_copy", "bulk_pipeline",
                 "window", "ll", "rows", "rs_nvls"]
        return dict(zip(names, [int(v) for v in out]))

    def status(self) -> dict:
        out = (C.c_uint64 * 6)()
        self._lib.al_dev_comm_status(self._h, out)
        return dict(zip(["code", "rank", "peer", "where", "epoch", "seen"], [int(v) for v in out]))

    def split(self, color: int, key: int, stream=None) -> "DeviceComm":
        s = C.c_void_p(stream.cuda_stream if stream is not None else 0)
        return DeviceComm(_handle=check_ptr(self._lib.al_dev_comm_split(self._h, color, key, s)))

    def close(self) -> None:
        if self._h:
            self._torch.cuda.synchronize()
            self._lib.al_dev_comm_destroy(self._h)
            self._h = C.c_void_p(None)

    def __del__(self):
        try:
            if self._lib.al_initialized():
                self.close()
        except Exception:
            pass

    # ---- helpers ---------------------------------------------------------------------------
    def _stream(self, stream=None) -> C.c_void_p:
        s = stream if stream is not None else self._torch.cuda.current_stream()
        return C.c_void_p(s.cuda_stream)

    def _as_list(self, x):
        if x is None:
            return [None] * self.nlocal
        if isinstance(x, (list, tuple)):
            if len(x) != self.nlocal:
                raise AlError(f"expected {self.nlocal} tensors (one per local rank), got {len(x)}")
            return list(x)
        if self.nlocal != 1:
            raise AlError("an emulated communicator takes a list with one tensor per rank")
        return [x]

    def _ptrs(self, tensors):
        arr = (C.c_void_p * self.nlocal)()
        for i, t in enumerate(tensors):
            if t is None:
                arr[i] = None
                continue
            if not t.is_cuda or not t.is_contiguous():
                raise AlError("device buffers must be contiguous CUDA tensors")
            arr[i] = t.data_ptr()
        return arr

    def _tables(self, tables):
        """Flatten {name: rows} into four ctypes arrays of nlocal*size entries (or None)."""
        out = []
        for name in ("send_counts", "send_displs", "recv_counts", "recv_displs"):
            rows = None if tables is None else tables.get(name)
            if rows is None:
                out.append(None)
                continue
            if self.nlocal == 1 and rows and not isinstance(rows[0], (list, tuple)):
                rows = [rows]
            flat = [int(v) for row in rows for v in row]
            if len(flat) != self.nlocal * self.size:
                raise AlError(f"{name}: expected {self.nlocal} row(s) of {self.size} entries")
            out.append(size_array(flat))
        return out

    def _coll(self, kind, send, recv, count, op="sum", root=0, inplace=False, nonblocking=False, tables=None,
              wire_dtype=None, scale=1.0, algo="auto", ctas=0, stream=None):
        sends, recvs = self._as_list(send), self._as_list(recv)
        first_in = next((t for t in (sends if not inplace else recvs) if t is not None), None)
        first_out = next((t for t in recvs if t is not None), None)
        ref = first_in if first_in is not None else first_out
        dt_in = _code(ref) if ref is not None else DTYPES["uint8"]
        dt_out = _code(first_out) if first_out is not None else -1
        dt_wire = _dtype_code(wire_dtype) if wire_dtype is not None else -1
        if dt_out == dt_in:
            dt_out = -1
        sc, sd, rc, rd = self._tables(tables)
        req = C.c_void_p(None)
        check(self._lib.al_dev_collective(
            self._h, KINDS[kind], self.nlocal, self._ptrs(sends), self._ptrs(recvs), int(count), dt_in, dt_wire, dt_out,
            OPS[op], int(root), 1 if inplace else 0, 1 if tables else 0, sc, sd, rc, rd, float(scale),
            ALGOS[algo] if kind == "allreduce" else PATHS[algo],
            int(ctas), self._stream(stream), C.byref(req) if nonblocking else None))
        return Request(req, True, (sends, recvs)) if nonblocking else None

    def _numel(self, x) -> int:
        t = x[0] if isinstance(x, (list, tuple)) else x
        return t.numel()

    # ---- collectives (recv=None selects the in-place form on `send`) ------------------------
    def allreduce(self, send, recv=None, op="sum", **kw):
        """Element-wise reduction over all ranks.  Keyword options: ``scale`` (factor fused into the
        result), ``wire_dtype`` (e.g. torch.bfloat16 to halve NVLink traffic of an fp32 reduction),
        ``algo`` in {auto, one_shot, two_shot, nvls}, ``ctas``, ``nonblocking``, ``stream``."""
        if recv is None:
            return self._coll("allreduce", None, send, self._numel(send), op, inplace=True, **kw)
        return self._coll("allreduce", send, recv, self._numel(send), op, **kw)

    def reduce(self, send, recv=None, op="sum", root=0, **kw):
        if recv is None:
            return self._coll("reduce", None, send, self._numel(send), op, root, inplace=True, **kw)
        return self._coll("reduce", send, recv, self._numel(send), op, root, **kw)

    def reduce_scatter(self, send, recv=None, op="sum", **kw):
        n = self._numel(send) // self.size
        if recv is None:
            return self._coll("reduce_scatter", None, send, n, op, inplace=True, **kw)
        return self._coll("reduce_scatter", send, recv, n, op, **kw)

    def allgather(self, send, recv=None, **kw):
        if recv is None:
            return self._coll("allgather", None, send, self._numel(send) // self.size, inplace=True, **kw)
        return self._coll("allgather", send, recv, self._numel(send), **kw)

    def alltoall(self, send, recv=None, **kw):
        n = self._numel(send) // self.size
        if recv is None:
            return self._coll("alltoall", None, send, n, inplace=True, **kw)
        return self._coll("alltoall", send, recv, n, **kw)

    def bcast(self, buf, root=0, **kw):
        return self._coll("bcast", None, buf, self._numel(buf), root=root, inplace=True, **kw)

    def gather(self, send, recv, root=0, **kw):
        return self._coll("gather", send, recv, self._numel(send), root=root, **kw)

    def scatter(self, send, recv, root=0, **kw):
        return self._coll("scatter", send, recv, self._numel(recv), root=root, **kw)

    def barrier(self, **kw):
        return self._coll("barrier", None, None, 0, **kw)

    def time_collective(self, kind: str, send, recv, count: int, warmup: int = 20, iters: int = 100, op: str = "sum",
                        stream=None):
        """Benchmark helper: device times (ms) of ``iters`` out-of-place calls of one collective, each preceded
        by a host barrier of the ranks and bracketed by a CUDA event pair (native loop, no Python in between).
        ``count`` is the element count the operation takes (per-rank slice for reduce_scatter / allgather /
        alltoall)."""
        out = (C.c_float * iters)()
        check(self._lib.al_dev_time_collective(self._h, KINDS[kind], C.c_void_p(send.data_ptr()),
                                               C.c_void_p(recv.data_ptr()), int(count), _code(recv), OPS[op],
                                               int(warmup), int(iters), self._stream(stream), out))
        return [float(v) for v in out]

    def exchange_rows(self, send, recv, row_bytes: int, send_row_stride: int, recv_row_stride: int, send_rows,
                      send_first, send_peer_off, recv_rows, recv_first, recv_peer_off, send_idx=None, recv_idx=None,
                      nonblocking=False, stream=None):
        """Alltoall(v) of strided or index-selected rows with the pack / unpack fused into the kernel.

        Row ``k`` of what this rank sends to peer ``d`` is read at byte ``send_peer_off[d] + id * send_row_stride`` of
        ``send`` with ``id = send_first[d] + k`` (or ``send_idx[send_first[d] + k]`` when an int64 index tensor is
        given); row ``k`` received from rank ``r`` is written at ``recv_peer_off[r] + id * recv_row_stride`` of
        ``recv`` likewise.  Tables have one entry per rank (one row of entries per local rank in emulation)."""
        sends, recvs = self._as_list(send), self._as_list(recv)
        sidx = self._as_list(send_idx) if send_idx is not None else None
        ridx = self._as_list(recv_idx) if recv_idx is not None else None

        def table(t):
            rows = [t] if (self.nlocal == 1 and t and not isinstance(t[0], (list, tuple))) else t
            flat = [int(v) for row in rows for v in row]
            if len(flat) != self.nlocal * self.size:
                raise AlError(f"exchange_rows: tables need {self.nlocal} row(s) of {self.size} entries")
            return size_array(flat)

        def idx_ptrs(lst):
            if lst is None:
                return None
            arr = (C.c_void_p * self.nlocal)()
            for i, t in enumerate(lst):
                if t is not None and (str(t.dtype) != "torch.int64" or not t.is_cuda or not t.is_contiguous()):
                    raise AlError("exchange_rows: index tensors must be contiguous CUDA int64 tensors")
                arr[i] = t.data_ptr() if t is not None else None
            return arr

        sp = (C.c_void_p * self.nlocal)(*[t.data_ptr() for t in sends])
        rp = (C.c_void_p * self.nlocal)(*[t.data_ptr() for t in recvs])
        req = C.c_void_p(None)
        check(self._lib.al_dev_exchange_rows(
            self._h, self.nlocal, sp, rp, idx_ptrs(sidx), idx_ptrs(ridx), int(row_bytes), int(send_row_stride),
            int(recv_row_stride), table(send_rows), table(send_first), table(send_peer_off), table(recv_rows),
            table(recv_first), table(recv_peer_off), self._stream(stream), C.byref(req) if nonblocking else None))
        return Request(req, True, (sends, recvs, sidx, ridx)) if nonblocking else None

    def latency_breakdown(self, kind: str, send, recv, count: int, algo: str = "auto", warmup: int = 20,
                          iters: int = 100, op: str = "sum", stream=None) -> dict:
        """Median microseconds of one small collective, split into host enqueue, launch overhead and the kernel's
        phases (entry -> data sent -> first data seen -> exit), from %globaltimer stamps inside the kernel."""
        out = (C.c_double * 6)()
        code = ALGOS[algo] if kind == "allreduce" else PATHS[algo]
        check(self._lib.al_dev_latency_breakdown(self._h, KINDS[kind], C.c_void_p(send.data_ptr()),
                                                 C.c_void_p(recv.data_ptr()), int(count), _code(recv), OPS[op], code,
                                                 int(warmup), int(iters), self._stream(stream), out))
        names = ["event_us", "host_enqueue_us", "kernel_send_us", "kernel_wait_us", "kernel_finish_us", "kernel_us"]
        d = dict(zip(names, [float(v) for v in out]))
        d["launch_overhead_us"] = d["event_us"] - d["kernel_us"]
        return d

    # vector forms: counts / displacements in elements, one row per local rank in emulation
    def reduce_scatterv(self, send, recv, counts, op="sum", **kw):
        return self._coll("reduce_scatter", send, recv, 0, op, tables={"recv_counts": counts}, **kw)

    def allgatherv(self, send, recv, counts, displs, **kw):
        return self._coll("allgather", send, recv, 0, tables={"recv_counts": counts, "recv_displs": displs}, **kw)

    def alltoallv(self, send, send_counts, send_displs, recv, recv_counts, recv_displs, **kw):
        return self._coll("alltoall", send, recv, 0, tables={"send_counts": send_counts, "send_displs": send_displs,
                                                              "recv_counts": recv_counts, "recv_displs": recv_displs}, **kw)

    def gatherv(self, send, recv, counts, displs, root=0, **kw):
        return self._coll("gather", send, recv, 0, root=root, tables={"recv_counts": counts, "recv_displs": displs}, **kw)

    def scatterv(self, send, recv, counts, displs, root=0, **kw):
        return self._coll("scatter", send, recv, 0, root=root, tables={"send_counts": counts, "send_displs": displs}, **kw)

    # ---- point-to-point -----------------------------------------------------------------------
    def p2p(self, items, nonblocking=False, stream=None):
        """items: (is_send, peer, tensor[, owner]) tuples progressing together as one operation."""
        n = len(items)
        is_send = (C.c_int * n)(*[1 if it[0] else 0 for it in items])
        peer = (C.c_int * n)(*[int(it[1]) for it in items])
        owner = (C.c_int * n)(*[int(it[3]) if len(it) > 3 else self.rank for it in items])
        bufs = (C.c_void_p * n)(*[it[2].data_ptr() for it in items])
        nbytes = (C.c_size_t * n)(*[it[2].numel() * it[2].element_size() for it in items])
        req = C.c_void_p(None)
        check(self._lib.al_dev_p2p(self._h, n, is_send, peer, owner, bufs, nbytes, self._stream(stream),
                                   C.byref(req) if nonblocking else None))
        return Request(req, True, [it[2] for it in items]) if nonblocking else None

    def send(self, buf, dest, **kw):
        return self.p2p([(True, dest, buf)], **kw)

    def recv(self, buf, src, **kw):
        return self.p2p([(False, src, buf)], **kw)

    def sendrecv(self, send, dest, recv, src, **kw):
        return self.p2p([(True, dest, send), (False, src, recv)], **kw)

    # ---- registered buffers -----------------------------------------------------------------------
    def register(self, tensor) -> int:
        """Collective (every rank, same order, each with its own tensor): make the tensor's memory addressable by
        all ranks, so that reduce_scatter (as input) and allgather / alltoall / bcast (as output) on it skip the
        staging area.  In emulation pass the list of all ranks' tensors.  Returns the window index, or -1 when the
        memory cannot be shared (the tensor then simply keeps using the staged path).  Tensors from
        :meth:`symm_empty` are registered already."""
        if self.emulated:
            ts = list(tensor)
            arr = (C.c_void_p * len(ts))(*[t.data_ptr() for t in ts])
            w = self._lib.al_dev_register_emulated(self._h, arr, len(ts), ts[0].numel() * ts[0].element_size())
        else:
            w = self._lib.al_dev_register(self._h, C.c_void_p(tensor.data_ptr()), tensor.numel() * tensor.element_size())
        if w == -2:
            check(1)
        return int(w)

    def unregister(self, tensor) -> None:
        """Collective: forget a registered tensor (before its memory is freed)."""
        t = tensor[0] if isinstance(tensor, (list, tuple)) else tensor
        check(self._lib.al_dev_unregister(self._h, C.c_void_p(t.data_ptr())))

    # ---- symmetric memory ------------------------------------------------------------------------
    def symm_empty(self, shape, dtype):
        """Collective: a tensor in symmetric (peer-mapped, multicast-bound when possible) memory.
        In emulation returns a list with every rank's tensor."""
        torch = self._torch
        numel = 1
        for s in (shape if isinstance(shape, (tuple, list)) else (shape,)):
            numel *= int(s)
        nbytes = max(16, numel * torch.empty((), dtype=dtype).element_size())
        base = check_ptr(self._lib.al_dev_symm_alloc(self._h, nbytes))

        def view(ptr):
            blob = _CudaBlob(ptr, nbytes, self)
            t = torch.as_tensor(blob, device="cuda").view(torch.uint8)[: numel * torch.empty((), dtype=dtype).element_size()]
            return t.view(dtype).view(shape)

        if self.nlocal == 1:
            t = view(base)
            self._symm[t.data_ptr()] = base
            return t
        out = []
        for r in range(self.size):
            p = check_ptr(self._lib.al_dev_symm_peer_ptr(self._h, C.c_void_p(base), r))
            out.append(view(p))
        self._symm[out[0].data_ptr()] = base
        return out

    def check_guards(self) -> None:
        """Guard mode (``set_tuning("debug_guard", 1)`` before allocating): raises if anything wrote outside a
        :meth:`symm_empty` tensor of this rank (4 KiB of a known pattern sit before and after each)."""
        check(self._lib.al_dev_check_guards(self._h))

    def symm_free(self, tensor) -> None:
        t = tensor[0] if isinstance(tensor, (list, tuple)) else tensor
        base = self._symm.pop(t.data_ptr(), None)
        if base is None:
            raise AlError("tensor was not created by symm_empty of this communicator")
        check(self._lib.al_dev_symm_free(self._h, C.c_void_p(base)))

    def peer_ptr(self, tensor, peer: int) -> int:
        """Address, in this process, of rank ``peer``'s copy of a symmetric tensor (usable by kernels of this
        library; it is not wrapped in a tensor because the memory physically lives on another GPU)."""
        return int(check_ptr(self._lib.al_dev_symm_peer_ptr(self._h, C.c_void_p(tensor.data_ptr()), int(peer))))

    def peer_tensor(self, tensor, peer: int):
        """The view, in this process, of rank ``peer``'s copy of a symmetric tensor."""
        torch = self._torch
        p = check_ptr(self._lib.al_dev_symm_peer_ptr(self._h, C.c_void_p(tensor.data_ptr()), int(peer)))
        nbytes = tensor.numel() * tensor.element_size()
        blob = _CudaBlob(p, nbytes, self)
        return torch.as_tensor(blob, device="cuda").view(torch.uint8).view(tensor.dtype).view(tensor.shape)

    # ---- RMA -----------------------------------------------------------------------------------------
    def attach(self, tensor, peer: int) -> int:
        """Pairwise collective; returns the address of the peer's buffer as mapped here (0 if none)."""
        return self._lib.al_rma_attach(self._h, C.c_void_p(tensor.data_ptr() if tensor is not None else 0), int(peer)) or 0

    def detach(self, remote_addr: int, peer: int) -> None:
        check(self._lib.al_rma_detach(self._h, C.c_void_p(remote_addr), int(peer)))

    def put(self, src, dest: int, remote_addr: int) -> None:
        check(self._lib.al_rma_put(self._h, C.c_void_p(src.data_ptr()), int(dest), C.c_void_p(remote_addr),
                                   src.numel() * src.element_size()))

    def get(self, dst, src_rank: int, remote_addr: int) -> None:
        """Fill ``dst`` from the buffer at ``remote_addr`` (an :meth:`attach` result for ``src_rank``), stream-ordered."""
        check(self._lib.al_rma_get(self._h, C.c_void_p(dst.data_ptr()), int(src_rank), C.c_void_p(remote_addr),
                                   dst.numel() * dst.element_size()))

    def notify(self, peer: int) -> None:
        check(self._lib.al_rma_notify(self._h, int(peer)))

    def wait(self, peer: int) -> None:
        check(self._lib.al_rma_wait(self._h, int(peer)))

    def sync(self, peer: int) -> None:
        check(self._lib.al_rma_sync(self._h, int(peer)))

    def halo_exchange(self, tensors, depth: int = 1, periodic: bool = False, ctas: int = 0, stream=None) -> None:
        """Fused halo exchange of fp32 tensors shaped (N, C, D_local + 2*depth, H, W) split along D.

        ``tensors[r]`` must be rank r's tensor as addressable from this process: the own tensor plus
        :meth:`peer_ptr` addresses of the neighbours (all ranks' tensors in emulation)."""
        ref = next(t for t in tensors if t is not None and not isinstance(t, int))
        n, c, dtot, h, w = ref.shape
        arr = (C.c_void_p * self.size)(*[(None if t is None else (t if isinstance(t, int) else t.data_ptr()))
                                         for t in tensors])
        check(self._lib.al_halo_exchange(self._h, arr, n * c, dtot - 2 * depth, h * w, depth, 1 if periodic else 0,
                                         int(ctas), self._stream(stream)))
