"""Python face of the communicators.

``HostComm`` works on NumPy arrays / CPU tensors between the CPU ranks of one
host; ``DeviceComm`` works on CUDA tensors and launches the library's sm_100a
kernels on the current PyTorch stream.  Semantics (stream-ordered "blocking"
calls, ``nonblocking=True`` returning a :class:`Request` whose ``wait()`` joins
on the device and whose ``test()`` polls on the host, in-place forms when
``recv`` is omitted) follow the C++ API in ``include/Al.hpp`` - which itself
mirrors the reference's ``include/Al.hpp:118-1911``.

An *emulated* ``DeviceComm`` holds all ``p`` ranks in one process on one GPU;
every argument then is a list with one tensor per rank and each call is one
cooperative kernel launch.  It exists so that the device protocol can be
tested on a single GPU.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import _lib
from ._lib import ALGOS, DTYPES, KINDS, OPS, AlError, check, check_ptr, size_array

_initialized_here = False


def init() -> None:
    """Initialise the native library (idempotent): rank discovery, control plane, CUDA pools."""
    global _initialized_here
    lib = _lib.load()
    if not lib.al_initialized():
        check(lib.al_init())
        _initialized_here = True


def finalize() -> None:
    lib = _lib.load()
    if lib.al_initialized():
        check(lib.al_finalize())


def world_rank() -> int:
    return _lib.load().al_world_rank()


def world_size() -> int:
    return _lib.load().al_world_size()


def local_rank() -> int:
    """Rank among the processes of this node."""
    return _lib.load().al_world_local_rank()


def local_size() -> int:
    return _lib.load().al_world_local_size()


def num_nodes() -> int:
    """Number of nodes the world spans (1 unless the TCP transport connected several hosts)."""
    return _lib.load().al_world_num_nodes()


def node_index() -> int:
    """Index of this rank's node; `comm.split(node_index(), rank)` gives the node-local communicator."""
    return _lib.load().al_world_node_index()


def peer_alive(world_rank: int) -> bool:
    """False once the process of that world rank has exited (or finalised the library)."""
    v = _lib.load().al_world_peer_alive(int(world_rank))
    if v < 0:
        raise AlError(f"no such world rank: {world_rank}")
    return bool(v)


def alive_ranks() -> list:
    """World ranks whose processes are still there, this one included: after a failure the survivors
    build a new communicator from this list (``HostComm.from_ranks``) and carry on."""
    return [r for r in range(world_size()) if peer_alive(r)]


def info() -> str:
    buf = C.create_string_buffer(16384)
    check(_lib.load().al_info(buf, len(buf)))
    return buf.value.decode()


def set_tuning(name: str, value: float) -> None:
    check(_lib.load().al_set_tuning(name.encode(), float(value)))


def get_tuning(name: str) -> float:
    return _lib.load().al_get_tuning(name.encode())


# ---------------------------------------------------------------------------------------
def _np_code(a: np.ndarray) -> int:
    name = {"bool": "uint8"}.get(a.dtype.name, a.dtype.name)
    if name not in DTYPES:
        raise AlError(f"unsupported dtype {a.dtype}")
    return DTYPES[name]


def _torch_code(t) -> int:
    name = str(t.dtype).replace("torch.", "")
    if name not in DTYPES:
        raise AlError(f"unsupported dtype {t.dtype}")
    return DTYPES[name]


def _host_view(x):
    """(address, element count, dtype code, keep-alive) of a NumPy array or CPU tensor."""
    if x is None:
        return None, 0, DTYPES["uint8"], None
    if isinstance(x, np.ndarray):
        if not x.flags["C_CONTIGUOUS"]:
            raise AlError("host buffers must be contiguous")
        return x.ctypes.data, x.size, _np_code(x), x
    import torch
    if isinstance(x, torch.Tensor):
        if x.is_cuda or not x.is_contiguous():
            raise AlError("host buffers must be contiguous CPU tensors")
        return x.data_ptr(), x.numel(), _torch_code(x), x
    raise AlError(f"unsupported buffer type {type(x)}")


class Request:
    """Handle of a non-blocking operation."""

    def __init__(self, handle: C.c_void_p, device: bool, keep=None):
        self._h = handle
        self._device = device
        self._keep = keep

    def test(self) -> bool:
        """Host-side poll; True once complete (the handle is released then)."""
        if not self._h:
            return True
        done = C.c_int(0)
        lib = _lib.load()
        check((lib.al_dev_test if self._device else lib.al_host_test)(C.byref(self._h), C.byref(done)))
        if done.value:
            self._keep = None
        return bool(done.value)

    def wait(self) -> None:
        """Host backend: block.  Device backend: make the communicator's stream wait (host returns at once)."""
        if not self._h:
            return
        lib = _lib.load()
        check((lib.al_dev_wait if self._device else lib.al_host_wait)(C.byref(self._h)))
        self._keep = None


# ---------------------------------------------------------------------------------------
class HostComm:
    """CPU communicator: shared memory inside a node, sockets between nodes."""

    def __init__(self, _handle=None):
        init()
        lib = _lib.load()
        self._lib = lib
        self._h = C.c_void_p(_handle if _handle else check_ptr(lib.al_host_comm_create()))
        self.rank = lib.al_host_comm_rank(self._h)
        self.size = lib.al_host_comm_size(self._h)
        self.local_rank = lib.al_host_comm_local_rank(self._h)   # among the members on this rank's node
        self.local_size = lib.al_host_comm_local_size(self._h)

    @classmethod
    def from_ranks(cls, world_ranks: Sequence[int]) -> "HostComm":
        """Communicator over the listed world ranks, in that order.  Collective over those ranks only:
        every one of them passes the same list, nobody else takes part."""
        init()
        arr = (C.c_int * len(world_ranks))(*[int(r) for r in world_ranks])
        return cls(check_ptr(_lib.load().al_host_comm_create_group(arr, len(world_ranks))))

    def local(self) -> "HostComm":
        """Collective: the communicator of the members that run on this rank's node."""
        return HostComm(check_ptr(self._lib.al_host_comm_local(self._h)))

    def split(self, color: int, key: int) -> "HostComm":
        return HostComm(check_ptr(self._lib.al_host_comm_split(self._h, color, key)))

    def stats(self) -> dict:
        """Counters of this rank: collectives, p2p_ops, bytes contributed or sent, failures."""
        out = (C.c_uint64 * 4)()
        check(self._lib.al_host_comm_stats(self._h, out))
        return dict(zip(["collectives", "p2p_ops", "bytes", "failures"], [int(v) for v in out]))

    def abort(self, why: str = "aborted by the caller") -> None:
        """Fail the communicator on this rank: operations in flight end with an error, later calls raise."""
        check(self._lib.al_host_comm_abort(self._h, why.encode()))

    def close(self) -> None:
        if self._h:
            self._lib.al_host_comm_destroy(self._h)
            self._h = C.c_void_p(None)

    def __del__(self):
        try:
            if self._lib.al_initialized():
                self.close()
        except Exception:
            pass

    def _coll(self, kind, send, recv, count, op="sum", root=0, inplace=False, nonblocking=False, tables=None):
        sp, _, sc, k1 = _host_view(send)
        rp, _, rc, k2 = _host_view(recv)
        code = rc if recv is not None else sc
        t = tables or {}
        arrs = [size_array(t.get(n)) for n in ("send_counts", "send_displs", "recv_counts", "recv_displs")]
        req = C.c_void_p(None)
        check(self._lib.al_host_collective(self._h, KINDS[kind], sp, rp, int(count), code, OPS[op], root,
                                           1 if inplace else 0, 1 if tables else 0, *arrs,
                                           C.byref(req) if nonblocking else None))
        return Request(req, False, (k1, k2)) if nonblocking else None

    # uniform collectives; `recv=None` selects the in-place form on `send`
    def allreduce(self, send, recv=None, op="sum", nonblocking=False):
        if recv is None:
            return self._coll("allreduce", None, send, _host_view(send)[1], op, inplace=True, nonblocking=nonblocking)
        return self._coll("allreduce", send, recv, _host_view(send)[1], op, nonblocking=nonblocking)

    def reduce(self, send, recv=None, op="sum", root=0, nonblocking=False):
        if recv is None:
            return self._coll("reduce", None, send, _host_view(send)[1], op, root, True, nonblocking)
        return self._coll("reduce", send, recv, _host_view(send)[1], op, root, False, nonblocking)

    def reduce_scatter(self, send, recv=None, op="sum", nonblocking=False):
        n = _host_view(send)[1] // self.size
        if recv is None:
            return self._coll("reduce_scatter", None, send, n, op, inplace=True, nonblocking=nonblocking)
        return self._coll("reduce_scatter", send, recv, n, op, nonblocking=nonblocking)

    def allgather(self, send, recv=None, nonblocking=False):
        if recv is None:
            return self._coll("allgather", None, send, _host_view(send)[1] // self.size, inplace=True, nonblocking=nonblocking)
        return self._coll("allgather", send, recv, _host_view(send)[1], nonblocking=nonblocking)

    def alltoall(self, send, recv=None, nonblocking=False):
        n = _host_view(send)[1] // self.size
        if recv is None:
            return self._coll("alltoall", None, send, n, inplace=True, nonblocking=nonblocking)
        return self._coll("alltoall", send, recv, n, nonblocking=nonblocking)

    def bcast(self, buf, root=0, nonblocking=False):
        return self._coll("bcast", None, buf, _host_view(buf)[1], root=root, inplace=True, nonblocking=nonblocking)

    def gather(self, send, recv, root=0, nonblocking=False):
        return self._coll("gather", send, recv if self.rank == root else None, _host_view(send)[1], root=root, nonblocking=nonblocking)

    def scatter(self, send, recv, root=0, nonblocking=False):
        return self._coll("scatter", send if self.rank == root else None, recv, _host_view(recv)[1], root=root, nonblocking=nonblocking)

    def barrier(self, nonblocking=False):
        return self._coll("barrier", None, None, 0, nonblocking=nonblocking)

    # vector collectives
    def reduce_scatterv(self, send, recv, counts, op="sum", nonblocking=False):
        return self._coll("reduce_scatter", send, recv, 0, op, nonblocking=nonblocking, tables={"recv_counts": counts})

    def allgatherv(self, send, recv, counts, displs, nonblocking=False):
        return self._coll("allgather", send, recv, 0, nonblocking=nonblocking, tables={"recv_counts": counts, "recv_displs": displs})

    def alltoallv(self, send, send_counts, send_displs, recv, recv_counts, recv_displs, nonblocking=False):
        return self._coll("alltoall", send, recv, 0, nonblocking=nonblocking,
                          tables={"send_counts": send_counts, "send_displs": send_displs,
                                  "recv_counts": recv_counts, "recv_displs": recv_displs})

    def gatherv(self, send, recv, counts, displs, root=0, nonblocking=False):
        return self._coll("gather", send, recv if self.rank == root else None, 0, root=root, nonblocking=nonblocking,
                          tables={"recv_counts": counts, "recv_displs": displs})

    def scatterv(self, send, recv, counts, displs, root=0, nonblocking=False):
        return self._coll("scatter", send if self.rank == root else None, recv, 0, root=root, nonblocking=nonblocking,
                          tables={"send_counts": counts, "send_displs": displs})

    # point-to-point
    def _p2p(self, items, nonblocking=False):
        n = len(items)
        is_send = (C.c_int * n)(*[1 if it[0] else 0 for it in items])
        peer = (C.c_int * n)(*[it[1] for it in items])
        views = [_host_view(it[2]) for it in items]
        bufs = (C.c_void_p * n)(*[v[0] for v in views])
        nbytes = (C.c_size_t * n)(*[v[1] * _lib.DTYPE_SIZES[v[2]] for v in views])
        req = C.c_void_p(None)
        check(self._lib.al_host_p2p(self._h, n, is_send, peer, bufs, nbytes, C.byref(req) if nonblocking else None))
        return Request(req, False, [v[3] for v in views]) if nonblocking else None

    def send(self, buf, dest, nonblocking=False):
        return self._p2p([(True, dest, buf)], nonblocking)

    def recv(self, buf, src, nonblocking=False):
        return self._p2p([(False, src, buf)], nonblocking)

    def sendrecv(self, send, dest, recv, src, nonblocking=False):
        return self._p2p([(True, dest, send), (False, src, recv)], nonblocking)

    def multisendrecv(self, sends: Sequence, dests: Sequence[int], recvs: Sequence, srcs: Sequence[int], nonblocking=False):
        items = [(True, d, b) for b, d in zip(sends, dests)] + [(False, s, b) for b, s in zip(recvs, srcs)]
        return self._p2p(items, nonblocking)
