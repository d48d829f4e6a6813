"""aluminum_b200 - a Blackwell-native communication library with the capabilities of LLNL's Aluminum.

Layers (bottom up): a C++17 host runtime and hand-written sm_100a CUDA kernels
in ``libal_b200.so`` (sources under ``src/``, ``kernels/``, ``include/``), the
ctypes binding in :mod:`aluminum_b200._lib`, communicators in
:mod:`aluminum_b200.comm` / :mod:`aluminum_b200.device`, element-wise and halo
ops in :mod:`aluminum_b200.ops`, parallelism helpers (data / tensor / sequence /
expert / context / pipeline) in :mod:`aluminum_b200.parallel` and the models
used by the end-to-end benchmark in :mod:`aluminum_b200.models`.
"""
from ._lib import AlError, lib_path
from .comm import (HostComm, Request, alive_ranks, finalize, get_tuning, info, init, local_rank, local_size,
                   node_index, num_nodes, peer_alive, set_tuning, world_rank, world_size)


def __getattr__(name):
    if name == "DeviceComm":
        from .device import DeviceComm
        return DeviceComm
    raise AttributeError(name)


__version__ = "0.1.0"
__all__ = ["AlError", "HostComm", "DeviceComm", "Request", "init", "finalize", "info", "world_rank", "world_size", "local_rank", "local_size", "num_nodes", "node_index",
           "set_tuning", "get_tuning", "lib_path", "peer_alive", "alive_ranks"]
