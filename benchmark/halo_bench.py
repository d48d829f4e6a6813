"""Halo exchange of a spatially partitioned 3-D tensor (fp32, global 1x32x512x512x512 split along D).

    python -m torch.distributed.run --nproc-per-node N benchmark/halo_bench.py [--iters 50]

Every rank exchanges its 1-plane-deep boundary slabs (32 x 512 x 512 fp32 = 32 MiB) with both
neighbours per iteration.  Two paths are timed on the device (max over ranks):
  fused    one kernel per rank: boundary planes are read from the interior and stored straight
           into the neighbours' halo planes over NVLink, flags included
  unfused  the reference's structure: pack kernel -> contiguous Put into the peer (the role of
           cudaMemcpyPeerAsync in include/aluminum/mpi_cuda/rma_ipc.hpp:298-299) -> unpack kernel,
           ordered with Sync (notify / wait)
Reported: microseconds per exchange and GB/s of slab payload leaving an interior rank (2 slabs).
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import aluminum_b200 as al  # noqa: E402
from aluminum_b200.ops import HaloExchange, halo_pack, halo_unpack  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--d", type=int, default=512)
    ap.add_argument("--hw", type=int, default=512)
    ap.add_argument("--c", type=int, default=32)
    a = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    al.init()
    comm = al.DeviceComm()
    p, me = comm.size, comm.rank
    d_local = a.d // p
    hx = HaloExchange(comm, 1, a.c, d_local, a.hw, a.hw, depth=1)
    t = hx.local
    t.uniform_(0, 1)
    slab = a.c * a.hw * a.hw * 4
    nslabs = (1 if me == 0 else 0) + (1 if me == p - 1 else 0)
    nslabs = 2 - nslabs if p > 1 else 0

    def timed(fn):
        for _ in range(a.warmup):
            fn()
        comm.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        x = torch.tensor([e0.elapsed_time(e1) / a.iters * 1e3], device="cuda")
        comm.allreduce(x, op="max")
        return float(x.item())

    fused_us = timed(lambda: hx.exchange())

    # unfused comparison path
    lo, hi = me - 1, me + 1
    pack_lo = torch.empty(a.c * a.hw * a.hw, device="cuda") if lo >= 0 else None
    pack_hi = torch.empty(a.c * a.hw * a.hw, device="cuda") if hi < p else None
    land_lo = comm.symm_empty((a.c * a.hw * a.hw,), torch.float32)  # landing buffers, peer-visible
    land_hi = comm.symm_empty((a.c * a.hw * a.hw,), torch.float32)
    peer_land_hi_of_lo = comm.peer_ptr(land_hi, lo) if lo >= 0 else None  # my low slab lands in lo's "from hi" buffer
    peer_land_lo_of_hi = comm.peer_ptr(land_lo, hi) if hi < p else None

    def unfused():
        for nb in (lo, hi):
            if 0 <= nb < p:
                comm.sync(nb)                       # neighbour is done with its landing buffers
        if lo >= 0:
            halo_pack(t, 1, 1, pack_lo)
            comm.put(pack_lo, lo, peer_land_hi_of_lo)   # contiguous put into the peer
        if hi < p:
            halo_pack(t, d_local, 1, pack_hi)
            comm.put(pack_hi, hi, peer_land_lo_of_hi)
        for nb in (lo, hi):
            if 0 <= nb < p:
                comm.sync(nb)                       # data has landed
        if lo >= 0:
            halo_unpack(t, land_lo, 0, 1)
        if hi < p:
            halo_unpack(t, land_hi, d_local + 1, 1)

    unfused_us = timed(unfused)
    if me == 0:
        out = {"op": "halo_exchange", "ranks": p, "global": [1, a.c, a.d, a.hw, a.hw], "slab_bytes": slab,
               "fused_us": fused_us, "unfused_us": unfused_us,
               "fused_GBs_interior_rank": 2 * slab / (fused_us * 1e-6) / 1e9 if p > 2 else slab / (fused_us * 1e-6) / 1e9,
               "speedup_vs_unfused": unfused_us / fused_us}
        print(json.dumps(out))
    comm.close()
    al.finalize()


if __name__ == "__main__":
    main()
