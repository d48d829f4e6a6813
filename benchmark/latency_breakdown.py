"""Where the time of a small collective goes, per path (run under alrun / torchrun, one GPU per rank):

    alrun -n 8 python benchmark/latency_breakdown.py [--bytes 1024 65536] [--iters 100]

For allreduce / reduce_scatter / allgather / alltoall of the given sizes it prints, for the low-latency
packet path and for the staged path, the medians of: the event-pair time (what the collective sweep reports),
the host time inside the enqueueing call, and the kernel's phases from %globaltimer stamps written inside the
kernel (entry -> data sent -> first data seen -> exit).  Event time minus kernel time is launch and front-end
overhead.  Max over ranks of every column.
"""
import argparse
import os
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
import aluminum_b200 as al  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--bytes", type=int, nargs="+", default=[1024, 8192, 65536])
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=20)
    a = ap.parse_args()
    local = int(os.environ.get("AL_LOCAL_RANK", os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(local)
    al.init()
    comm = al.DeviceComm()
    p, me = comm.size, comm.rank
    send = torch.rand(max(a.bytes) // 4 + 16, device="cuda")
    recv = torch.empty_like(send)
    cols = ["event_us", "host_enqueue_us", "launch_overhead_us", "kernel_us", "kernel_send_us", "kernel_wait_us",
            "kernel_finish_us"]
    if me == 0:
        print(f"ranks={p}  (medians of {a.iters} calls, max over ranks, microseconds)")
        print(f"{'op':<15}{'bytes':>9}{'path':>8}" + "".join(f"{c[:-3]:>17}" for c in cols))
    for kind in ("allreduce", "reduce_scatter", "allgather", "alltoall"):
        for total in a.bytes:
            n = total // 4
            per = max(1, n // p)
            count = n if kind == "allreduce" else per
            for path in ("ll", "staged" if kind != "allreduce" else "one_shot"):
                pair_bytes = count * 4
                if path == "ll" and pair_bytes > 65536:
                    continue
                d = comm.latency_breakdown(kind, send, recv, count, algo=path, warmup=a.warmup, iters=a.iters)
                t = torch.tensor([d[c] for c in cols], device="cuda", dtype=torch.float32)
                comm.allreduce(t, op="max")
                if me == 0:
                    print(f"{kind:<15}{total:>9}{path:>8}" + "".join(f"{float(v):>17.2f}" for v in t.tolist()))
    comm.close()
    al.finalize()


if __name__ == "__main__":
    main()
