"""Small single-GPU cases of the library's kernels, sized for profiler captures
(inputs larger than the 126 MB L2, a few GB on the device at most, a handful of launches).

    python benchmark/profile_kernels.py --case sgd|cast|allreduce|alltoall|halo|ll|window_ag|window_rs|rows|p2p|rs_pipelined [--iters 3]

The multi-rank cases run all ranks of an emulated communicator in one launch on one GPU: "remote" traffic
lands in local HBM, so the figures show the kernels' memory behaviour, not NVLink.

Prints the CUDA-event time of the case and the achieved fraction of the measured copy bandwidth.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import aluminum_b200 as al  # noqa: E402
from aluminum_b200.ops import HaloExchange, scale_cast, sgd_momentum_step  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="sgd")
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
    al.init()
    peaks = {"hbm_gbs": 6549.1}
    try:
        peaks = json.load(open(os.path.join(os.path.dirname(__file__), "..", "MEASURED_PEAKS.json")))
    except Exception:
        pass
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    comm = None
    if a.case != "p2p":   # keep the emulated communicators' workspaces small: these cases do not use the mailboxes
        al.set_tuning("dev_mailbox_bytes", 1 << 20)
        al.set_tuning("p2p_ll_max_bytes", 65536)
    if a.case == "sgd":
        n = 64 << 20
        p, m, g = (torch.randn(n, device="cuda") for _ in range(3))
        fn = lambda: sgd_momentum_step(p, m, g, 0.1, 0.9, 1e-4, 1.0, False, True)
        nbytes = n * 4 * 5  # read p, m, g; write p, m (+ zeroed g)
        nbytes += n * 4
    elif a.case == "cast":
        n = 128 << 20
        x = torch.randn(n, device="cuda")
        y = torch.empty(n, device="cuda", dtype=torch.bfloat16)
        fn = lambda: scale_cast(x, y, 0.125)
        nbytes = n * 6
    elif a.case in ("allreduce", "alltoall"):
        pr = 8
        comm = al.DeviceComm(emulate=pr)
        n = 8 << 20  # 32 MiB per rank
        xs = [torch.randn(n, device="cuda") for _ in range(pr)]
        outs = [torch.empty(n, device="cuda") for _ in range(pr)]
        if a.case == "allreduce":
            fn = lambda: comm.allreduce(xs, outs, algo="two_shot")
            nbytes = pr * n * 4 * 6  # per rank: read in, write slots, read slots, write result area x p, read, write out
        else:
            fn = lambda: comm.alltoall(xs, outs)
            nbytes = pr * n * 4 * 4
    elif a.case == "ll":
        pr = 8
        comm = al.DeviceComm(emulate=pr)
        n = 16 << 10  # 64 KiB per rank: the packet path's upper range
        xs = [torch.randn(n, device="cuda") for _ in range(pr)]
        outs = [torch.empty(n, device="cuda") for _ in range(pr)]
        fn = lambda: comm.allreduce(xs, outs, algo="ll")
        nbytes = pr * n * 4 * (1 + 2 * (pr - 1) * 2 + 1)  # read in; packets written and read at 2x payload; write out
    elif a.case in ("window_ag", "window_rs"):
        pr = 8
        comm = al.DeviceComm(emulate=pr)
        n = 4 << 20  # 16 MiB per rank slice, 128 MiB per rank buffer
        full = [torch.randn(n * pr, device="cuda") for _ in range(pr)]
        assert comm.register(full) >= 0
        part = [torch.randn(n, device="cuda") for _ in range(pr)]
        if a.case == "window_ag":
            fn = lambda: comm.allgather(part, full, algo="window")
            nbytes = pr * n * 4 * (1 + pr)          # read own slice, write it into p buffers
        else:
            fn = lambda: comm.reduce_scatter(full, part, algo="window")
            nbytes = pr * n * 4 * (pr + 1)          # read p slices, write one
    elif a.case == "rows":
        pr = 8
        comm = al.DeviceComm(emulate=pr)
        from aluminum_b200.parallel import ulysses
        s_, h_, d_ = 2048, 32, 128                  # per rank: 2048 x 32 x 128 bf16 = 16 MiB
        shards = [torch.randn(s_, h_, d_, device="cuda", dtype=torch.bfloat16) for _ in range(pr)]
        fn = lambda: ulysses.seq_to_head(comm, shards)
        nbytes = pr * s_ * h_ * d_ * 2 * 4          # read, write slot, read slot, write
    elif a.case == "p2p":
        pr = 2
        comm = al.DeviceComm(emulate=pr)
        n = 32 << 20                                # 128 MiB each way
        src = [torch.randn(n, device="cuda") for _ in range(pr)]
        dst = [torch.empty(n, device="cuda") for _ in range(pr)]
        assert comm.register(dst) >= 0
        items = []
        for r in range(pr):
            items.append((True, (r + 1) % pr, src[r], r))
            items.append((False, (r - 1) % pr, dst[r], r))
        fn = lambda: comm.p2p(items)
        nbytes = pr * n * 4 * 2                     # rendezvous into registered buffers: read once, write once
    elif a.case == "rs_pipelined":
        pr = 8
        al.set_tuning("pipeline_min_bytes", 8 << 20)
        comm = al.DeviceComm(emulate=pr)
        n = 4 << 20                                 # 16 MiB per rank slice, 128 MiB per rank: publisher / consumer CTAs
        full = [torch.randn(n * pr, device="cuda") for _ in range(pr)]
        part = [torch.empty(n, device="cuda") for _ in range(pr)]
        fn = lambda: comm.reduce_scatter(full, part)
        nbytes = pr * n * 4 * (pr + pr + pr + 1)    # read p slices, write p slots, read p slots, write one
    elif a.case == "halo":
        pr = 4
        comm = al.DeviceComm(emulate=pr)
        hx = HaloExchange(comm, 1, 32, 16, 512, 512, depth=1)
        fn = lambda: hx.exchange()
        nbytes = (2 * pr - 2) * 32 * 512 * 512 * 4 * 2
    else:
        raise SystemExit("unknown case")
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(a.iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.iters
    gbs = nbytes / (ms * 1e-3) / 1e9
    print(json.dumps({"case": a.case, "ms": ms, "algorithmic_GBs": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"]}))
    if comm is not None:
        comm.close()
    al.finalize()


if __name__ == "__main__":
    main()
