"""Small single-GPU cases of the library's kernels, sized for profiler captures
(inputs larger than the 126 MB L2, a few GB on the device at most, a handful of launches).

    python benchmark/profile_kernels.py --case sgd|cast|allreduce|alltoall|halo [--iters 3]

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
