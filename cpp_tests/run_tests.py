"""Sweep of test_ops over rank counts x backends x operations x datatypes x {blocking, non-blocking} x
{out-of-place, in-place} x roots, with a per-run time limit (role of test/run_tests.py:61-319 of the reference;
ranks are started by the library's own launcher).

    python cpp_tests/run_tests.py --backends host --max-ranks 4
    python cpp_tests/run_tests.py --backends device --max-ranks 8      # one GPU per rank
    python cpp_tests/run_tests.py --backends host --max-ranks 8 --nodes 1 2 4   # also over modelled nodes (TCP)
"""
import argparse
import itertools
import subprocess
import sys
from pathlib import Path

BIN = Path(__file__).resolve().parent.parent / "aluminum_b200" / "bin"
OPS = ["allreduce", "reduce", "reduce_scatter", "reduce_scatterv", "allgather", "allgatherv", "alltoall", "alltoallv",
       "bcast", "gather", "gatherv", "scatter", "scatterv", "barrier", "send", "sendrecv", "multisendrecv"]
ROOTED = {"reduce", "bcast", "gather", "gatherv", "scatter", "scatterv"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backends", nargs="+", default=["host"])
    ap.add_argument("--datatypes", nargs="+", default=["float", "int"])
    ap.add_argument("--max-ranks", type=int, default=4)
    ap.add_argument("--min-ranks", type=int, default=1)
    ap.add_argument("--max-size", type=int, default=1 << 14)
    ap.add_argument("--timeout", type=int, default=60)
    ap.add_argument("--max-fails", type=int, default=5)
    ap.add_argument("--nodes", nargs="+", type=int, default=[1],
                    help="node counts to model on this machine (host / ht backends; 1 = everything on one node)")
    a = ap.parse_args()
    ranks = [n for n in (1, 2, 4, 8) if a.min_ranks <= n <= a.max_ranks]
    fails = total = 0
    for n, nodes, be, op, dt, nb, ip in itertools.product(ranks, a.nodes, a.backends, OPS, a.datatypes, (False, True),
                                                         (False, True)):
        if op in ("barrier", "send", "bcast") and ip:
            continue
        if nodes > 1 and (nodes > n or be == "device"):
            continue  # a device communicator lives inside one node
        for root in ((0, 1) if op in ROOTED and n > 1 else (0,)):
            launch = ["--nodes", str(nodes)] if nodes > 1 else []
            cmd = [str(BIN / "alrun"), "-n", str(n), *launch, "--timeout", str(a.timeout), str(BIN / "test_ops"), "--backend", be,
                   "--op", op, "--datatype", dt, "--max-size", str(a.max_size), "--odd-sizes", "--zero", "--quiet",
                   "--root", str(root), "--hang-timeout", str(max(5, a.timeout // 2))]
            cmd += ["--nonblocking"] if nb else []
            cmd += ["--inplace"] if ip else []
            total += 1
            tail = ""
            try:
                r = subprocess.run(cmd, capture_output=True, text=True, timeout=2 * a.timeout)
                rc, tail = r.returncode, (r.stdout + r.stderr)[-600:]
            except subprocess.TimeoutExpired:
                rc, tail = -1, "timed out"
            if rc != 0:
                fails += 1
                print("FAIL:", " ".join(cmd[1:3] + launch + cmd[5 + len(launch):]), file=sys.stderr)
                print("      " + tail.strip().replace("\n", "\n      "), file=sys.stderr)
                if fails >= a.max_fails:
                    print(f"stopping after {fails} failures", file=sys.stderr)
                    return 1
    print(f"{total - fails} of {total} configurations passed")
    return 1 if fails else 0


if __name__ == "__main__":
    sys.exit(main())
