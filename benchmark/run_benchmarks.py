"""Sweep launcher: runs benchmark_ops for every requested backend x operation x datatype x rank count
and writes one result file per configuration (role of benchmark/run_benchmarks.py:158-253 of the
reference, with the library's own launcher instead of jsrun / srun).

    python benchmark/run_benchmarks.py --out results --ranks 2 4 8 --backends device nccl \
        --ops allreduce reduce_scatter allgather alltoall --datatypes float bfloat16
"""
import argparse
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "aluminum_b200" / "bin"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="benchmark_results")
    ap.add_argument("--ranks", type=int, nargs="+", default=[2])
    ap.add_argument("--backends", nargs="+", default=["device", "nccl"])
    ap.add_argument("--ops", nargs="+", default=["allreduce", "reduce_scatter", "allgather", "alltoall"])
    ap.add_argument("--datatypes", nargs="+", default=["float"])
    ap.add_argument("--min-bytes", type=int, default=8)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--num-warmup", type=int, default=20)
    ap.add_argument("--num-iters", type=int, default=100)
    ap.add_argument("--timeout", type=int, default=600)
    ap.add_argument("--extra", nargs="*", default=[], help="extra flags passed to benchmark_ops, e.g. --symmetric")
    a = ap.parse_args()
    out = Path(a.out)
    out.mkdir(parents=True, exist_ok=True)
    failures = 0
    for n in a.ranks:
        for be in a.backends:
            for dt in a.datatypes:
                name = out / f"{be}_{dt}_{n}.txt"
                cmd = [str(BIN / "alrun"), "-n", str(n), "--timeout", str(a.timeout), str(BIN / "benchmark_ops"),
                       "--backend", be, "--op", ",".join(a.ops), "--datatype", dt, "--min-bytes", str(a.min_bytes),
                       "--max-bytes", str(a.max_bytes), "--num-warmup", str(a.num_warmup), "--num-iters", str(a.num_iters)]
                cmd += a.extra
                print(" ".join(cmd), flush=True)
                with open(name, "w") as f:
                    rc = subprocess.run(cmd, stdout=f, stderr=subprocess.STDOUT, timeout=a.timeout + 60).returncode
                if rc != 0:
                    failures += 1
                    print(f"  FAILED (rc={rc}), see {name}", file=sys.stderr)
    return 1 if failures else 0


if __name__ == "__main__":
    sys.exit(main())
