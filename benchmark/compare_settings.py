"""Side-by-side timing of one benchmark_ops sweep under several settings of the tuning table.

Every setting is a name plus `AL_*` environment variables (and, optionally, extra benchmark_ops
flags); the same sweep runs once per setting and one table per operation shows, for every size,
the median time under each setting, its ratio to the first setting and which one is fastest.
This is how a cross-over point or an opt-in data path is judged on a given machine:

    python benchmark/compare_settings.py --ranks 8 --ops allgather alltoall --min-bytes 1048576 \\
        --setting default --setting pipe8m:AL_PIPELINE_MIN=8388609 \\
        --setting bulk:AL_DEV_BULK_PIPELINE=1,AL_DEV_BULK_PUB_CTAS=16

    python benchmark/compare_settings.py --ranks 8 --nodes 2 --backend host --ops allreduce \\
        --setting two-level --setting flat:AL_HOST_TWO_LEVEL=0

A setting is `name[:VAR=value[,VAR=value...]][:flag flag ...]`, e.g. `win64:AL_WINDOW_CTAS=64:--symmetric`.
The table is Markdown on stdout (and in --out when given).  Role: the tuning side of the
reference's benchmark/run_benchmarks.py + plot_benchmarks.py "best implementation" heat-map
(benchmark/plot_benchmarks.py:220-309), for one library under different settings.
"""
import argparse
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "aluminum_b200" / "bin"


def parse_setting(text):
    parts = text.split(":")
    name = parts[0]
    env, flags = {}, []
    for part in parts[1:]:
        if "=" in part and not part.lstrip().startswith("-"):
            for kv in part.split(","):
                k, v = kv.split("=", 1)
                env[k.strip()] = v.strip()
        elif part.strip():
            flags += part.split()
    return name, env, flags


def parse_table(text):
    """{(operation, bytes): median_us} from benchmark_ops output."""
    out = {}
    for line in text.splitlines():
        w = line.split()
        if len(w) == 14 and w[8].isdigit():
            try:
                out[(w[2], int(w[8]))] = float(w[9])
            except ValueError:
                pass
    return out


def human(n):
    for unit, k in (("GiB", 1 << 30), ("MiB", 1 << 20), ("KiB", 1 << 10)):
        if n >= k and n % k == 0:
            return f"{n // k} {unit}"
    return f"{n} B"


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--ranks", type=int, default=2)
    ap.add_argument("--nodes", type=int, default=0, help="modelled nodes (alrun --nodes)")
    ap.add_argument("--backend", default="device")
    ap.add_argument("--ops", nargs="+", default=["allreduce"])
    ap.add_argument("--datatype", default="float")
    ap.add_argument("--min-bytes", type=int, default=8)
    ap.add_argument("--max-bytes", type=int, default=1 << 26)
    ap.add_argument("--num-warmup", type=int, default=10)
    ap.add_argument("--num-iters", type=int, default=40)
    ap.add_argument("--timeout", type=int, default=600)
    ap.add_argument("--setting", action="append", default=[], help="name[:VAR=value,...][:flags]; first one is the reference")
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    settings = [parse_setting(s) for s in (a.setting or ["default"])]
    results, failed = {}, []
    for name, env, flags in settings:
        print(f"# {name}: {' '.join(f'{k}={v}' for k, v in env.items())} {' '.join(flags)}".rstrip(), file=sys.stderr, flush=True)
        table = {}
        for op in a.ops:  # one run per operation: the host path of benchmark_ops takes one at a time
            cmd = [str(BIN / "alrun"), "-n", str(a.ranks)] + (["--nodes", str(a.nodes)] if a.nodes else []) + \
                  ["--timeout", str(a.timeout), str(BIN / "benchmark_ops"), "--backend", a.backend, "--op", op,
                   "--datatype", a.datatype, "--min-bytes", str(a.min_bytes), "--max-bytes", str(a.max_bytes),
                   "--num-warmup", str(a.num_warmup), "--num-iters", str(a.num_iters)] + flags
            r = subprocess.run(cmd, env={**os.environ, **env}, capture_output=True, text=True, timeout=a.timeout + 60)
            if r.returncode != 0:
                failed.append(f"{name}/{op}")
                print(f"  {op} FAILED (rc={r.returncode}):\n{(r.stdout + r.stderr)[-2000:]}", file=sys.stderr)
                continue
            table.update(parse_table(r.stdout))
        if table:
            results[name] = table
    names = [n for n, _, _ in settings if n in results]
    lines = []
    if names:
        ref = names[0]
        for op in a.ops:
            sizes = sorted({b for n in names for (o, b) in results[n] if o == op})
            if not sizes:
                continue
            lines += [f"### {op}, {a.ranks} ranks, {a.backend}, {a.datatype} (median us; ratio = {ref} / setting)", ""]
            lines.append("| bytes | " + " | ".join(names) + " | fastest |")
            lines.append("|---|" + "---|" * (len(names) + 1))
            for b in sizes:
                base = results[ref].get((op, b))
                cells, best, best_t = [], "-", None
                for n in names:
                    t = results[n].get((op, b))
                    if t is None:
                        cells.append("-")
                        continue
                    cells.append(f"{t:.1f}" if n == ref or not base else f"{t:.1f} ({base / t:.2f})")
                    if best_t is None or t < best_t:
                        best, best_t = n, t
                lines.append(f"| {human(b)} | " + " | ".join(cells) + f" | {best} |")
            lines.append("")
    text = "\n".join(lines)
    print(text)
    if a.out:
        Path(a.out).write_text(text + "\n")
    return 1 if failed or not names else 0


if __name__ == "__main__":
    sys.exit(main())
