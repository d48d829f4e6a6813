"""Tables and plots from benchmark_ops result files (role of benchmark/plot_benchmarks.py:220-309 of the
reference): time versus size per backend, time versus rank count, and a "who is faster" table.

    python benchmark/plot_benchmarks.py results/*.txt [--plot out.png] [--op allreduce]

Plotting needs matplotlib; without it only the text tables are produced.
"""
import argparse
import sys

import pandas as pd

COLS = ["Backend", "Type", "Operation", "Algo", "NonBlocking", "InPlace", "Root", "CommSize", "Bytes", "Median_us",
        "Mean_us", "Min_us", "Max_us", "BusGBs"]


def load(paths):
    rows = []
    for p in paths:
        for line in open(p):
            w = line.split()
            if len(w) == len(COLS) and w[8].isdigit():
                rows.append(w)
    df = pd.DataFrame(rows, columns=COLS)
    for c in ("CommSize", "Bytes"):
        df[c] = df[c].astype(int)
    for c in ("Median_us", "Mean_us", "Min_us", "Max_us", "BusGBs"):
        df[c] = df[c].astype(float)
    return df


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("files", nargs="+")
    ap.add_argument("--op", default=None)
    ap.add_argument("--plot", default=None)
    a = ap.parse_args()
    df = load(a.files)
    if a.op:
        df = df[df.Operation == a.op]
    if df.empty:
        print("no result rows found", file=sys.stderr)
        return 1
    pivot = df.pivot_table(index=["Operation", "CommSize", "Bytes"], columns="Backend", values="Median_us", aggfunc="min")
    if {"device", "nccl"} <= set(pivot.columns):
        pivot["nccl/device"] = pivot["nccl"] / pivot["device"]
    pd.set_option("display.width", 200, "display.max_rows", 500)
    print(pivot.round(2))
    best = pivot.drop(columns=[c for c in pivot.columns if "/" in c]).idxmin(axis=1)
    print("\nfastest backend per configuration:\n", best.value_counts())
    if a.plot:
        try:
            import matplotlib
            matplotlib.use("Agg")
            import matplotlib.pyplot as plt
        except ImportError:
            print("matplotlib not available: skipping the plot", file=sys.stderr)
            return 0
        ops = sorted(df.Operation.unique())
        fig, axes = plt.subplots(1, len(ops), figsize=(5 * len(ops), 4), squeeze=False)
        for ax, op in zip(axes[0], ops):
            for (be, n), g in df[df.Operation == op].groupby(["Backend", "CommSize"]):
                g = g.sort_values("Bytes")
                ax.loglog(g.Bytes, g.Median_us, marker="o", ms=3, label=f"{be} p={n}")
            ax.set_title(op)
            ax.set_xlabel("bytes")
            ax.set_ylabel("median us (max over ranks)")
            ax.legend(fontsize=7)
        fig.tight_layout()
        fig.savefig(a.plot, dpi=120)
    return 0


if __name__ == "__main__":
    sys.exit(main())
