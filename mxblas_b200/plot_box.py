"""Summarise and plot a sweep written by ``python -m mxblas_b200.bench_all``.

    python -m mxblas_b200.plot_box bench_all.csv [--summary summary.md] [--figure boxplot.png]

Stands where the reference has bench/plot_box.py (a 2 x 2 grid of box plots, one panel per scaling pattern,
TFLOPS over M with one box per method). The same figure is drawn here when matplotlib is importable; the
summary table needs only pandas: per scaling pattern and M the median / minimum / maximum TFLOP/s of this
library over the model shapes, the median of cuBLASLt where it ran, and the ratio of the two medians.
"""

from __future__ import annotations

import argparse
from typing import Optional

import pandas as pd

PATTERNS = ["BB", "GB", "CC", "TT", "GG"]
OURS, LT = "MXBLAS_B200", "CUBLASLT"


def summary_table(df: pd.DataFrame) -> str:
    lines = ["| SP | M | shapes | ours TFLOP/s median (min .. max) | cuBLASLt median | ours / cuBLASLt | time vs TT on the same shape |",
             "|---|---|---|---|---|---|---|"]
    ours = df[df["Method"] == OURS]
    tt_ms = ours[ours["SP"] == "TT"].set_index(["Model", "M", "N", "K"])["Time(ms)"]
    for sp in PATTERNS:
        for m in sorted(ours[ours["SP"] == sp]["M"].unique()):
            sub = ours[(ours["SP"] == sp) & (ours["M"] == m)]
            tf = sub["TFLOPS"].dropna()
            if tf.empty:
                continue
            lt = df[(df["Method"] == LT) & (df["SP"] == sp) & (df["M"] == m)]["TFLOPS"].dropna()
            ratio = f"{tf.median() / lt.median():.2f}" if not lt.empty else "-"
            lt_txt = f"{lt.median():.0f}" if not lt.empty else "-"
            rel = "-"
            if sp != "TT" and not tt_ms.empty:
                own = sub.set_index(["Model", "M", "N", "K"])["Time(ms)"]
                both = own.index.intersection(tt_ms.index)
                if len(both):
                    rel = f"{(own[both] / tt_ms[both]).median():.2f}x"
            lines.append(f"| {sp} | {m} | {len(tf)} | {tf.median():.0f} ({tf.min():.0f} .. {tf.max():.0f}) | {lt_txt} | "
                         f"{ratio} | {rel} |")
    return "\n".join(lines) + "\n"


def box_plot(df: pd.DataFrame, path: str) -> bool:
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError:
        return False
    shown = [sp for sp in PATTERNS if not df[df["SP"] == sp].empty][:4]
    fig, axes = plt.subplots(2, 2, figsize=(20, 9))
    colors = {OURS: "#0b3c5d", LT: "#d9b310"}
    for ax, sp in zip(axes.flatten(), shown):
        sub = df[df["SP"] == sp]
        ms = sorted(sub["M"].unique())
        methods = [m for m in (LT, OURS) if m in set(sub["Method"])]
        width = 0.8 / max(len(methods), 1)
        for j, method in enumerate(methods):
            data = [sub[(sub["M"] == m) & (sub["Method"] == method)]["TFLOPS"].dropna().values for m in ms]
            pos = [i + (j - (len(methods) - 1) / 2) * width for i in range(len(ms))]
            bp = ax.boxplot(data, positions=pos, widths=width * 0.9, patch_artist=True, manage_ticks=False)
            for box in bp["boxes"]:
                box.set_facecolor(colors[method])
            ax.plot([], [], color=colors[method], linewidth=8, label=method)
        ax.set_xticks(range(len(ms)))
        ax.set_xticklabels([str(m) for m in ms])
        ax.set_title(f"SP = {sp[0]}x{sp[1]}")
        ax.set_xlabel("M")
        ax.set_ylabel("TFLOP/s")
        ax.grid(axis="y", linestyle="--", alpha=0.6)
        ax.legend()
    fig.tight_layout()
    fig.savefig(path, dpi=100)
    return True


def main(csv_path: str, summary: Optional[str], figure: Optional[str]) -> None:
    df = pd.read_csv(csv_path)
    text = summary_table(df)
    if summary:
        with open(summary, "w", encoding="utf-8") as f:
            f.write(text)
    print(text)
    if figure:
        print(f"figure written to {figure}" if box_plot(df, figure) else "matplotlib is not installed: no figure")


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("csv")
    ap.add_argument("--summary")
    ap.add_argument("--figure")
    a = ap.parse_args()
    main(a.csv, a.summary, a.figure)
