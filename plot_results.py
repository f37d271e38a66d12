#!/usr/bin/env python3
"""Plot decode-step latency (milliseconds, max over ranks) from the CSV written by run.py.

  --x B         latency vs global batch, one line per implementation
  --x num_sms   latency vs CTA count of the swept implementation (one line per batch), the
                other implementations drawn as horizontal reference bands

Same inputs and outputs as the reference's plot_results.py (CSV schema run.py:233-238; log2 x
axis with 1k/128k/1M tick labels, log y axis, last point annotated with %.2f ms, EP inferred
from the length of per_rank_counts).  matplotlib (Agg) is optional: without it the script
prints the table and draws the same chart itself as an SVG file (``--out`` with its extension
replaced by ``.svg``), so a machine without matplotlib still gets an image.
"""
from __future__ import annotations

import argparse
import csv
import statistics
import sys

IMPL_NAME = {"a2a": "A2A-V (peer ld/st)", "a2a-fp8": "A2A-V e4m3 dispatch", "dense": "dense AGV/RSV (multimem)",
             "nccl": "NCCL AllGather/RS", "deepep": "DeepEP-v2 (A2A)", "nvls": "reference NVLS (Triton)",
             "fused": "fused experts (tcgen05)"}
IMPL_COLOR = {"a2a": "tab:blue", "a2a-fp8": "tab:cyan", "dense": "tab:orange", "nccl": "tab:green",
              "deepep": "tab:blue", "nvls": "tab:red", "fused": "tab:cyan"}


def load(path):
    """-> (rows, ep).  rows: dicts impl, B, num_sms, ms.  Only ``decode_step`` rows are kept."""
    rows, ep = [], None
    with open(path, newline="") as f:
        for r in csv.DictReader(f):
            if r["phase"] != "decode_step":
                continue
            if ep is None:
                parts = [c for c in r.get("per_rank_counts", "").strip().strip("[]").split(",") if c.strip()]
                if parts:
                    ep = len(parts)
            rows.append({"impl": r["impl"], "B": int(r["global_B"]), "num_sms": int(r.get("num_sms", -1)),
                         "ms": float(r["latency_us"]) / 1000.0})
    return rows, ep


def ktick(v: int) -> str:
    if v >= 1 << 20:
        return f"{v >> 20}M"
    if v > 999:
        return f"{v >> 10}k"
    return str(v)


def subtitle(ep, shape="512 experts · top-k=22 · hidden=1024"):
    tail = f"{shape} · bf16 · CUDA-graph timing"
    if not ep:
        return tail
    return f"EP={ep} · {ep}×B200 · {tail}"


def series_vs_b(rows):
    out = {}
    for impl in sorted({r["impl"] for r in rows}):
        pts = sorted((r["B"], r["ms"]) for r in rows if r["impl"] == impl)
        out[impl] = pts
    return out


def text_table(rows) -> str:
    ser = series_vs_b(rows)
    bs = sorted({b for pts in ser.values() for b, _ in pts})
    lines = ["global_B " + " ".join(f"{i:>12s}" for i in ser)]
    for b in bs:
        cells = []
        for i in ser:
            d = dict(ser[i])
            cells.append(f"{d[b]:12.3f}" if b in d else " " * 12)
        lines.append(f"{ktick(b):>8s} " + " ".join(cells))
    return "\n".join(lines)


SVG_COLORS = {"tab:blue": "#1f77b4", "tab:cyan": "#17becf", "tab:orange": "#ff7f0e", "tab:green": "#2ca02c",
              "tab:red": "#d62728", "gray": "#7f7f7f"}


def render_svg(rows, title, xlabel="global batch size B  (decode tokens across all EP ranks)") -> str:
    """Latency-vs-B chart as a stand-alone SVG: log2 x axis with 1k/128k/1M ticks, log10 y axis,
    one line per implementation, last point annotated with %.2f ms."""
    import math
    ser = series_vs_b(rows)
    if not ser:
        return "<svg xmlns='http://www.w3.org/2000/svg' width='10' height='10'/>"
    W, H, L, R, T, B = 860, 540, 70, 150, 60, 60
    xs = sorted({b for pts in ser.values() for b, _ in pts})
    ys = [y for pts in ser.values() for _, y in pts if y > 0]
    x0, x1 = math.log2(xs[0]), math.log2(xs[-1]) if xs[-1] > xs[0] else math.log2(xs[0]) + 1
    y0, y1 = math.floor(math.log10(min(ys))), math.ceil(math.log10(max(ys)))
    if y1 == y0:
        y1 += 1

    def px(b):
        return L + (math.log2(b) - x0) / (x1 - x0) * (W - L - R)

    def py(v):
        return H - B - (math.log10(v) - y0) / (y1 - y0) * (H - T - B)

    out = [f"<svg xmlns='http://www.w3.org/2000/svg' width='{W}' height='{H}' font-family='sans-serif' font-size='11'>",
           f"<rect width='{W}' height='{H}' fill='white'/>"]
    for i, line in enumerate(title.split("\n")):
        out.append(f"<text x='{W / 2}' y='{22 + 15 * i}' text-anchor='middle' font-size='12'>{line}</text>")
    for e in range(y0, y1 + 1):
        y = py(10.0 ** e)
        out.append(f"<line x1='{L}' y1='{y:.1f}' x2='{W - R}' y2='{y:.1f}' stroke='#cccccc'/>")
        out.append(f"<text x='{L - 6}' y='{y + 4:.1f}' text-anchor='end'>{10.0 ** e:g}</text>")
        for m in range(2, 10):
            if e < y1:
                ym = py(m * 10.0 ** e)
                out.append(f"<line x1='{L}' y1='{ym:.1f}' x2='{W - R}' y2='{ym:.1f}' stroke='#eeeeee'/>")
    for b in xs:
        x = px(b)
        out.append(f"<line x1='{x:.1f}' y1='{T}' x2='{x:.1f}' y2='{H - B}' stroke='#eeeeee'/>")
        out.append(f"<text x='{x:.1f}' y='{H - B + 15}' text-anchor='middle'>{ktick(b)}</text>")
    out.append(f"<rect x='{L}' y='{T}' width='{W - L - R}' height='{H - T - B}' fill='none' stroke='black'/>")
    out.append(f"<text x='{(L + W - R) / 2}' y='{H - 18}' text-anchor='middle'>{xlabel}</text>")
    out.append(f"<text x='16' y='{(T + H - B) / 2}' text-anchor='middle' transform='rotate(-90 16 {(T + H - B) / 2})'>"
               "latency per decode step (ms)</text>")
    for i, (impl, pts) in enumerate(ser.items()):
        col = SVG_COLORS.get(IMPL_COLOR.get(impl, "gray"), "#7f7f7f")
        path = " ".join(f"{px(b):.1f},{py(v):.1f}" for b, v in pts if v > 0)
        out.append(f"<polyline points='{path}' fill='none' stroke='{col}' stroke-width='2'/>")
        for b, v in pts:
            if v > 0:
                out.append(f"<circle cx='{px(b):.1f}' cy='{py(v):.1f}' r='3' fill='{col}'/>")
        lb, lv = pts[-1]
        out.append(f"<text x='{px(lb) + 6:.1f}' y='{py(lv) + 4:.1f}' fill='{col}' font-size='10'>{lv:.2f}</text>")
        ly = T + 14 + 16 * i
        out.append(f"<line x1='{W - R + 40}' y1='{ly - 4}' x2='{W - R + 60}' y2='{ly - 4}' stroke='{col}' stroke-width='2'/>")
        out.append(f"<text x='{W - R + 64}' y='{ly}' font-size='9'>{IMPL_NAME.get(impl, impl)[:26]}</text>")
    out.append("</svg>")
    return "\n".join(out)


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--csv", default="results.csv")
    p.add_argument("--out", default="results.png")
    p.add_argument("--x", choices=["B", "num_sms"], default="B")
    p.add_argument("--num-layers", type=int, default=88, help="for the title only")
    p.add_argument("--title", default=None)
    p.add_argument("--sweep-impl", default="a2a", help="implementation whose num_sms was swept (--x num_sms)")
    args = p.parse_args(argv)
    rows, ep = load(args.csv)
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
        from matplotlib import cm
    except ImportError:
        print("matplotlib is not installed; table (ms per decode step) and a self-drawn SVG instead:")
        print(text_table(rows))
        if args.x == "B" and rows:
            svg_path = (args.out[:-4] if args.out.lower().endswith(".png") else args.out) + ".svg"
            title = args.title or (f"MoE decode dispatch+combine latency — {args.num_layers} MoE layers/step\n"
                                   f"{subtitle(ep)}")
            with open(svg_path, "w") as f:
                f.write(render_svg(rows, title))
            print(f"wrote {svg_path}")
        return 0
    fig, ax = plt.subplots(figsize=(8.5, 5.5))
    if args.x == "num_sms":
        swept = [r for r in rows if r["impl"] == args.sweep_impl]
        bs = sorted({r["B"] for r in swept})
        sms = sorted({r["num_sms"] for r in swept})
        for i, b in enumerate(bs):
            pts = sorted((r["num_sms"], r["ms"]) for r in swept if r["B"] == b)
            ax.plot([x for x, _ in pts], [y for _, y in pts], marker="o", lw=1.8, ms=5,
                    color=cm.viridis(i / max(1, len(bs) - 1)), label=f"{args.sweep_impl}  B={b}")
        for ref in sorted({r["impl"] for r in rows} - {args.sweep_impl}):
            vals = [r["ms"] for r in rows if r["impl"] == ref]
            m = statistics.mean(vals)
            ax.axhspan(min(vals), max(vals), color=IMPL_COLOR.get(ref, "gray"), alpha=0.12)
            ax.axhline(m, color=IMPL_COLOR.get(ref, "gray"), ls="--", lw=2,
                       label=f"{IMPL_NAME.get(ref, ref)} (~{m:.2f} ms)")
        ax.set_xscale("log", base=2)
        ax.set_xticks(sms)
        ax.set_xticklabels([str(s) for s in sms])
        ax.set_xlabel("CTA count (num_sms) of the swept implementation")
        title = f"MoE decode dispatch+combine vs num_sms — {args.num_layers} MoE layers/step\n{subtitle(ep)}"
    else:
        for impl, pts in series_vs_b(rows).items():
            xs, ys = [x for x, _ in pts], [y for _, y in pts]
            col = IMPL_COLOR.get(impl, "gray")
            ax.plot(xs, ys, marker="o", lw=2, ms=6, color=col, label=IMPL_NAME.get(impl, impl))
            ax.annotate(f"{ys[-1]:.2f}", (xs[-1], ys[-1]), textcoords="offset points", xytext=(6, 0),
                        fontsize=8, color=col)
        all_b = sorted({r["B"] for r in rows})
        ax.set_xscale("log", base=2)
        ax.set_xticks(all_b)
        ax.set_xticklabels([ktick(b) for b in all_b])
        ax.set_xlabel("global batch size B  (decode tokens across all EP ranks)")
        title = f"MoE decode dispatch+combine latency — {args.num_layers} MoE layers/step\n{subtitle(ep)}"
    ax.set_ylabel("latency per decode step (ms)")
    ax.set_yscale("log")
    ax.grid(True, which="both", alpha=0.3)
    ax.legend(loc="best", fontsize=8, ncol=2)
    ax.set_title(args.title or title, fontsize=10)
    fig.tight_layout()
    fig.savefig(args.out, dpi=150)
    print(f"wrote {args.out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
