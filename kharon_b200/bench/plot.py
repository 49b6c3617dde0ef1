"""Charts of ``results.json`` without a display (counterpart of the reference's bench/plot.py, which
renders PNGs with matplotlib's Agg backend, bench/plot.py:5-6).

    python -m kharon_b200.bench.plot [results.json] [out_dir]

With matplotlib installed the charts are PNGs drawn with the Agg backend; without it the same
charts are written as SVG by the small writer below, so the harness has no hard dependency.
"""
from __future__ import annotations

import json
import math
import os
import sys

COLORS = ["#1f77b4", "#d62728", "#2ca02c", "#9467bd", "#ff7f0e"]


def _svg_lines(title, xlabel, ylabel, xs, series, path, logy=True):
    """series: [(name, [y or None])].  Categorical x axis, optional log y."""
    W, H, L, R, T, B = 640, 420, 80, 20, 40, 60
    vals = [v for _, ys in series for v in ys if v]
    lo, hi = min(vals), max(vals)
    if logy:
        f = lambda v: math.log10(v)
        lo_t, hi_t = math.floor(f(lo)), math.ceil(f(hi))
    else:
        f = lambda v: v
        lo_t, hi_t = 0.0, hi * 1.1
    px = lambda i: L + (W - L - R) * (i + 0.5) / len(xs)
    py = lambda v: H - B - (H - T - B) * (f(v) - lo_t) / max(hi_t - lo_t, 1e-9)
    out = ['<svg xmlns="http://www.w3.org/2000/svg" width="%d" height="%d" font-family="sans-serif" font-size="12">' % (W, H),
           '<rect width="100%" height="100%" fill="white"/>',
           '<text x="%d" y="22" font-size="15" text-anchor="middle">%s</text>' % (W // 2, title),
           '<text x="%d" y="%d" text-anchor="middle">%s</text>' % (W // 2, H - 15, xlabel),
           '<text x="16" y="%d" text-anchor="middle" transform="rotate(-90 16 %d)">%s</text>' % (H // 2, H // 2, ylabel),
           '<line x1="%d" y1="%d" x2="%d" y2="%d" stroke="black"/>' % (L, H - B, W - R, H - B),
           '<line x1="%d" y1="%d" x2="%d" y2="%d" stroke="black"/>' % (L, T, L, H - B)]
    ticks = [10 ** e for e in range(int(lo_t), int(hi_t) + 1)] if logy else [hi_t * k / 5 for k in range(6)]
    for t in ticks:
        if t <= 0 and logy:
            continue
        y = py(t) if t > 0 or not logy else H - B
        out.append('<line x1="%d" y1="%.1f" x2="%d" y2="%.1f" stroke="#ddd"/>' % (L, y, W - R, y))
        out.append('<text x="%d" y="%.1f" text-anchor="end">%s</text>' % (L - 6, y + 4, ("%g" % t)))
    for i, x in enumerate(xs):
        out.append('<text x="%.1f" y="%d" text-anchor="middle">%s</text>' % (px(i), H - B + 18, x))
    for k, (name, ys) in enumerate(series):
        c = COLORS[k % len(COLORS)]
        pts = [(px(i), py(v)) for i, v in enumerate(ys) if v]
        if len(pts) > 1:
            out.append('<polyline fill="none" stroke="%s" stroke-width="2" points="%s"/>' %
                       (c, " ".join("%.1f,%.1f" % p for p in pts)))
        for p in pts:
            out.append('<circle cx="%.1f" cy="%.1f" r="4" fill="%s"/>' % (p[0], p[1], c))
        out.append('<rect x="%d" y="%d" width="12" height="12" fill="%s"/>' % (L + 12, T + 6 + 18 * k, c))
        out.append('<text x="%d" y="%d">%s</text>' % (L + 30, T + 17 + 18 * k, name))
    out.append("</svg>")
    with open(path, "w") as fh:
        fh.write("\n".join(out))
    return path


def _mpl_lines(plt, title, xlabel, ylabel, xs, series, path, logy=True):
    fig, ax = plt.subplots(figsize=(6.4, 4.2))
    for name, ys in series:
        idx = [i for i, v in enumerate(ys) if v]
        ax.plot(idx, [ys[i] for i in idx], marker="o", label=name)
    ax.set_xticks(range(len(xs)))
    ax.set_xticklabels([str(x) for x in xs])
    if logy:
        ax.set_yscale("log")
    ax.set_title(title); ax.set_xlabel(xlabel); ax.set_ylabel(ylabel); ax.grid(True, alpha=0.3); ax.legend()
    fig.tight_layout()
    fig.savefig(path, dpi=120)
    plt.close(fig)
    return path


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    here = os.path.dirname(os.path.abspath(__file__))
    src = argv[0] if argv else os.path.join(here, "results.json")
    out_dir = argv[1] if len(argv) > 1 else os.path.join(here, "plots")
    os.makedirs(out_dir, exist_ok=True)
    res = json.load(open(src))
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
        draw, ext = (lambda *a, **k: _mpl_lines(plt, *a, **k)), "png"
    except ImportError:
        draw, ext = _svg_lines, "svg"
    made = []
    t = res.get("train_1p2b")
    if t:
        made.append(draw("1.2B GPT training throughput", "GPUs (mesh of the 3-D sweep)", "tokens / s", t["gpus"],
                         [("this framework, B200", t["ours_tok_s"]), ("reference rebuilt, same B200s", t["reference_b200_tok_s"]),
                          ("reference published, L40S", t["reference_l40s_tok_s"])],
                         os.path.join(out_dir, "train_scaling." + ext)))
    d = res.get("decode_l24_d1024")
    if d:
        made.append(draw("Paged-KV decode, L24 d1024", "sequences in flight (G)", "tokens / s", d["G"],
                         [("this framework, 1 x B200", d["ours_tok_s"]), ("this framework, TP2", d["ours_tp2_tok_s"]),
                          ("reference rebuilt, B200", d["reference_b200_tok_s"]), ("reference published, L40S", d["reference_l40s_tok_s"])],
                         os.path.join(out_dir, "decode." + ext)))
    g = res.get("gemm_bf16_tflops")
    if g:
        made.append(draw("bf16 GEMM (tcgen05)", "shape", "TFLOP/s", [s.split()[0] for s in g["shapes"]],
                         [("this framework", g["ours"]), ("cuBLAS sustained peak", [g["measured_peak_sustained"]] * len(g["shapes"]))],
                         os.path.join(out_dir, "gemm." + ext), logy=False))
    for m in made:
        print("wrote", m)
    return made


if __name__ == "__main__":
    main()
