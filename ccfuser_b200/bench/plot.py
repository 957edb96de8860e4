"""Figures for the three evaluation experiments, drawn from the CSV files that ``bench/ae.py`` writes.

Counterpart of mix_moe/ae/fig10_plot.py, fig11_plot.py and fig12_plot.py (pandas + matplotlib + scipy there). Neither
plotting package is a dependency of this library, so the charts are written as plain SVG: grouped bars for the layer
and end-to-end experiments, stacked bars (compute + all-to-all) next to the fused kernels for the kernel experiment.

    python -m ccfuser_b200.bench.plot --data results --out results/figures

Files read (whichever exist): moe_layer_*.csv, e2e_model_*.csv, kernel_eval_*.csv, kernel_eval_expert_*.csv.
Extra CSV files with the same columns (for instance the recorded data of another system) can be laid into the same
chart with ``--overlay file.csv``; their series are appended.
"""
from __future__ import annotations

import argparse
import csv
import glob
import os
from typing import Dict, List, Optional, Sequence, Tuple

PALETTE = ["#4e79a7", "#f28e2b", "#59a14f", "#e15759", "#b07aa1", "#76b7b2", "#edc948", "#9c755f"]


def _read_csv(path: str) -> List[Dict[str, str]]:
    """Rows as dicts; header cells and values are stripped (the reference's recorded files carry stray blanks and a
    literal backslash-n in the header, mix_moe/ae/output_data/moe_layer_pcie.csv:1)."""
    with open(path, newline="") as f:
        rows = list(csv.reader(f))
    if not rows:
        return []
    header = [h.strip().replace("\\n", "") for h in rows[0]]
    out = []
    for r in rows[1:]:
        if not any(c.strip() for c in r):
            continue
        out.append({h: (r[i].strip() if i < len(r) else "") for i, h in enumerate(header)})
    return out


def _num(v: str) -> Optional[float]:
    try:
        return float(v)
    except (TypeError, ValueError):
        return None


def _nice_max(v: float) -> float:
    if v <= 0:
        return 1.0
    import math
    mag = 10 ** math.floor(math.log10(v))
    for m in (1, 2, 2.5, 5, 10):
        if v <= m * mag:
            return m * mag
    return 10 * mag


def bar_chart(path: str, title: str, categories: Sequence[str], series: Sequence[Tuple[str, Sequence[Optional[float]]]],
              ylabel: str, xlabel: str = "", stacked: Optional[Sequence[Tuple[str, Sequence[Optional[float]]]]] = None):
    """Grouped bars: one group per category, one bar per series. ``stacked`` optionally gives, for the same series
    names, the part of each bar that is drawn hatched at its bottom (e.g. the all-to-all share of a baseline)."""
    w, h, ml, mr, mt, mb = 760, 420, 70, 20, 50, 70
    pw, ph = w - ml - mr, h - mt - mb
    vals = [v for _, ys in series for v in ys if v is not None]
    ymax = _nice_max(max(vals) if vals else 1.0)
    n_cat, n_ser = max(1, len(categories)), max(1, len(series))
    gw = pw / n_cat
    bw = gw * 0.8 / n_ser
    stk = dict(stacked) if stacked else {}
    o = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{w}" height="{h}" viewBox="0 0 {w} {h}" '
         f'font-family="Helvetica,Arial,sans-serif" font-size="12">',
         '<defs><pattern id="hatch" width="6" height="6" patternTransform="rotate(45)" patternUnits="userSpaceOnUse">'
         '<line x1="0" y1="0" x2="0" y2="6" stroke="#000" stroke-width="1.2" opacity="0.55"/></pattern></defs>',
         f'<rect width="{w}" height="{h}" fill="#fff"/>',
         f'<text x="{w / 2}" y="24" text-anchor="middle" font-size="15">{_esc(title)}</text>']
    for i in range(6):
        yv = ymax * i / 5
        y = mt + ph - ph * i / 5
        o.append(f'<line x1="{ml}" y1="{y:.1f}" x2="{ml + pw}" y2="{y:.1f}" stroke="#bbb" stroke-dasharray="3,3"/>')
        o.append(f'<text x="{ml - 6}" y="{y + 4:.1f}" text-anchor="end">{yv:g}</text>')
    o.append(f'<text transform="translate(16,{mt + ph / 2}) rotate(-90)" text-anchor="middle">{_esc(ylabel)}</text>')
    if xlabel:
        o.append(f'<text x="{ml + pw / 2}" y="{h - 34}" text-anchor="middle">{_esc(xlabel)}</text>')
    for c, cat in enumerate(categories):
        x0 = ml + c * gw + gw * 0.1
        o.append(f'<text x="{ml + c * gw + gw / 2:.1f}" y="{mt + ph + 16}" text-anchor="middle">{_esc(str(cat))}</text>')
        for s, (name, ys) in enumerate(series):
            v = ys[c] if c < len(ys) else None
            if v is None:
                continue
            bh = ph * v / ymax
            x, y = x0 + s * bw, mt + ph - bh
            o.append(f'<rect x="{x:.1f}" y="{y:.1f}" width="{bw * 0.92:.1f}" height="{bh:.1f}" '
                     f'fill="{PALETTE[s % len(PALETTE)]}"><title>{_esc(name)}: {v:.4g}</title></rect>')
            part = stk.get(name)
            pv = part[c] if part is not None and c < len(part) else None
            if pv:
                sh = ph * min(pv, v) / ymax
                o.append(f'<rect x="{x:.1f}" y="{mt + ph - sh:.1f}" width="{bw * 0.92:.1f}" height="{sh:.1f}" '
                         f'fill="url(#hatch)"/>')
    o.append(f'<line x1="{ml}" y1="{mt + ph}" x2="{ml + pw}" y2="{mt + ph}" stroke="#000"/>')
    o.append(f'<line x1="{ml}" y1="{mt}" x2="{ml}" y2="{mt + ph}" stroke="#000"/>')
    lx = ml
    for s, (name, _) in enumerate(series):
        o.append(f'<rect x="{lx}" y="{h - 22}" width="12" height="12" fill="{PALETTE[s % len(PALETTE)]}"/>')
        o.append(f'<text x="{lx + 16}" y="{h - 12}">{_esc(name)}</text>')
        lx += 28 + 7 * len(name)
    if stk:
        o.append(f'<rect x="{lx}" y="{h - 22}" width="12" height="12" fill="url(#hatch)" stroke="#000" stroke-width="0.5"/>')
        o.append(f'<text x="{lx + 16}" y="{h - 12}">all-to-all share</text>')
    o.append("</svg>")
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        f.write("\n".join(o))
    return path


def _esc(s: str) -> str:
    return s.replace("&", "&amp;").replace("<", "&lt;").replace(">", "&gt;")


# ---------------------------------------------------------------------------------------------------------------
def plot_layer(rows: List[Dict[str, str]], out_prefix: str, tag: str) -> List[str]:
    """fig. 10: forward / backward / total time of one MoE layer over experts per GPU, one series per system."""
    names = list(dict.fromkeys(r["name"] for r in rows))
    cats = sorted({int(float(r["num_expert"])) for r in rows if _num(r.get("num_expert"))})
    paths = []
    for col, what in (("total_time", "total"), ("forward_time", "forward"), ("backward_time", "backward")):
        series = []
        for n in names:
            by = {int(float(r["num_expert"])): _num(r.get(col)) for r in rows if r["name"] == n and _num(r.get("num_expert"))}
            series.append((n, [by.get(c) for c in cats]))
        paths.append(bar_chart(f"{out_prefix}moe_layer_{what}_{tag}.svg", f"MoE layer, {what} time", [str(c) for c in cats],
                               series, "time (ms)", "experts per GPU"))
    return paths


def plot_e2e(rows: List[Dict[str, str]], out_prefix: str, tag: str) -> List[str]:
    """fig. 11: step time of the three models, one series per system."""
    models = [k for k in rows[0].keys() if k != "name"] if rows else []
    series = [(r["name"], [_num(r.get(m)) for m in models]) for r in rows]
    return [bar_chart(f"{out_prefix}e2e_model_{tag}.svg", "End-to-end training step", models, series, "time per step (ms)")]


def plot_kernels(rows: List[Dict[str, str]], out_prefix: str, tag: str, by_expert: bool) -> List[str]:
    """fig. 12: fused dispatch+GEMM ("AG") and GEMM+combine ("GA") against all-to-all + GEMM; the baselines' bars show
    their all-to-all share hatched. The x axis is the remote fraction of the rows or the experts per GPU."""
    key = "num_expert" if by_expert else "locality"
    # the reference's recorded files give num_expert on one row of each group of four only: carry it forward
    last = None
    for r in reversed(rows):
        if by_expert:
            if r.get("num_expert"):
                last = r["num_expert"]
            elif last is not None:
                r["num_expert"] = last
    cats: List[str] = []
    for r in rows:
        c = r.get(key, "")
        if by_expert or r["kernel"] in ("AG", "GA"):
            if c and c not in cats:
                cats.append(c)
    paths = []
    for fused, base, what in (("AG", "All2All-GEMM", "dispatch + GEMM-1"), ("GA", "GEMM-All2All", "GEMM-2 + combine")):
        f_rows = [r for r in rows if r["kernel"] == fused]
        b_rows = [r for r in rows if r["kernel"] == base]
        if not f_rows:
            continue
        n = min(len(f_rows), len(b_rows)) if b_rows else len(f_rows)
        labels = [f_rows[i].get(key, str(i)) for i in range(n)]
        series = [(f"fused {fused}", [_num(f_rows[i]["time"]) for i in range(n)])]
        stacked = None
        if b_rows:
            series.append((base, [_num(b_rows[i]["time"]) for i in range(n)]))
            stacked = [(base, [_num(b_rows[i].get("all2all")) for i in range(n)])]
        suffix = "expert" if by_expert else "locality"
        paths.append(bar_chart(f"{out_prefix}kernel_execution_{suffix}_{fused}_{tag}.svg", f"{what}", labels, series,
                               "time (ms)", "experts per GPU" if by_expert else "fraction of remote rows", stacked))
    return paths


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--data", default="results")
    ap.add_argument("--out", default="results/figures")
    ap.add_argument("--overlay", action="append", default=[], help="extra CSV with the same columns; rows are appended")
    a = ap.parse_args(argv)
    prefix = os.path.join(a.out, "")
    made: List[str] = []

    def with_overlay(rows, columns):
        for extra in a.overlay:
            er = _read_csv(extra)
            if er and set(columns) <= set(er[0].keys()):
                rows = rows + er
        return rows

    for path in sorted(glob.glob(os.path.join(a.data, "*.csv"))):
        base = os.path.basename(path)
        tag = os.path.splitext(base)[0]
        for known in ("moe_layer_", "e2e_model_", "kernel_eval_expert_", "kernel_eval_"):
            if tag.startswith(known):
                tag = tag[len(known):]
                break
        rows = _read_csv(path)
        if not rows:
            continue
        cols = set(rows[0].keys())
        if {"name", "num_expert", "total_time"} <= cols:
            made += plot_layer(with_overlay(rows, ["name", "num_expert", "total_time"]), prefix, tag)
        elif "name" in cols and len(cols) > 1 and "kernel" not in cols:
            made += plot_e2e(with_overlay(rows, list(cols)), prefix, tag)
        elif {"kernel", "time"} <= cols:
            made += plot_kernels(rows, prefix, tag, by_expert="num_expert" in cols)
    for p in made:
        print(p)
    return made


if __name__ == "__main__":
    main()
