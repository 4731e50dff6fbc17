"""Summarises and draws rollout session traces (``sessions-r*.jsonl`` written by the session tracer):
per-phase time statistics on stdout and a self-contained HTML page with one SVG timeline row per
session (phases coloured by name, rejected / failed sessions outlined).

    python -m areal_b200.tools.plot_session_trace TRACE_DIR_OR_FILE [-o sessions.html] [--max-rows 400]

Needs no plotting library. Counterpart of areal/tools/plot_session_trace.py.
"""

from __future__ import annotations

import argparse
import glob
import html
import json
import os
import statistics
from collections import defaultdict

PALETTE = ["#4e79a7", "#f28e2b", "#59a14f", "#e15759", "#b07aa1", "#76b7b2", "#edc948", "#9c755f"]


def load(src: str) -> list[dict]:
    files = sorted(glob.glob(os.path.join(src, "sessions-r*.jsonl"))) if os.path.isdir(src) else [src]
    out = []
    for f in files:
        with open(f) as fh:
            out += [json.loads(line) for line in fh if line.strip()]
    return sorted(out, key=lambda r: r["start"])


def summarize(records: list[dict]) -> dict:
    phases: dict[str, list[float]] = defaultdict(list)
    for r in records:
        for p in r.get("phases", []):
            phases[p["name"]].append(p["end"] - p["start"])
    total = [r["end"] - r["start"] for r in records if r.get("end")]
    status: dict[str, int] = defaultdict(int)
    for r in records:
        status[r.get("status", "?")] += 1
    return {"sessions": len(records), "status": dict(status),
            "session_s": _stats(total), "phases": {k: _stats(v) for k, v in sorted(phases.items())}}


def _stats(xs: list[float]) -> dict:
    if not xs:
        return {"n": 0}
    xs = sorted(xs)
    return {"n": len(xs), "mean": statistics.fmean(xs), "p50": xs[len(xs) // 2], "p95": xs[min(len(xs) - 1, int(0.95 * len(xs)))],
            "max": xs[-1], "total": sum(xs)}


def render_html(records: list[dict], max_rows: int = 400, width: int = 1200) -> str:
    records = records[:max_rows]
    if not records:
        return "<html><body>no sessions</body></html>"
    t0 = min(r["start"] for r in records)
    t1 = max((r.get("end") or r["start"]) for r in records)
    span = max(t1 - t0, 1e-6)
    names = sorted({p["name"] for r in records for p in r.get("phases", [])})
    color = {n: PALETTE[i % len(PALETTE)] for i, n in enumerate(names)}
    row_h, pad = 10, 2
    x = lambda t: (t - t0) / span * width
    parts = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{len(records) * (row_h + pad)}">']
    for i, r in enumerate(records):
        y = i * (row_h + pad)
        end = r.get("end") or t1
        stroke = {"accepted": "none", "running": "#999"}.get(r.get("status"), "#d00")
        parts.append(f'<rect x="{x(r["start"]):.1f}" y="{y}" width="{max(x(end) - x(r["start"]), 1):.1f}" height="{row_h}" '
                     f'fill="#eee" stroke="{stroke}"><title>session {r["session_id"]} task {r.get("task_id")} '
                     f'{html.escape(str(r.get("status")))} {end - r["start"]:.2f}s</title></rect>')
        for p in r.get("phases", []):
            parts.append(f'<rect x="{x(p["start"]):.1f}" y="{y}" width="{max(x(p["end"]) - x(p["start"]), 0.5):.1f}" '
                         f'height="{row_h}" fill="{color[p["name"]]}"><title>{html.escape(p["name"])} '
                         f'{p["end"] - p["start"]:.3f}s</title></rect>')
    parts.append("</svg>")
    legend = " ".join(f'<span style="background:{c};color:#fff;padding:2px 6px">{html.escape(n)}</span>' for n, c in color.items())
    return (f"<html><body style='font-family:sans-serif'><h3>{len(records)} sessions over {span:.1f} s</h3>"
            f"<p>{legend}</p>{''.join(parts)}</body></html>")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("src")
    ap.add_argument("-o", "--output", default=None)
    ap.add_argument("--max-rows", type=int, default=400)
    args = ap.parse_args(argv)
    records = load(args.src)
    print(json.dumps(summarize(records), indent=2))
    out = args.output or (os.path.join(args.src, "sessions.html") if os.path.isdir(args.src) else os.path.splitext(args.src)[0] + ".html")
    with open(out, "w") as f:
        f.write(render_html(records, args.max_rows))
    print(out)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
