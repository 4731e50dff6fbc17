"""Merges per-rank perf traces (``traces-r*.jsonl``, one Chrome-trace event per line) into one JSON
file that chrome://tracing and Perfetto open, and prints a per-category / per-name time summary.

    python -m areal_b200.tools.perf_trace_converter TRACE_DIR_OR_FILE [-o out.json] [--summary]

Each rank becomes a process row (``pid`` = rank), each category a thread row. Counterpart of
areal/tools/perf_trace_converter.py.
"""

from __future__ import annotations

import argparse
import json
from collections import defaultdict

from ..utils.perf_tracer import convert_jsonl_to_chrome_trace


def summarize(trace_json: str) -> list[tuple[str, str, int, float]]:
    """``(category, name, count, total_ms)`` over the complete ('X') events, longest first."""
    events = json.load(open(trace_json))["traceEvents"]
    acc: dict[tuple[str, str], list[float]] = defaultdict(lambda: [0, 0.0])
    for e in events:
        if e.get("ph") == "X":
            a = acc[(e.get("cat", "misc"), e.get("name", "?"))]
            a[0] += 1
            a[1] += float(e.get("dur", 0.0)) / 1e3
    return sorted(((c, n, int(v[0]), v[1]) for (c, n), v in acc.items()), key=lambda r: -r[3])


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("src", help="directory with traces-r*.jsonl, or one such file")
    ap.add_argument("-o", "--output", default=None)
    ap.add_argument("--summary", action="store_true", help="print total time per (category, name)")
    args = ap.parse_args(argv)
    out = convert_jsonl_to_chrome_trace(args.src, args.output)
    print(out)
    if args.summary:
        for cat, name, n, ms in summarize(out):
            print(f"{cat:10s} {name:40s} n={n:6d} total={ms:10.2f} ms")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
