"""Statistics as a compact multi-column table for the console."""

from __future__ import annotations


def tabulate_stats(data: dict[str, float], col: int = 4, floatfmt: str = ".4e") -> str:
    """``col`` key/value pairs per row, filled column by column (neighbouring keys stay under each other)."""
    items = list(data.items())
    if not items:
        return "(no stats)"
    rows = -(-len(items) // col)
    grid = []
    for i in range(rows):
        row = []
        for j in range(col):
            k = i + j * rows
            row.extend(items[k] if k < len(items) else (None, None))
        grid.append(row)
    try:
        from tabulate import tabulate

        return tabulate(grid, floatfmt=floatfmt, tablefmt="fancy_grid", missingval="")
    except ImportError:  # the package is optional: plain aligned columns
        fmt = lambda v: "" if v is None else (format(v, floatfmt) if isinstance(v, float) else str(v))
        cells = [[fmt(v) for v in row] for row in grid]
        widths = [max(len(r[c]) for r in cells) for c in range(2 * col)]
        return "\n".join("  ".join(v.ljust(w) for v, w in zip(r, widths)).rstrip() for r in cells)
