"""Integer helpers used when sizing buffers and batches."""


def ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def align(x: int, multiple: int) -> int:
    """``x`` rounded up to a multiple of ``multiple``."""
    return ceil_div(x, multiple) * multiple
