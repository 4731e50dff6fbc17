"""Sequence packing / partitioning front-end.

The heavy lifting is in the C++ host library (``csrc/host/seqpack.cpp``); every
function also has a pure-Python fallback with the same results, used when the
library has not been built and as the oracle in tests. Counterpart of
areal/utils/seqpack.py:22-615 in the reference.
"""

from __future__ import annotations

import ctypes
import heapq
from typing import Any, Sequence

import numpy as np

from ..ops import _lib

PACKING_ALGORITHMS = ("ffd", "kk")


def _i64(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.int64))


def _ffd_py(sizes, capacity, min_groups):
    order = sorted(range(len(sizes)), key=lambda i: -sizes[i])
    load, count = [0] * min_groups, [0] * min_groups
    out = [0] * len(sizes)
    for idx in order:
        s = sizes[idx]
        if s > capacity:
            raise ValueError(f"sequence of {s} tokens exceeds the micro-batch capacity {capacity}")
        chosen = next((b for b in range(min_groups) if count[b] == 0), -1)
        if chosen < 0:
            chosen = next((b for b in range(len(load)) if load[b] + s <= capacity), -1)
        if chosen < 0:
            load.append(0)
            count.append(0)
            chosen = len(load) - 1
        load[chosen] += s
        count[chosen] += 1
        out[idx] = chosen
    return out, len(load)


def ffd_allocate(sizes: Sequence[int], capacity: int, min_groups: int = 1) -> list[list[int]]:
    """First-fit-decreasing: groups of item indices, each group's total ≤ ``capacity``,
    at least ``min_groups`` groups (some may be empty only if there are fewer items)."""
    n = len(sizes)
    if n == 0:
        return [[] for _ in range(min_groups)]
    sizes = [int(s) for s in sizes]
    if _lib.have_host():
        arr = _i64(sizes)
        out = np.empty(n, dtype=np.int32)
        fn = _lib.host().b200_ffd_allocate
        fn.restype = ctypes.c_int
        nb = fn(arr.ctypes.data_as(ctypes.c_void_p), ctypes.c_int(n), ctypes.c_int64(int(capacity)),
                ctypes.c_int(int(min_groups)), out.ctypes.data_as(ctypes.c_void_p))
        if nb < 0:
            raise ValueError(f"a sequence exceeds the micro-batch capacity {capacity}")
        bins = out.tolist()
    else:
        bins, nb = _ffd_py(sizes, capacity, min_groups)
    groups: list[list[int]] = [[] for _ in range(max(nb, min_groups))]
    for i, b in enumerate(bins):
        groups[b].append(i)
    return [g for g in groups if g] if n >= min_groups else groups


def _kk_py(sizes, k, equal_size):
    # heap entries: (-spread, -largest_sum, tiebreak, sums(list desc), sets)
    heap = []
    cnt = 0
    if equal_size:
        order = sorted(range(len(sizes)), key=lambda i: -sizes[i])
        for i in range(0, len(order), k):
            sums, sets = [0] * k, [[] for _ in range(k)]
            for j, idx in enumerate(order[i:i + k]):
                sums[j] = sizes[idx]
                sets[j] = [idx]
            heapq.heappush(heap, (-(sums[0] - sums[-1]), -sums[0], cnt, sums, sets))
            cnt += 1
    else:
        for i, s in enumerate(sizes):
            sums, sets = [0] * k, [[] for _ in range(k)]
            sums[0], sets[0] = s, [i]
            heapq.heappush(heap, (-s, -s, cnt, sums, sets))
            cnt += 1
    while len(heap) > 1:
        _, _, _, sa, seta = heapq.heappop(heap)
        _, _, _, sb, setb = heapq.heappop(heap)
        parts = sorted(((sa[j] + sb[k - 1 - j], seta[j] + setb[k - 1 - j]) for j in range(k)),
                       key=lambda p: -p[0])
        sums = [p[0] for p in parts]
        sets = [p[1] for p in parts]
        heapq.heappush(heap, (-(sums[0] - sums[-1]), -sums[0], cnt, sums, sets))
        cnt += 1
    return heap[0][4] if heap else [[] for _ in range(k)]


def kk_allocate(sizes: Sequence[int], k: int, equal_size: bool = False) -> list[list[int]]:
    """Karmarkar–Karp k-way partition (balanced sums). Returns ``k`` index lists."""
    n = len(sizes)
    sizes = [int(s) for s in sizes]
    if n == 0:
        return [[] for _ in range(k)]
    if _lib.have_host():
        arr = _i64(sizes)
        out = np.empty(n, dtype=np.int32)
        fn = _lib.host().b200_kk_partition
        fn.restype = ctypes.c_int
        rc = fn(arr.ctypes.data_as(ctypes.c_void_p), ctypes.c_int(n), ctypes.c_int(k),
                ctypes.c_int(int(equal_size)), out.ctypes.data_as(ctypes.c_void_p))
        if rc < 0:
            raise ValueError("kk_partition failed")
        groups = [[] for _ in range(k)]
        for i, g in enumerate(out.tolist()):
            groups[g].append(i)
        return groups
    return [sorted(g) for g in _kk_py(sizes, k, equal_size)]


def partition_balanced(sizes: Sequence[int], k: int, min_size: int = 1) -> list[int]:
    """Contiguous k-way partition minimising the largest part; returns ``k+1`` boundaries."""
    n = len(sizes)
    if n < k * min_size:
        raise ValueError(f"cannot split {n} items into {k} parts of at least {min_size}")
    if _lib.have_host():
        arr = _i64(sizes)
        out = np.empty(k + 1, dtype=np.int32)
        fn = _lib.host().b200_partition_balanced
        fn.restype = ctypes.c_int
        rc = fn(arr.ctypes.data_as(ctypes.c_void_p), ctypes.c_int(n), ctypes.c_int(k),
                ctypes.c_int(min_size), out.ctypes.data_as(ctypes.c_void_p))
        if rc < 0:
            raise ValueError("partition_balanced failed")
        return out.tolist()
    pre = [0]
    for s in sizes:
        pre.append(pre[-1] + int(s))
    INF = float("inf")
    dp = [[INF] * (n + 1) for _ in range(k + 1)]
    arg = [[-1] * (n + 1) for _ in range(k + 1)]
    dp[0][0] = 0
    for j in range(1, k + 1):
        for i in range(j * min_size, n - (k - j) * min_size + 1):
            for p in range((j - 1) * min_size, i - min_size + 1):
                if dp[j - 1][p] == INF:
                    continue
                c = max(dp[j - 1][p], pre[i] - pre[p])
                if c < dp[j][i]:
                    dp[j][i], arg[j][i] = c, p
    bounds = [0] * (k + 1)
    bounds[k] = n
    i = n
    for j in range(k, 0, -1):
        i = arg[j][i]
        bounds[j - 1] = i
    return bounds


def balanced_greedy_partition(sizes: Sequence[int], k: int, equal_size: bool = True) -> list[list[int]]:
    """Largest-first greedy into the lightest of ``k`` groups; with ``equal_size`` every
    group receives at most ``ceil(n/k)`` items."""
    n = len(sizes)
    sizes = [int(s) for s in sizes]
    if _lib.have_host() and n:
        arr = _i64(sizes)
        out = np.empty(n, dtype=np.int32)
        fn = _lib.host().b200_greedy_partition
        fn.restype = ctypes.c_int
        fn(arr.ctypes.data_as(ctypes.c_void_p), ctypes.c_int(n), ctypes.c_int(k),
           ctypes.c_int(int(equal_size)), out.ctypes.data_as(ctypes.c_void_p))
        bins = out.tolist()
    else:
        load, count, bins = [0] * k, [0] * k, [0] * n
        cap = -(-n // k) if n else 0
        for idx in sorted(range(n), key=lambda i: -sizes[i]):
            cands = [g for g in range(k) if not equal_size or count[g] < cap]
            best = min(cands, key=lambda g: (load[g], g))
            load[best] += sizes[idx]
            count[best] += 1
            bins[idx] = best
    groups = [[] for _ in range(k)]
    for i, g in enumerate(bins):
        groups[g].append(i)
    return groups


def allocate(sizes: Sequence[int], capacity: int | None, min_groups: int, algorithm: str = "ffd",
             divisor: int = 1) -> list[list[int]]:
    """Micro-batch allocation used by the engines: at least ``min_groups`` groups (rounded
    up to a multiple of ``divisor``), none above ``capacity`` tokens."""
    total = sum(int(s) for s in sizes)
    k = max(min_groups, 1)
    if capacity is not None:
        k = max(k, -(-total // capacity))
    k = -(-k // divisor) * divisor
    if algorithm == "kk":
        while True:
            groups = [g for g in kk_allocate(sizes, k) if g] if len(sizes) >= k else \
                kk_allocate(sizes, k)
            if capacity is None or all(sum(int(sizes[i]) for i in g) <= capacity for g in groups):
                return groups
            k += divisor
    groups = ffd_allocate(sizes, capacity if capacity is not None else max(total, 1), k)
    while len(groups) % divisor:
        # split the heaviest splittable group to reach the divisor
        heavy = max((g for g in groups if len(g) > 1), key=lambda g: sum(int(sizes[i]) for i in g),
                    default=None)
        if heavy is None:
            break
        groups.remove(heavy)
        half = len(heavy) // 2
        groups += [heavy[:half], heavy[half:]]
    return groups


# ------------------------------------------------------------------ further partition helpers
def get_allocate_fn(algorithm: str = "ffd"):
    """``ffd_allocate`` or ``kk_allocate`` by name (the value of ``MicroBatchSpec.packing_algorithm``)."""
    table = {"ffd": ffd_allocate, "kk": kk_allocate}
    if algorithm not in table:
        raise ValueError(f"unknown packing algorithm {algorithm!r}; supported: {sorted(table)}")
    return table[algorithm]


def partition_balanced_tuples(sizes: Sequence[int], k: int, min_size: int = 1) -> list[tuple[int, int]]:
    """:func:`partition_balanced` as ``(start, end)`` pairs."""
    b = partition_balanced(sizes, k, min_size)
    return list(zip(b[:-1], b[1:]))


def min_abs_diff_partition(sizes: Sequence[int], k: int, min_size: int = 1) -> list[tuple[int, int]]:
    """Contiguous split of a 1-D array into ``k`` non-empty ranges of at least ``min_size`` items whose largest sum
    is as small as possible (micro-batches of a pipeline, shards of a sorted batch)."""
    arr = np.asarray(sizes)
    if arr.ndim != 1:
        raise ValueError(f"the array to be partitioned must be 1-D, got shape {arr.shape}")
    if len(arr) < k * max(min_size, 1):
        raise ValueError(f"cannot split {len(arr)} items into {k} parts of at least {min_size}")
    parts = partition_balanced_tuples(arr.tolist(), k, min_size)
    assert parts[0][0] == 0 and parts[-1][1] == len(arr) and all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
    return parts


def reorder_to_balanced_batches(seqlens: Sequence[int], n_seqs_per_batch: int) -> tuple[np.ndarray, int]:
    """A permutation that groups sequences into consecutive batches of ``n_seqs_per_batch`` with token counts as
    equal as possible (longest first, each into the lightest batch that still has room), and the largest difference
    between two batches' token counts. Batches are returned heaviest first."""
    lens = np.asarray(seqlens, dtype=np.int64)
    n_bins = -(-len(lens) // n_seqs_per_batch)
    bins: list[list[int]] = [[] for _ in range(n_bins)]
    load = np.zeros(n_bins, dtype=np.int64)
    for i in np.argsort(-lens, kind="stable"):
        open_bins = [b for b in range(n_bins) if len(bins[b]) < n_seqs_per_batch]
        b = min(open_bins, key=lambda j: (load[j], j))
        bins[b].append(int(i))
        load[b] += lens[i]
    order = np.argsort(-load, kind="stable")
    perm = np.array([i for b in order for i in bins[b]], dtype=np.int64)
    return perm, int(load.max() - load.min()) if n_bins else 0


def flat2d(rows: Sequence[Sequence[Any]]) -> list[Any]:
    return [x for row in rows for x in row]
