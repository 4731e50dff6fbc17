"""Native partitioners against their pure-Python restatements and invariants."""
import random

import pytest

from areal_b200.utils import seqpack


@pytest.mark.parametrize("seed", range(5))
def test_ffd_respects_capacity_and_matches_python(seed):
    rnd = random.Random(seed)
    sizes = [rnd.randint(1, 500) for _ in range(rnd.randint(1, 200))]
    cap = 1000
    groups = seqpack.ffd_allocate(sizes, cap, min_groups=3)
    assert sorted(i for g in groups for i in g) == list(range(len(sizes)))
    assert all(sum(sizes[i] for i in g) <= cap for g in groups)
    bins, nb = seqpack._ffd_py(sizes, cap, 3)
    ref = [[] for _ in range(nb)]
    for i, b in enumerate(bins):
        ref[b].append(i)
    assert [g for g in ref if g] == groups


def test_ffd_oversized_item_raises():
    with pytest.raises(ValueError):
        seqpack.ffd_allocate([5, 2000], 1000, 1)


@pytest.mark.parametrize("seed", range(5))
@pytest.mark.parametrize("equal", [False, True])
def test_kk_balances_and_matches_python(seed, equal):
    rnd = random.Random(seed)
    sizes = [rnd.randint(1, 1000) for _ in range(64)]
    k = 4
    groups = seqpack.kk_allocate(sizes, k, equal_size=equal)
    assert sorted(i for g in groups for i in g) == list(range(64))
    sums = sorted(sum(sizes[i] for i in g) for g in groups)
    ref = sorted(sum(sizes[i] for i in g) for g in seqpack._kk_py(sizes, k, equal))
    assert sums == ref
    assert sums[-1] - sums[0] <= max(sizes)
    if equal:
        assert all(len(g) == 16 for g in groups)
    # KK is at least as balanced as a naive contiguous split
    naive = [sum(sizes[i::k]) for i in range(k)]
    assert sums[-1] - sums[0] <= max(naive) - min(naive) + max(sizes)


def test_partition_balanced_optimal_small():
    sizes = [3, 1, 4, 1, 5, 9, 2, 6]
    b = seqpack.partition_balanced(sizes, 3)
    assert b[0] == 0 and b[-1] == len(sizes) and len(b) == 4
    best = min(max(sum(sizes[:i]), sum(sizes[i:j]), sum(sizes[j:]))
               for i in range(1, 7) for j in range(i + 1, 8))
    got = max(sum(sizes[b[i]:b[i + 1]]) for i in range(3))
    assert got == best
    with pytest.raises(ValueError):
        seqpack.partition_balanced([1, 2], 3)


def test_greedy_partition_equal_cardinality():
    sizes = list(range(1, 21))
    groups = seqpack.balanced_greedy_partition(sizes, 4, equal_size=True)
    assert all(len(g) == 5 for g in groups)
    sums = [sum(sizes[i] for i in g) for g in groups]
    assert max(sums) - min(sums) <= 8


def test_allocate_divisor_and_min_groups():
    sizes = [100] * 10
    groups = seqpack.allocate(sizes, 250, min_groups=3, algorithm="ffd", divisor=2)
    assert len(groups) % 2 == 0 and len(groups) >= 5
    groups = seqpack.allocate(sizes, None, min_groups=4, algorithm="kk")
    assert len(groups) == 4


def test_pipeline_layer_partition_minimises_the_slowest_stage():
    import itertools

    from areal_b200.parallel.context import partition_layers

    def cost(ranges, costs, fe, le):
        return max(sum(costs[a:b]) + (fe if i == 0 else 0) + (le if i == len(ranges) - 1 else 0)
                   for i, (a, b) in enumerate(ranges))

    for costs, k, fe, le in [([1.0] * 28, 4, 0.0, 6.2), ([1, 1, 4, 1, 1, 1], 3, 0.0, 0.0), ([1.0] * 7, 3, 0.5, 2.0),
                             ([1.0] * 2, 2, 0.0, 0.4)]:
        got = partition_layers(costs, k, fe, le)
        assert got[0][0] == 0 and got[-1][1] == len(costs) and all(a < b for a, b in got)
        assert all(got[i][1] == got[i + 1][0] for i in range(k - 1))
        best = min(cost(list(zip((0,) + cuts, cuts + (len(costs),))), costs, fe, le)
                   for cuts in itertools.combinations(range(1, len(costs)), k - 1))
        assert abs(cost(got, costs, fe, le) - best) < 1e-9
    with pytest.raises(ValueError):
        partition_layers([1.0, 1.0], 3)
