"""Pipeline schedules (GPipe, 1F1B, interleaved 1F1B over virtual stages, zero-bubble with split backward): structure of the action lists,
host replay (no deadlock, bubble, live activations) and equivalence of an optimizer step on gloo ranks with
the single-process run. Reference: areal/experimental/models/archon/pipeline_parallel.py:48-82,349-494."""
import os
import subprocess
import sys

import pytest

from areal_b200.parallel.pipeline import build_schedule, canonical_schedule, min_micro_batches, simulate

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "torchrun", "run_model_parallel.py")


@pytest.mark.parametrize("name,P,M,V", [("GPipe", 4, 8, 1), ("1F1B", 2, 8, 1), ("1F1B", 4, 8, 1), ("1F1B", 4, 3, 1),
                                        ("Interleaved1F1B", 2, 8, 2), ("Interleaved1F1B", 4, 8, 2),
                                        ("Interleaved1F1B", 4, 16, 3), ("ZBVZeroBubble", 4, 8, 2),
                                        ("InterleavedZeroBubble", 2, 4, 2), ("ZB1P", 4, 8, 1), ("ZB1P", 8, 16, 1),
                                        ("ZB1P", 4, 3, 1)])
def test_every_rank_runs_each_forward_and_backward_once_in_a_valid_order(name, P, M, V):
    for r in range(P):
        acts = build_schedule(name, P, M, r, V)
        assert sorted(a for a in acts if a[0] == "F") == sorted(("F", m, c) for m in range(M) for c in range(V))
        assert sorted(a for a in acts if a[0] == "B") == sorted(("B", m, c) for m in range(M) for c in range(V))
        for m in range(M):
            for c in range(V):
                assert acts.index(("F", m, c)) < acts.index(("B", m, c))
                if canonical_schedule(name, V) == "zero_bubble":
                    assert acts.index(("B", m, c)) < acts.index(("W", m, c)) and acts.count(("W", m, c)) == 1
        if canonical_schedule(name, V) != "zero_bubble":
            assert not [a for a in acts if a[0] == "W"]
    res = simulate(name, P, M, V)  # raises on a deadlock
    assert res.makespan > 0


def test_1f1b_bounds_live_activations_and_interleaving_shrinks_the_bubble():
    P, M = 4, 8
    g, o = simulate("GPipe", P, M), simulate("1F1B", P, M)
    assert g.peak_live == [M] * P
    assert o.peak_live == [P - r for r in range(P)]            # at most P - rank micro-batches alive
    assert abs(o.makespan - g.makespan) < 1e-9                 # same bubble, (P - 1) / (M + P - 1) of the step
    assert abs(o.bubble_fraction - (P - 1) / (M + P - 1)) < 1e-9
    i2 = simulate("Interleaved1F1B", P, M, 2)
    assert abs(i2.bubble_fraction - ((P - 1) / 2) / (M + (P - 1) / 2)) < 1e-9   # bubble divided by V
    i4 = simulate("Interleaved1F1B", P, 16, 4)
    assert i4.bubble_fraction < simulate("1F1B", P, 16).bubble_fraction / 3


def test_zero_bubble_fills_idle_time_with_weight_gradients_at_the_memory_of_1f1b():
    for P, M, V, base in [(4, 8, 1, "1F1B"), (8, 32, 1, "1F1B"), (4, 8, 2, "Interleaved1F1B"), (2, 4, 2, "Interleaved1F1B")]:
        z, o = simulate("InterleavedZeroBubble", P, M, V), simulate(base, P, M, V)
        assert z.makespan < o.makespan and z.bubble_fraction < 0.75 * o.bubble_fraction
        assert abs(sum(z.busy) - sum(o.busy)) < 1e-9                    # same work, less waiting
        assert z.peak_live == o.peak_live                                # F-to-B activations: the 1F1B bound
        # same order of forwards and of input-gradient passes on every rank: messages on every link keep their order
        for r in range(P):
            za, oa = build_schedule("InterleavedZeroBubble", P, M, r, V), build_schedule(base, P, M, r, V)
            assert [a for a in za if a[0] == "F"] == [a for a in oa if a[0] == "F"]
            assert [a for a in za if a[0] == "B"] == [a for a in oa if a[0] == "B"]
    # memory: live activations plus half a set per parked micro-batch never exceed the 1F1B bound of the rank
    P, M = 4, 8
    for r in range(P):
        nf = nb = nw = 0
        for kind, _, _ in build_schedule("ZB1P", P, M, r):
            nf, nb, nw = nf + (kind == "F"), nb + (kind == "B"), nw + (kind == "W")
            assert (nf - nb) + 0.5 * (nb - nw) <= P - r


def test_v_shaped_placement_halves_the_bubble_at_balanced_memory():
    """ZBVZeroBubble: chunk 0 of rank p is stage p, chunk 1 stage 2P - 1 - p. Against the split schedule over the
    interleaved placement it waits about half as long, and no rank holds more than 2P live chunks (P stages' worth,
    what plain 1F1B holds on its first rank), where the interleaved placement piles ~3P on the first rank."""
    from areal_b200.parallel.pipeline import placement_of, rank_of, stage_of

    assert placement_of("ZBVZeroBubble") == "v" and placement_of("InterleavedZeroBubble") == "interleaved"
    assert [stage_of(r, c, 4, "v") for c in (0, 1) for r in range(4)] == [0, 1, 2, 3, 7, 6, 5, 4]
    assert [rank_of(s, 4, "v") for s in range(8)] == [0, 1, 2, 3, 3, 2, 1, 0]
    for P, M in [(2, 4), (4, 8), (4, 16), (8, 32)]:
        v, i = simulate("ZBVZeroBubble", P, M, 2), simulate("InterleavedZeroBubble", P, M, 2)
        assert v.bubble_fraction < 0.6 * i.bubble_fraction, (P, M, v.bubble_fraction, i.bubble_fraction)
        assert abs(sum(v.busy) - sum(i.busy)) < 1e-9
        assert max(v.peak_live) <= 2 * P < max(i.peak_live)
        for r in range(P):
            acts = build_schedule("ZBVZeroBubble", P, M, r, 2, placement="v")
            assert sorted(acts) == sorted((k, m, c) for k in "FBW" for m in range(M) for c in (0, 1))
            for kind in "FB":            # every stream of every link is in micro-batch order on both ends
                for c in (0, 1):
                    assert [a[1] for a in acts if a[0] == kind and a[2] == c] == list(range(M))
            live = parked = 0            # live activations plus half a set per parked product stay within 2P chunks
            for kind, _, _ in acts:
                live += (kind == "F") - (kind == "B")
                parked += (kind == "B") - (kind == "W")
                assert live + 0.5 * parked <= 2 * P + 0.5
    fwd = [build_schedule("ZBVZeroBubble", 4, 8, r, 2, forward_only=True, placement="v") for r in range(4)]
    assert all(sorted(a) == sorted(("F", m, c) for m in range(8) for c in (0, 1)) for a in fwd)
    with pytest.raises(ValueError, match="two chunks"):
        simulate("ZBVZeroBubble", 4, 8, 1)


def test_weight_gradient_products_can_be_parked_and_run_later():
    import torch

    from areal_b200.ops import wgrad_defer
    from areal_b200.ops.gemm import linear

    torch.manual_seed(0)
    x = torch.randn(5, 7, 16, requires_grad=True)
    w1, b1 = torch.randn(32, 16, requires_grad=True), torch.randn(32, requires_grad=True)
    w2 = torch.randn(8, 32, requires_grad=True)
    ref = torch.nn.functional.linear(torch.nn.functional.linear(x, w1, b1).relu(), w2).square().sum()
    gx, g1, gb, g2 = torch.autograd.grad(ref, [x, w1, b1, w2])
    wgrad_defer.arm(True)
    try:
        out = linear(linear(x, w1, b1).relu(), w2).square().sum()
        q = wgrad_defer.WgradQueue()
        with q.collect():
            out.backward()
        assert torch.allclose(x.grad, gx, atol=1e-5) and torch.allclose(b1.grad, gb, atol=1e-5)
        assert w1.grad is None and w2.grad is None and len(q) == 2      # parked, not computed
        assert wgrad_defer.active() is None
        assert q.run() == 2 and len(q) == 0
        assert torch.allclose(w1.grad, g1, atol=1e-4) and torch.allclose(w2.grad, g2, atol=1e-4)
        # a second micro-batch accumulates; with a main_grad the product lands there in fp32
        w2.main_grad = torch.zeros_like(w2)
        out = linear(linear(x, w1, b1).relu(), w2).square().sum()
        with q.collect():
            out.backward()
        q.run()
        assert torch.allclose(w1.grad, 2 * g1, atol=2e-4) and torch.allclose(w2.main_grad, g2, atol=1e-4)
        # without an active queue the same function computes both halves at once
        w1.grad = None
        linear(x, w1, b1).sum().backward()
        assert w1.grad is not None
    finally:
        wgrad_defer.arm(False)
    assert type(linear(x, w1, None).grad_fn).__name__ != "SplitLinearBackward"


def test_names_and_limits():
    assert canonical_schedule("Interleaved1F1B", 1) == "1f1b" and canonical_schedule("interleaved_1f1b", 2) == "interleaved_1f1b"
    assert min_micro_batches("1F1B", 4) == 8 and min_micro_batches("GPipe", 4) == 4
    with pytest.raises(ValueError):
        canonical_schedule("1F1B", 2)
    with pytest.raises(ValueError):
        build_schedule("Interleaved1F1B", 4, 6, 0, 2)
    with pytest.raises(ValueError):
        canonical_schedule("looped", 1)


def _free_port():
    import socket

    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def _ref(tmp_path, n_mbs):
    f = str(tmp_path / "ref.pt")
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    r = subprocess.run([sys.executable, WORKER, "--ref", "--n-mbs", str(n_mbs), "--preset", "tiny-qwen2-4l", f],
                       env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    return f


@pytest.mark.parametrize("n,flags", [(2, ["--pp", "2", "--schedule", "1F1B"]),
                                     (2, ["--pp", "2", "--schedule", "GPipe"]),
                                     (2, ["--pp", "2", "--vpp", "2", "--schedule", "Interleaved1F1B"]),
                                     (4, ["--pp", "4", "--schedule", "1F1B"]),
                                     (2, ["--pp", "2", "--schedule", "ZB1P"]),
                                     (4, ["--pp", "4", "--schedule", "ZB1P"]),
                                     (2, ["--pp", "2", "--schedule", "ZBVZeroBubble"]),
                                     (3, ["--pp", "3", "--schedule", "ZBVZeroBubble"]),
                                     (4, ["--pp", "2", "--tp", "2", "--schedule", "ZBVZeroBubble"]),
                                     (2, ["--pp", "2", "--vpp", "2", "--schedule", "InterleavedZeroBubble"]),
                                     (4, ["--pp", "2", "--tp", "2", "--vpp", "2"])])
def test_step_with_eight_micro_batches_matches_single_process(tmp_path, n, flags):
    """Loss, gradient norm and every gradient of one optimizer step over 8 micro-batches."""
    ref = _ref(tmp_path, 8)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), WORKER,
           "--n-mbs", "8", "--preset", "tiny-qwen2-4l"] + flags + [ref]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


def test_v_shaped_placement_with_expert_parallelism_matches_single_process(tmp_path):
    """ZBVZeroBubble over two pipeline ranks whose stages spread their experts over two expert-parallel ranks (a
    four-block MoE model: one block per stage): the experts' own flat buffer, optimizer and gradient norm follow the
    V-shaped layer assignment."""
    ref = str(tmp_path / "ref.pt")
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    common = ["--n-mbs", "4", "--layers", "4", "--preset", "tiny-qwen3-moe"]
    r = subprocess.run([sys.executable, WORKER, "--ref"] + common + [ref], env=env, capture_output=True, text=True,
                       timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), WORKER] + common + \
          ["--pp", "2", "--ep", "2", "--schedule", "ZBVZeroBubble", ref]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
