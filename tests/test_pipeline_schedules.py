"""Pipeline schedules (GPipe, 1F1B, interleaved 1F1B over virtual stages): structure of the action lists,
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
                                        ("Interleaved1F1B", 4, 16, 3), ("ZBVZeroBubble", 4, 8, 2)])
def test_every_rank_runs_each_forward_and_backward_once_in_a_valid_order(name, P, M, V):
    for r in range(P):
        acts = build_schedule(name, P, M, r, V)
        assert sorted(a for a in acts if a[0] == "F") == sorted(("F", m, c) for m in range(M) for c in range(V))
        assert sorted(a for a in acts if a[0] == "B") == sorted(("B", m, c) for m in range(M) for c in range(V))
        for m in range(M):
            for c in range(V):
                assert acts.index(("F", m, c)) < acts.index(("B", m, c))
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


def test_names_and_limits():
    assert canonical_schedule("Interleaved1F1B", 1) == "1f1b" and canonical_schedule("interleaved_1f1b", 2) == "interleaved_1f1b"
    assert min_micro_batches("1F1B", 4) == 8 and min_micro_batches("GPipe", 4) == 4
    with pytest.raises(ValueError):
        canonical_schedule("1F1B", 2)
    with pytest.raises(ValueError):
        build_schedule("Interleaved1F1B", 4, 6, 0, 2)
    with pytest.raises(ValueError):
        canonical_schedule("looped", 1)


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
                                     (4, ["--pp", "2", "--tp", "2", "--vpp", "2"])])
def test_step_with_eight_micro_batches_matches_single_process(tmp_path, n, flags):
    """Loss, gradient norm and every gradient of one optimizer step over 8 micro-batches."""
    ref = _ref(tmp_path, 8)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(29750 + 7 * n + len(flags) + len("".join(flags)) % 5), WORKER,
           "--n-mbs", "8", "--preset", "tiny-qwen2-4l"] + flags + [ref]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
