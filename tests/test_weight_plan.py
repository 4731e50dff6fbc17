"""Re-sharding plan of the trainer -> rollout weight push (``infra/weight_plan.py``): tensor-, pipeline- and
expert-parallel trainers, with data-parallel replicas sharing the work, rebuild the rollout engine's flat
buffer exactly. Counterpart of the reference's gather-and-broadcast update (areal/engine/fsdp_engine.py:
1507-1597) and of its shard-to-shard plans (areal/experimental/weight_update/awex/fsdp_adapter.py:118-170)."""
import os
import subprocess
import sys

import pytest
import torch

from tests.conftest import free_port

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "torchrun", "run_weight_plan.py")


@pytest.mark.parametrize("n,flags", [(2, ["--tp", "2"]), (4, ["--tp", "2"]), (2, ["--pp", "2"]),
                                     (2, ["--pp", "2", "--vpp", "2"]), (2, ["--ep", "2", "--preset", "tiny-qwen3-moe"]),
                                     (4, ["--tp", "2", "--pp", "2"]),
                                     (2, ["--tp", "2", "--ep", "2", "--preset", "tiny-qwen3-moe"]),
                                     (4, ["--tp", "2", "--ep", "4", "--preset", "tiny-qwen3-moe"]),
                                     (2, ["--tp", "2", "--etp", "2", "--preset", "tiny-qwen3-moe"]),
                                     (4, ["--tp", "2", "--ep", "2", "--etp", "2", "--preset", "tiny-qwen3-moe"]),
                                     (2, ["--tp", "2", "--ep", "2", "--preset", "tiny-deepseek-v3"]),
                                     (2, ["--pp", "2", "--preset", "tiny-bailing-hybrid"])])
def test_plan_rebuilds_the_full_model_exactly_once(n, flags):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()), WORKER] + flags
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


def test_pieces_cut_large_segments_and_keep_strides():
    from areal_b200.infra.weight_plan import PIECE_VECS, Segment, _pieces

    big = Segment(src=64, dst=128, rows=1, row=8 * (PIECE_VECS * 2 + 5), src_pitch=0, dst_pitch=0)
    recs = _pieces([big], 2)
    assert recs.shape == (3, 5) and int(recs[:, 4].bitwise_and(0xFFFFFFFF).max()) == 1
    assert int((recs[:, 4] >> 32).sum()) == PIECE_VECS * 2 + 5 and int(recs[0, 0]) == 8 and int(recs[0, 1]) == 16
    strided = Segment(src=0, dst=1024, rows=3000, row=1024, src_pitch=1024, dst_pitch=4096)
    recs = _pieces([strided], 2)
    assert int(recs[:, 4].bitwise_and(0xFFFFFFFF).sum()) == 3000 and (recs[:, 2] == 128).all() and (recs[:, 3] == 512).all()
    with pytest.raises(ValueError):
        _pieces([Segment(src=3, dst=0, rows=1, row=8, src_pitch=8, dst_pitch=8)], 2)


@pytest.mark.gpu
def test_push_plan_kernel_matches_the_torch_statement():
    """The kernel against ``apply_plan_torch`` on one GPU (two destination buffers)."""
    import ctypes

    from areal_b200.infra.weight_plan import Segment, _pieces
    from areal_b200.ops import _lib

    torch.manual_seed(0)
    src = torch.randn(1 << 20, device="cuda").bfloat16()
    # destination ranges do not overlap: [8, 524808) strided, [1000000, 1560000) and [1600000, 1665536) contiguous
    segs = [Segment(0, 1000000, 1, 70000 * 8, 0, 0), Segment(700000, 8, 257, 512, 512, 2048),
            Segment(900000, 1600000, 64, 1024, 1024, 1024)]
    dsts = [torch.zeros(1 << 21, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    want = torch.zeros(1 << 21, device="cuda", dtype=torch.bfloat16)
    for g in segs:
        for r in range(g.rows):
            sp, dp = g.src_pitch or g.row, g.dst_pitch or g.row
            want[g.dst + r * dp: g.dst + r * dp + g.row] = src[g.src + r * sp: g.src + r * sp + g.row]
    recs = _pieces([Segment(g.src, g.dst, g.rows, g.row, g.src_pitch or g.row, g.dst_pitch or g.row) for g in segs], 2).cuda()
    table = (ctypes.c_void_p * 2)(dsts[0].data_ptr(), dsts[1].data_ptr())
    assert _lib.use_cuda_kernels(src)
    rc = _lib.kernels().b200_push_plan(table, ctypes.c_int(2), _lib.ptr(src), _lib.ptr(recs), ctypes.c_int(recs.shape[0]),
                                       _lib.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(dsts[0], want) and torch.equal(dsts[1], want)


def test_rollout_ranks_pair_with_data_parallel_heads_only():
    """Disaggregated layout with a model-parallel trainer: rollout ranks send batches to (and take control
    messages from) the first rank of each trainer replica; the other ranks of a replica get the batch from
    their head and have no rollout partner."""
    from areal_b200.infra.dist_rollout import DisaggTopology

    def topo(n_gen, n_train, replica, n_replicas):
        t = object.__new__(DisaggTopology)
        t.n_gen, t.n_train = n_gen, n_train
        t.gen_ranks = list(range(n_gen))
        t.train_ranks = list(range(n_gen, n_gen + n_train))
        t.train_heads = [t.train_ranks[d * replica] for d in range(n_replicas)]
        return t

    t = topo(2, 2, 2, 1)  # native:d2 + megatron:d1t2
    assert t.train_heads == [2] and t.trainers_of(0) == [2] and t.trainers_of(1) == [2]
    assert t.rollouts_of(2) == [0, 1] and t.rollouts_of(3) == []
    t = topo(4, 4, 2, 2)  # native:d4 + megatron:d2t2
    assert t.train_heads == [4, 6]
    assert [t.trainers_of(g) for g in range(4)] == [[4], [6], [4], [6]]
    assert t.rollouts_of(4) == [0, 2] and t.rollouts_of(5) == [] and t.rollouts_of(6) == [1, 3]
    t = topo(4, 4, 1, 4)  # native:d4 + fsdp:d4: one to one
    assert [t.trainers_of(g) for g in range(4)] == [[4], [5], [6], [7]]
    t = topo(2, 4, 1, 4)  # more trainers than rollout ranks: a rollout rank feeds two of them
    assert t.trainers_of(0) == [2, 4] and t.trainers_of(1) == [3, 5]
