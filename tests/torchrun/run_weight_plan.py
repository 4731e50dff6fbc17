"""Worker: the trainer -> rollout re-sharding plan on gloo ranks. Every rank builds its model-parallel
engine, applies ITS share of the plan to a zeroed copy of the rollout engine's flat buffer, and the sum over
all ranks must equal the single-process model's buffer: every element written exactly once."""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from areal_b200.api.alloc_mode import ParallelStrategy  # noqa: E402
from areal_b200.api.cli_args import OptimizerConfig, TrainEngineConfig  # noqa: E402
from areal_b200.engine.flat_params import FlatParams  # noqa: E402
from areal_b200.engine.train_engine import B200TrainEngine  # noqa: E402
from areal_b200.infra.weight_plan import _pieces, apply_plan_torch, build_plan, rollout_layout  # noqa: E402
from areal_b200.models.config import PRESETS  # noqa: E402
from areal_b200.models.qwen import build_model  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--ep", type=int, default=1)
    ap.add_argument("--etp", type=int, default=1)
    ap.add_argument("--vpp", type=int, default=1)
    ap.add_argument("--preset", default="tiny-qwen2-4l")
    args = ap.parse_args()
    dist.init_process_group("gloo")
    world = dist.get_world_size()
    cfg = TrainEngineConfig(experiment_name="t", trial_name="t", path="", init_from_scratch=True, dtype="float32",
                            model_preset=args.preset, optimizer=OptimizerConfig(lr=1e-3))
    cfg.megatron.virtual_pipeline_parallel_size = args.vpp
    eng = B200TrainEngine(cfg)
    dp = world // (args.tp * args.pp)
    eng.create_process_group(ParallelStrategy(tensor_parallel_size=args.tp, pipeline_parallel_size=args.pp,
                                              data_parallel_size=dp, expert_parallel_size=args.ep,
                                              expert_tensor_parallel_size=args.etp))
    eng.initialize(seed=3)
    # what the rollout engine holds: the whole model in one flat buffer
    full = build_model(PRESETS[args.preset], dtype=torch.float32, device="cpu", seed=3)
    ref = FlatParams(full, "local", with_grads=False)
    layout = rollout_layout(ref)
    plans = build_plan(eng, layout)
    dst = torch.zeros_like(ref.flat)
    apply_plan_torch(plans, dst)
    for f, segs in plans.values():
        _pieces(segs, 2)  # bf16 buffers: every segment is 16-byte aligned
    n_local = sum(len(s) for _, s in plans.values())
    dist.all_reduce(dst)
    err = (dst - ref.flat).abs().max().item()
    assert err == 0.0, err
    cnt = torch.tensor([n_local])
    dist.all_reduce(cnt)
    if dist.get_rank() == 0:
        print("OK", int(cnt), "segments")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
