"""Worker: a tensor-parallel vision-language model exports the same HF tensors as one process (decoder shards
gathered, the replicated tower written once) and loads them back into its shards. Launched by
tests/test_model_parallel_cpu.py through torchrun (gloo, CPU)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from areal_b200.api.alloc_mode import ParallelStrategy  # noqa: E402
from areal_b200.api.cli_args import OptimizerConfig, TrainEngineConfig  # noqa: E402
from areal_b200.engine.train_engine import B200TrainEngine  # noqa: E402
from areal_b200.models.config import PRESETS  # noqa: E402
from areal_b200.models.qwen import build_model  # noqa: E402


def main(preset: str):
    dist.init_process_group("gloo")
    cfg = TrainEngineConfig(experiment_name="t", trial_name="t", path="", init_from_scratch=True, dtype="float32",
                            model_preset=preset, optimizer=OptimizerConfig(lr=1e-3))
    eng = B200TrainEngine(cfg)
    eng.create_process_group(ParallelStrategy(tensor_parallel_size=dist.get_world_size(), data_parallel_size=1))
    eng.initialize(seed=3)
    got = {n: t.clone() for n, t in eng.model.to_hf()}
    want = dict(build_model(PRESETS[preset], dtype=torch.float32, seed=3).to_hf())
    assert set(got) == set(want), sorted(set(got) ^ set(want))[:6]
    for n, t in want.items():
        assert torch.equal(got[n], t), n
    other = build_model(PRESETS[preset], dtype=torch.float32, seed=9, pctx=eng.pctx)
    other.load_hf(want.items())
    for (n1, p1), (_, p2) in zip(eng.model.named_parameters(), other.named_parameters()):
        assert torch.equal(p1, p2), n1
    dist.barrier()
    if dist.get_rank() == 0:
        print("OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1])
