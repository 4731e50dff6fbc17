"""Worker: a tensor-parallel vision-language model exports the same HF tensors as one process (decoder shards
gathered, the replicated tower written once) and loads them back into its shards; with pipeline stages the
engine's checkpoint (a file set per stage plus an index) loads into a single-process model. Launched by
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


def main(preset: str, pp: int = 1, out: str = "", ep: int = 1, tp: int = 0, etp: int = 1):
    dist.init_process_group("gloo")
    cfg = TrainEngineConfig(experiment_name="t", trial_name="t", path="", init_from_scratch=True, dtype="float32",
                            model_preset=preset, optimizer=OptimizerConfig(lr=1e-3))
    eng = B200TrainEngine(cfg)
    if ep * etp > 1 and tp > 1:  # hybrid: attention tensor-parallel, experts spread / split over the same ranks
        world = dist.get_world_size()
        eng.create_process_group(ParallelStrategy(tensor_parallel_size=tp, pipeline_parallel_size=pp,
                                                  data_parallel_size=world // (tp * pp), expert_parallel_size=ep,
                                                  expert_tensor_parallel_size=etp))
    elif ep > 1:  # expert parallelism lives inside the data-parallel ranks
        eng.create_process_group(ParallelStrategy(data_parallel_size=dist.get_world_size(), expert_parallel_size=ep))
    else:
        eng.create_process_group(ParallelStrategy(tensor_parallel_size=dist.get_world_size() // pp,
                                                  pipeline_parallel_size=pp, data_parallel_size=1))
    eng.initialize(seed=3)
    ref = build_model(PRESETS[preset], dtype=torch.float32, seed=3)
    want = dict(ref.to_hf())
    if pp == 1 and ep == 1:
        got = {n: t.clone() for n, t in eng.model.to_hf()}
        assert set(got) == set(want), sorted(set(got) ^ set(want))[:6]
        for n, t in want.items():
            assert torch.equal(got[n], t), n
        other = build_model(PRESETS[preset], dtype=torch.float32, seed=9, pctx=eng.pctx)
        other.load_hf(want.items())
        for (n1, p1), (_, p2) in zip(eng.model.named_parameters(), other.named_parameters()):
            assert torch.equal(p1, p2), n1
    if out:
        # the engine's checkpoint (one file set per pipeline stage + an index) loads into a single-process model
        from areal_b200.api.io_struct import SaveLoadMeta
        from areal_b200.utils.hf_io import load_hf_weights

        eng.save(SaveLoadMeta(path=out, weight_format="hf", with_optim=False))
        dist.barrier()
        if dist.get_rank() == 0:
            import json

            loaded = load_hf_weights(build_model(PRESETS[preset], dtype=torch.float32, seed=9), out)
            for (n1, p1), (_, p2) in zip(ref.named_parameters(), loaded.named_parameters()):
                assert torch.equal(p1, p2), n1
            if (pp > 1 or ep > 1) and etp == 1:
                idx = json.load(open(os.path.join(out, "model.safetensors.index.json")))["weight_map"]
                assert set(idx) == set(want) and len(set(idx.values())) == pp * ep
        if ep * etp > 1:
            # and back into an expert-parallel model: every rank picks its own experts out of the directory
            other = build_model(PRESETS[preset], dtype=torch.float32, seed=9, pctx=eng.pctx)
            load_hf_weights(other, out)
            for (n1, p1), (_, p2) in zip(eng.model.named_parameters(), other.named_parameters()):
                assert torch.equal(p1, p2), n1
    dist.barrier()
    if dist.get_rank() == 0:
        print("OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1], int(sys.argv[2]) if len(sys.argv) > 2 else 1, sys.argv[3] if len(sys.argv) > 3 else "",
         int(sys.argv[4]) if len(sys.argv) > 4 else 1, int(sys.argv[5]) if len(sys.argv) > 5 else 0,
         int(sys.argv[6]) if len(sys.argv) > 6 else 1)
