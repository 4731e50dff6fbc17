"""Worker: aux-loss-free balancing under data parallelism. Every rank routes its own tokens; after one optimizer
step the selection biases must be the same on all ranks and equal the update computed from the SUM of the ranks'
token counts. Launched by tests/test_qwen3_5.py through torchrun (gloo, CPU)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from areal_b200.api.alloc_mode import ParallelStrategy  # noqa: E402
from areal_b200.api.cli_args import OptimizerConfig, TrainEngineConfig  # noqa: E402
from areal_b200.engine.train_engine import B200TrainEngine  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    eng = B200TrainEngine(TrainEngineConfig(experiment_name="t", trial_name="t", path="", init_from_scratch=True,
                                            dtype="float32", model_preset="tiny-qwen3-moe",
                                            model_overrides={"moe_load_balance_coeff": 0.02},
                                            optimizer=OptimizerConfig(lr=1e-3, warmup_steps_proportion=0.0)))
    eng.create_process_group(ParallelStrategy(data_parallel_size=world))
    eng.initialize(seed=1)
    mlps = [l.mlp for l in eng.model.layers]
    counted = []
    for m in mlps:  # record what each rank counted before the hook sums and clears it
        orig = m.update_expert_bias

        def wrapped(groups=(), m=m, orig=orig):
            counted.append(m.load_acc.clone())
            return orig(groups)

        m.update_expert_bias = wrapped
    g = torch.Generator().manual_seed(100 + rank)   # different tokens on every rank
    ids = torch.randint(0, 1024, (4, 40), generator=g)
    batch = dict(input_ids=ids, attention_mask=torch.ones_like(ids), loss_mask=torch.ones_like(ids))
    eng.train_batch(batch, lambda lp, ent, mb: -(lp * mb["loss_mask"].float()).sum() / mb["loss_mask"].sum(),
                    lambda mb: float(mb["loss_mask"].sum()))
    for m, mine in zip(mlps, counted):
        total = mine.clone()
        dist.all_reduce(total)
        assert float(total.sum()) == world * 4 * 40 * eng.model_config.num_experts_per_tok
        assert not torch.equal(total, mine * world), "the ranks were meant to route different tokens"
        want = 0.02 * torch.sign(total.mean() - total)
        assert torch.allclose(m.expert_bias, want), (m.expert_bias, want)
        both = [torch.empty_like(m.expert_bias) for _ in range(world)]
        dist.all_gather(both, m.expert_bias)
        assert all(torch.equal(b, both[0]) for b in both)
    dist.barrier()
    if rank == 0:
        print("OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
