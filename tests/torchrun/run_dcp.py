"""Worker of the torch-DCP checkpoint tests (gloo, CPU).

    run_dcp.py --phase train  --dir D [--tp 2 ...]   # 2 steps, save D/ckpt (with optimizer), 1 more step, save D/after
    run_dcp.py --phase resume --dir D [--tp 1 ...]   # load D/ckpt, save D/reload at once, 1 step, save D/resumed

The batch of every step is a function of the step number only and is dealt out by data-parallel rank, so
any layout optimises the same objective. Launch under torchrun for more than one rank.
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from areal_b200.api.alloc_mode import ParallelStrategy  # noqa: E402
from areal_b200.api.cli_args import MicroBatchSpec, OptimizerConfig, TrainEngineConfig  # noqa: E402
from areal_b200.api.io_struct import FinetuneSpec, SaveLoadMeta  # noqa: E402
from areal_b200.engine.train_engine import B200TrainEngine  # noqa: E402


def batch_of(step: int, n_seq=8, L=40, vocab=1024):
    g = torch.Generator().manual_seed(100 + step)
    lens = torch.randint(L // 3, L + 1, (n_seq,), generator=g)
    ids = torch.randint(0, vocab, (n_seq, L), generator=g)
    mask = torch.arange(L)[None, :] < lens[:, None]
    return dict(input_ids=ids * mask, attention_mask=mask, loss_mask=(mask & (torch.arange(L)[None, :] >= 2)).int())


def loss_fn(logp, ent, mb):
    m = torch.roll(mb["loss_mask"], shifts=-1, dims=0).float()
    return -(logp * m).sum() / m.sum().clamp(min=1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--phase", choices=["train", "resume"], required=True)
    ap.add_argument("--dir", required=True)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--sp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--ep", type=int, default=1)
    ap.add_argument("--etp", type=int, default=1)
    ap.add_argument("--lora", action="store_true")
    ap.add_argument("--preset", default="tiny-qwen2")
    ap.add_argument("--n-mbs", type=int, default=1)
    ap.add_argument("--async-save", action="store_true")
    ap.add_argument("--format", default="dcp", choices=["dcp", "hf"])
    args = ap.parse_args()
    cfg = TrainEngineConfig(experiment_name="t", trial_name="t", path="", init_from_scratch=True, dtype="float32",
                            model_preset=args.preset, mb_spec=MicroBatchSpec(n_mbs=args.n_mbs),
                            optimizer=OptimizerConfig(lr=2e-3, weight_decay=0.01, gradient_clipping=1.0,
                                                      warmup_steps_proportion=0.5, lr_scheduler_type="cosine"))
    if args.lora:
        cfg.use_lora, cfg.lora_rank, cfg.lora_alpha, cfg.target_modules = True, 4, 8, ["q_proj", "v_proj", "down_proj"]
    eng = B200TrainEngine(cfg)
    multi = "RANK" in os.environ
    if multi:
        dist.init_process_group("gloo")
        world = dist.get_world_size()
        dp = world // (args.tp * args.sp * args.pp)
        eng.create_process_group(ParallelStrategy(tensor_parallel_size=args.tp, context_parallel_size=args.sp,
                                                  pipeline_parallel_size=args.pp, data_parallel_size=dp,
                                                  expert_parallel_size=args.ep,
                                                  expert_tensor_parallel_size=args.etp))
    else:
        dp = 1
        eng.create_process_group()
    # the schedule is 6 steps long: steps 0-2 are warm-up, so a frozen scheduler would show
    eng.initialize(None, FinetuneSpec(1, 6 * 8, 8), seed=3 if args.phase == "train" else 11)
    d = eng.data_parallel_rank

    def step(i):
        b = batch_of(i)
        st = eng.train_batch({k: v[d::dp] for k, v in b.items()}, loss_fn, lambda mb: float(mb["loss_mask"].sum()))
        assert st["update_successful"] == 1.0
        return st

    def save(name, with_optim, async_save=False):
        eng.save(SaveLoadMeta(path=os.path.join(args.dir, name), weight_format=args.format, with_optim=with_optim,
                              async_save=async_save))

    if args.phase == "train":
        step(0)
        step(1)
        save("ckpt", True, args.async_save)
        st = step(2)  # with an asynchronous save this step overlaps the write: the staged copy must be used
        eng.wait_for_checkpoint()
        save("after", True)
    else:
        eng.load(SaveLoadMeta(path=os.path.join(args.dir, "ckpt"), weight_format=args.format, with_optim=True))
        assert eng.optimizer.step_count == 2 and eng.optimizer.sched_step == 2, \
            (eng.optimizer.step_count, eng.optimizer.sched_step)
        if eng.optimizer.partner is not None:
            assert eng.optimizer.partner.sched_step == 2 and eng.optimizer.partner.step_count == 2
        save("reload", True)
        st = step(2)
        save("resumed", True)
    if multi:
        # a rank's loss is the sum over its own micro-batches: add up the data-parallel ranks' shares
        t = torch.tensor([st["loss"]], dtype=torch.float64)
        if dp > 1:
            dist.all_reduce(t, group=eng.data_parallel_group)
        st["loss"] = float(t)
        dist.barrier()
    if not multi or dist.get_rank() == 0:
        print("OK", st["loss"], st["grad_norm"], st["lr"])
    if multi:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
