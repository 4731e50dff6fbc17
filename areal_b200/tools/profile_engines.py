"""Micro-profiler of the train engine: runs forward-only and train steps on synthetic packed batches of
a chosen model shape and reports step time, tokens/s, model FLOP/s, peak memory, the number of this
library's kernel launches, and (``--top N``) the most expensive device ops seen by ``torch.profiler``.
Numbers printed here are diagnostics; benchmark numbers come from ``bench.py`` (CUDA events, no profiler).

    python -m areal_b200.tools.profile_engines --preset qwen3-1.7b --tokens 16384 --seq-len 2048 --steps 3
    python -m areal_b200.tools.profile_engines --preset tiny-qwen2 --device cpu --tokens 512 --seq-len 64

Counterpart of areal/tools/profile_engines.py / profile_fsdp.py / profile_archon.py (one engine here).
"""

from __future__ import annotations

import argparse
import json
import time


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--preset", default="qwen3-1.7b")
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (0 = preset)")
    ap.add_argument("--tokens", type=int, default=16384, help="tokens per step (one micro-batch)")
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--device", default=None, choices=[None, "cpu", "cuda"])
    ap.add_argument("--top", type=int, default=0, help="profile one extra step with torch.profiler and list N ops")
    ap.add_argument("--trace", default=None, help="write that step's Chrome trace here")
    args = ap.parse_args(argv)

    import torch

    from ..api.cli_args import MicroBatchSpec, OptimizerConfig, TrainEngineConfig
    from ..engine.train_engine import B200TrainEngine
    from ..ops import _lib

    cuda = torch.cuda.is_available() if args.device is None else args.device == "cuda"
    over = {"num_hidden_layers": args.layers} if args.layers else {}
    cfg = TrainEngineConfig(backend="fsdp:d1", model_preset=args.preset, model_overrides=over, init_from_scratch=True,
                            dtype="bfloat16" if cuda else "float32_cpu",
                            optimizer=OptimizerConfig(lr=1e-6, warmup_steps_proportion=0.0),
                            mb_spec=MicroBatchSpec(max_tokens_per_mb=args.tokens))
    eng = B200TrainEngine(cfg)
    eng.create_process_group()
    eng.initialize(None, None)
    mc = eng.model_config
    n_seq = max(args.tokens // args.seq_len, 1)
    g = torch.Generator().manual_seed(0)
    batch = dict(input_ids=torch.randint(0, mc.vocab_size, (n_seq, args.seq_len), generator=g),
                 attention_mask=torch.ones(n_seq, args.seq_len, dtype=torch.bool),
                 loss_mask=torch.ones(n_seq, args.seq_len, dtype=torch.long))

    def loss_fn(logp, ent, mb):
        m = mb["loss_mask"].float()
        return -(logp * m).sum() / m.sum()

    def weight_fn(mb):
        return mb["loss_mask"].float().sum()

    def sync():
        if cuda:
            torch.cuda.synchronize()

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        sync()
        _lib.reset_launch_count()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            fn()
        sync()
        return (time.perf_counter() - t0) / args.steps, _lib.launch_count() // max(args.steps, 1)

    tokens = n_seq * args.seq_len
    report = {"preset": args.preset, "tokens_per_step": tokens, "seq_len": args.seq_len, "device": "cuda" if cuda else "cpu",
              "params_b": mc.num_params() / 1e9}
    for name, fn, bwd in (("forward", lambda: eng.forward_batch(batch), False),
                          ("train", lambda: eng.train_batch(batch, loss_fn, weight_fn), True)):
        if cuda:
            torch.cuda.reset_peak_memory_stats()
        s, launches = timed(fn)
        flops = mc.flops_per_token(args.seq_len, backward=bwd) * tokens
        report[name] = {"ms_per_step": s * 1e3, "tokens_per_s": tokens / s, "model_tflops": flops / s / 1e12,
                        "kernel_launches_per_step": launches,
                        "peak_mem_gb": torch.cuda.max_memory_allocated() / 2**30 if cuda else None}
    print(json.dumps(report, indent=2))
    if args.top:
        from torch.profiler import ProfilerActivity, profile

        acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if cuda else [])
        with profile(activities=acts) as prof:
            eng.train_batch(batch, loss_fn, weight_fn)
            sync()
        key = "cuda_time_total" if cuda else "cpu_time_total"
        print(prof.key_averages().table(sort_by=key, row_limit=args.top))
        if args.trace:
            prof.export_chrome_trace(args.trace)
    eng.destroy()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
