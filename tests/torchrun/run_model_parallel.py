"""Worker: one train_batch of a tiny model under tensor / Ulysses / data parallelism (gloo, CPU)
compared with a single-process run of the same global batch.

    python run_model_parallel.py --ref FILE                 # writes loss, grad-norm and full gradients
    torchrun ... run_model_parallel.py --tp 2 --sp 1 FILE   # every rank checks itself against FILE
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from areal_b200.api.alloc_mode import ParallelStrategy  # noqa: E402
from areal_b200.api.cli_args import MicroBatchSpec, OptimizerConfig, TrainEngineConfig  # noqa: E402
from areal_b200.engine.train_engine import B200TrainEngine  # noqa: E402
from areal_b200.parallel.tensor_parallel import is_tp_replicated, tp_unslice  # noqa: E402


def global_batch(n_seq=8, L=48, vocab=1024, images=False, one_image=False):
    g = torch.Generator().manual_seed(7)
    lens = torch.randint(L // 3, L + 1, (n_seq,), generator=g)
    ids = torch.randint(0, 900 if images else vocab, (n_seq, L), generator=g)
    mask = torch.arange(L)[None, :] < lens[:, None]
    loss_mask = mask & (torch.arange(L)[None, :] >= 4)
    out = dict(input_ids=ids * mask, attention_mask=mask, loss_mask=loss_mask.int())
    if images:
        # every sequence but the third starts with one image: <start> pads <end>; placeholder ids of the tiny presets
        mm = []
        for i in range(n_seq):
            if i % 3 == 2 or (one_image and i > 0):
                mm.append({})
                continue
            h, w = [(4, 4), (4, 6)][i % 2]
            n = h * w // 4
            out["input_ids"][i, 0] = 1002
            out["input_ids"][i, 1:1 + n] = 1000
            out["input_ids"][i, 1 + n] = 1003
            mm.append(dict(pixel_values=torch.randn(h * w, 3 * 2 * 14 * 14, generator=g),
                           image_grid_thw=torch.tensor([[1, h, w]])))
        out["multi_modal_input"] = mm
    return out


def loss_fn(logp, ent, mb):
    m = torch.roll(mb["loss_mask"], shifts=-1, dims=0).float()
    return -(logp * m).sum() / m.sum().clamp(min=1)


def weight_fn(mb):
    return float(mb["loss_mask"].sum())


def perturb_lora_b(eng):
    """Adapters start with B = 0 (the adapted model equals the base model), which leaves A without a gradient:
    give B values that depend only on the parameter's global name, so that every layout sees the same adapter."""
    import zlib

    from areal_b200.parallel.tensor_parallel import tp_slice_lora_b

    pctx = eng.pctx
    with torch.no_grad():
        for name, p in eng.model.named_parameters():
            if ".lora_B." not in name:
                continue
            gname = name
            if name.startswith("layers."):
                _, idx, rest = name.split(".", 2)
                gname = f"layers.{eng.model.layer_ids[int(idx)]}.{rest}"
            tp = pctx.tp_size if pctx is not None else 1
            g = torch.Generator().manual_seed(zlib.crc32(gname.encode()))
            full_rows = p.shape[0] * (tp if tp_slice_lora_b(gname) else 1)
            full = torch.randn(full_rows, p.shape[1], generator=g) * 0.05
            full[:, eng.model_config.lora_rank:] = 0  # the rank padding stays zero
            if tp > 1 and tp_slice_lora_b(gname):
                n = p.shape[0]
                full = full[pctx.tp_rank * n:(pctx.tp_rank + 1) * n]
            p.copy_(full.to(p.dtype))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("file")
    ap.add_argument("--ref", action="store_true")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--sp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--ep", type=int, default=1)
    ap.add_argument("--lora", action="store_true", help="low-rank adapters on every dense projection, base frozen")
    ap.add_argument("--etp", type=int, default=1, help="expert tensor parallelism: ranks that hold slices of the same experts")
    ap.add_argument("--preset", default="tiny-qwen2")
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    ap.add_argument("--no-bias", action="store_true", help="Qwen3-style attention (no qkv bias): enables the fused Ulysses projection")
    ap.add_argument("--n-mbs", type=int, default=1)
    ap.add_argument("--critic", action="store_true")
    ap.add_argument("--images", action="store_true", help="image prompts (vision-language presets)")
    ap.add_argument("--one-image", action="store_true", help="only the first sequence carries an image")
    ap.add_argument("--shard-vision", action="store_true", help="divide the vision tower's images over the sp ranks")
    ap.add_argument("--layers", type=int, default=0, help="override the preset's number of blocks")
    ap.add_argument("--vpp", type=int, default=1, help="virtual pipeline stages (model chunks) per rank")
    ap.add_argument("--schedule", default="", help="pipeline schedule: GPipe | 1F1B | Interleaved1F1B")
    ap.add_argument("--zigzag", action="store_true", help="context parallelism with zig-zag chunks and gathered K/V "
                                                          "(the Megatron-style engine's mode) instead of Ulysses")
    args = ap.parse_args()
    cuda = args.device == "cuda"
    tol = 4e-2 if cuda else 2e-4
    over = {}
    if cuda:
        # the CUDA kernels want head_dim 128 and 16-byte aligned rows
        over = dict(head_dim=128, intermediate_size=768)
        if args.no_bias:
            over["attention_bias"] = False
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        if "LOCAL_RANK" in os.environ:
            torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    if args.layers:
        over["num_hidden_layers"] = args.layers
    cfg = TrainEngineConfig(experiment_name="t", trial_name="t", path="", init_from_scratch=True,
                            dtype="bfloat16" if cuda else "float32", model_overrides=over,
                            model_preset=args.preset, mb_spec=MicroBatchSpec(n_mbs=args.n_mbs), is_critic=args.critic,
                            optimizer=OptimizerConfig(lr=1e-3, weight_decay=0.0, gradient_clipping=1.0,
                                                      warmup_steps_proportion=0.0, lr_scheduler_type="constant"))
    if args.lora:
        cfg.use_lora, cfg.lora_rank, cfg.lora_alpha, cfg.target_modules = True, 8, 16, ["all-linear"]
    if args.zigzag:
        cfg.backend = "megatron:d1"
    cfg.megatron.virtual_pipeline_parallel_size = args.vpp
    if args.schedule:
        os.environ["AREAL_B200_PP_SCHEDULE"] = args.schedule
    cfg.fsdp.shard_vision_across_sp = args.shard_vision
    eng = B200TrainEngine(cfg)
    batch = global_batch(L=512 if cuda else 48, images=args.images, one_image=args.one_image)
    if args.ref:
        eng.create_process_group()
        eng.initialize(seed=3)
        data = batch
    else:
        import datetime

        # a short collective timeout: a wedged exchange ends with an error instead of hanging the run
        dist.init_process_group("nccl" if cuda else "gloo", timeout=datetime.timedelta(seconds=120 if cuda else 600))
        world = dist.get_world_size()
        dp = world // (args.tp * args.sp * args.pp)
        eng.create_process_group(ParallelStrategy(tensor_parallel_size=args.tp, context_parallel_size=args.sp,
                                                  pipeline_parallel_size=args.pp, data_parallel_size=dp,
                                                  expert_parallel_size=args.ep,
                                                  expert_tensor_parallel_size=args.etp))
        eng.initialize(seed=3)
        d = eng.data_parallel_rank
        data = {k: v[d::dp] for k, v in batch.items()}  # tensors and the per-sequence image list alike
    if args.lora:
        perturb_lora_b(eng)
    captured = {}
    orig_step = eng.optimizer.step

    def step(*a, **k):
        eng.flat.collect_autograd_grads()
        entries = list(eng.flat.entries)
        if getattr(eng, "flat_experts", None) is not None:
            eng.flat_experts.collect_autograd_grads()
            entries += list(eng.flat_experts.entries)
        for name, p, _, _ in entries:
            captured[name] = p.main_grad.clone()
        return orig_step(*a, **k)

    eng.optimizer.step = step
    # per-token outputs before the step (under pipeline parallelism: computed on the last stage, handed to all)
    before = None if (args.images or cuda) else eng.forward_batch(data)
    lf = (lambda v, mb: ((v - 0.3) ** 2 * mb["loss_mask"].float()).sum() / mb["loss_mask"].sum()) if args.critic else loss_fn
    stats = eng.train_batch(data, lf, weight_fn)
    if args.ref:
        torch.save(dict(loss=stats["loss"], grad_norm=stats["grad_norm"], grads=captured, before=before), args.file)
        print("ref", stats["loss"], stats["grad_norm"])
        return
    ref = torch.load(args.file, map_location="cuda" if cuda else "cpu")
    pctx, mesh = eng.pctx, eng.mesh
    if before is not None and ref.get("before") is not None:
        want = ref["before"][eng.data_parallel_rank::mesh.dp_size]
        assert (before - want).abs().max() < 2e-4, ("forward_batch", float((before - want).abs().max()))
    full = {}
    for name, g in captured.items():
        g = g.clone()
        if pctx.ep_size * pctx.etp_size > 1 and g.dim() == 3 and ".mlp." in name:
            if mesh.edp_size > 1:
                dist.all_reduce(g, group=mesh.edp_group)
            if pctx.etp_size > 1:
                from areal_b200.parallel.tensor_parallel import expert_unslice

                parts = [torch.empty_like(g) for _ in range(pctx.etp_size)]
                dist.all_gather(parts, g.contiguous(), group=pctx.etp_group)
                g = expert_unslice(name, parts)
            if pctx.ep_size > 1:
                parts = [torch.empty_like(g) for _ in range(pctx.ep_size)]
                dist.all_gather(parts, g.contiguous(), group=pctx.ep_group)
                g = torch.cat(parts, 0)
            full[name] = g
            continue
        if mesh.shard_size > 1:
            dist.all_reduce(g, group=mesh.shard_group)
        if pctx.pp_size > 1 and name == "embed" and eng.model_config.tie_word_embeddings and not args.critic \
                and pctx.last_stage_rank != 0:  # (V-shaped placement: one copy serves the lookup and the head)
            # tied embedding / head: the first stage holds the lookup's share of the gradient, the last the head's
            dist.all_reduce(g, group=pctx.pp_tie_group)
        if pctx.tp_size > 1:
            if is_tp_replicated(name):
                if not name.endswith("score"):
                    dist.all_reduce(g, group=pctx.tp_group)
            else:
                parts = [torch.empty_like(g) for _ in range(pctx.tp_size)]
                dist.all_gather(parts, g.contiguous(), group=pctx.tp_group)
                g = tp_unslice(name, parts, eng.model_config)
        full[name] = g
    # the loss is the sum over this rank's micro-batches; data-parallel ranks hold different ones
    loss = torch.tensor([stats["loss"]], dtype=torch.float64, device="cuda" if cuda else "cpu")
    if mesh.dp_size > 1:
        dist.all_reduce(loss, group=mesh.dp_group)
    assert abs(float(loss) - ref["loss"]) < (2e-2 if cuda else 1e-4) * max(1.0, abs(ref["loss"])), (float(loss), ref["loss"])
    for name, g in full.items():
        if name.startswith("layers."):
            _, idx, rest = name.split(".", 2)
            name = f"layers.{eng.model.layer_ids[int(idx)]}.{rest}"
        r = ref["grads"][name]
        err = (g - r).abs().max().item()
        assert err <= tol * (r.abs().max().item() + 1e-6) + (1e-3 if cuda else 0), (name, err, r.abs().max().item(), g.abs().max().item(), (g - 2 * r).abs().max().item())
    assert abs(stats["grad_norm"] - ref["grad_norm"]) < tol * ref["grad_norm"], (stats["grad_norm"], ref["grad_norm"])
    if cuda:
        from areal_b200.ops import _lib

        assert _lib.read_status() == 0
        if args.sp > 1 and args.no_bias:
            # the projection + sequence→head exchange must have gone through the fused kernel
            assert eng.pctx.extras.get("qkv_perm"), "fused Ulysses projection did not run"
    # and the update itself went through on every rank
    assert stats["update_successful"] == 1.0
    dist.barrier()
    if dist.get_rank() == 0:
        print("OK", float(loss), stats["grad_norm"])
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
