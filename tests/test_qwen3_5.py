"""Qwen3.5 hybrid family: chunk-parallel gated delta rule against the per-token recurrence, the two
layer types against explicit restatements built from checkpoint-named tensors, checkpoint round
trip (1-centred norm weights), and training through the engine."""
import dataclasses
import json
import math
import os

import pytest
import torch
import torch.nn.functional as F

from areal_b200.models.config import PRESETS, ModelConfig
from areal_b200.models.qwen import build_model
from areal_b200.ops.attention import VarlenMeta
from areal_b200.ops.linear_attn import linear_attn_chunked, linear_attn_ref

CFG = PRESETS["tiny-qwen3_5"]


@pytest.mark.parametrize("mode", ["gated_delta", "simple_gla"])
def test_chunked_recurrence_matches_per_token(mode):
    torch.manual_seed(0)
    T, H, DK, DV = 150, 3, 16, 24
    cu = torch.tensor([0, 70, 71, 150])
    base = [F.normalize(torch.randn(T, H, DK), dim=-1), F.normalize(torch.randn(T, H, DK), dim=-1),
            torch.randn(T, H, DV), torch.rand(T, H) * 0.6 + 0.4, torch.rand(T, H)]
    a = [t.clone().requires_grad_(True) for t in base]
    b = [t.clone().requires_grad_(True) for t in base]
    o1 = linear_attn_ref(*a, cu, 0.25, mode)
    o2 = linear_attn_chunked(*b, cu, 0.25, mode, chunk=32)
    assert torch.allclose(o1, o2, atol=1e-5)
    gy = torch.randn_like(o1)
    o1.backward(gy)
    o2.backward(gy)
    for x, y in zip(a, b):
        if x.grad is not None:
            assert torch.allclose(x.grad, y.grad, atol=2e-5)


def _setup(lens=(23, 41)):
    torch.manual_seed(1)
    m = build_model(CFG, dtype=torch.float32, seed=5)
    with torch.no_grad():  # move norms away from their initial ones so that the 1-centring is exercised
        for n, p in m.named_parameters():
            if n.endswith("norm") or "_norm" in n:
                p.add_(torch.randn_like(p) * 0.1)
    T = sum(lens)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    pos = torch.cat([torch.arange(n) for n in lens])
    meta = VarlenMeta(torch.tensor(cu, dtype=torch.int32), "cpu")
    return m, T, cu, pos, meta


def test_gated_delta_net_layer_matches_restatement():
    m, T, cu, pos, meta = _setup()
    layer = m.layers[0].attn
    hf = {k: v.detach() for k, v in m.to_hf()}
    p = "model.layers.0.linear_attn."
    x = torch.randn(T, CFG.hidden_size)
    cos, sin = m.rope("cpu")
    got = layer(x, cos, sin, pos, meta)
    nk, nv, dk, dv = CFG.linear_num_key_heads, CFG.linear_num_value_heads, CFG.linear_key_head_dim, CFG.linear_value_head_dim
    outs = []
    for s, e in zip(cu[:-1], cu[1:]):
        xs = x[s:e]
        mixed = xs @ hf[p + "in_proj_qkv.weight"].T
        z = xs @ hf[p + "in_proj_z.weight"].T
        a = xs @ hf[p + "in_proj_a.weight"].T
        b = xs @ hf[p + "in_proj_b.weight"].T
        conv = F.conv1d(mixed.T[None], hf[p + "conv1d.weight"], padding=CFG.linear_conv_kernel_dim - 1,
                        groups=mixed.shape[1])[0, :, :e - s].T
        mixed = F.silu(conv)
        q, k, v = mixed.split([nk * dk, nk * dk, nv * dv], -1)
        q = F.normalize(q.reshape(-1, nk, dk), dim=-1, eps=0).repeat_interleave(nv // nk, 1)
        k = F.normalize(k.reshape(-1, nk, dk), dim=-1, eps=0).repeat_interleave(nv // nk, 1)
        v = v.reshape(-1, nv, dv)
        beta = torch.sigmoid(b)
        g = -hf[p + "A_log"].exp() * F.softplus(a + hf[p + "dt_bias"])
        S = torch.zeros(nv, dk, dv)
        o = []
        for t in range(e - s):
            S = S * g[t].exp()[:, None, None]
            u = beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, k[t]))
            S = S + torch.einsum("hk,hv->hkv", k[t], u)
            o.append(torch.einsum("hkv,hk->hv", S, q[t]) * dk ** -0.5)
        o = torch.stack(o)
        o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + CFG.rms_norm_eps) * hf[p + "norm.weight"]
        o = o * F.silu(z.reshape(-1, nv, dv))
        outs.append(o.reshape(e - s, -1) @ hf[p + "out_proj.weight"].T)
    want = torch.cat(outs)
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), float((got - want).abs().max())


def test_gated_attention_layer_matches_restatement():
    m, T, cu, pos, meta = _setup()
    li = CFG.layer_types.index("full_attention")
    layer = m.layers[li].attn
    hf = {k: v.detach() for k, v in m.to_hf()}
    p = f"model.layers.{li}.self_attn."
    x = torch.randn(T, CFG.hidden_size)
    cos, sin = m.rope("cpu")
    got = layer(x, cos, sin, pos, meta)
    nq, nkv, D = CFG.num_attention_heads, CFG.num_key_value_heads, CFG.head_dim
    R = int(D * CFG.partial_rotary_factor)
    inv = 1.0 / (CFG.rope_theta ** (torch.arange(0, R, 2).float() / R))

    def norm1p(t, w):  # checkpoint semantics: (1 + w) * norm(x)
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + CFG.rms_norm_eps) * (1 + w)

    def rope(t, positions):
        fr = torch.outer(positions.float(), inv)
        c, s = torch.cat([fr.cos()] * 2, -1)[:, None], torch.cat([fr.sin()] * 2, -1)[:, None]
        tr, tp = t[..., :R], t[..., R:]
        rot = torch.cat([-tr[..., R // 2:], tr[..., :R // 2]], -1)
        return torch.cat([tr * c + rot * s, tp], -1)

    outs = []
    for s, e in zip(cu[:-1], cu[1:]):
        xs, L = x[s:e], e - s
        qg = (xs @ hf[p + "q_proj.weight"].T).view(L, nq, 2 * D)
        q, gate = qg[..., :D], qg[..., D:].reshape(L, -1)
        k = (xs @ hf[p + "k_proj.weight"].T).view(L, nkv, D)
        v = (xs @ hf[p + "v_proj.weight"].T).view(L, nkv, D)
        q, k = rope(norm1p(q, hf[p + "q_norm.weight"]), pos[s:e]), rope(norm1p(k, hf[p + "k_norm.weight"]), pos[s:e])
        k, v = k.repeat_interleave(nq // nkv, 1), v.repeat_interleave(nq // nkv, 1)
        att = torch.einsum("ihd,jhd->hij", q, k) / math.sqrt(D)
        att = att.masked_fill(~torch.ones(L, L, dtype=torch.bool).tril(), float("-inf")).softmax(-1)
        o = torch.einsum("hij,jhd->ihd", att, v).reshape(L, -1) * torch.sigmoid(gate)
        outs.append(o @ hf[p + "o_proj.weight"].T)
    want = torch.cat(outs)
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), float((got - want).abs().max())


def test_checkpoint_round_trip(tmp_path):
    from areal_b200.utils.hf_io import load_hf_weights, save_hf_checkpoint

    m, T, cu, pos, meta = _setup()
    ids = torch.randint(0, CFG.vocab_size, (T,))
    with torch.no_grad():
        h0 = m(ids, pos, meta)
    fresh = build_model(CFG, dtype=torch.float32, seed=9)
    hf = dict(fresh.to_hf())
    assert float(hf["model.norm.weight"].detach().abs().max()) == 0.0  # initial multiplier 1 is stored as 0
    save_hf_checkpoint(m, CFG, str(tmp_path))
    conf = json.load(open(os.path.join(tmp_path, "config.json")))
    assert conf["model_type"] == "qwen3_5_text" and conf["layer_types"] == CFG.layer_types
    cfg2 = ModelConfig.from_hf_config(str(tmp_path))
    assert cfg2.layer_types == CFG.layer_types and cfg2.norm_one_plus and cfg2.attn_output_gate
    assert cfg2.partial_rotary_factor == CFG.partial_rotary_factor and cfg2.linear_num_value_heads == 4
    m2 = build_model(cfg2, dtype=torch.float32, seed=None)
    load_hf_weights(m2, str(tmp_path))
    with torch.no_grad():
        h1 = m2(ids, pos, meta)
    assert torch.allclose(h0, h1, atol=1e-5)


def test_engine_trains_hybrid_model(tmp_path):
    from areal_b200.api.cli_args import MicroBatchSpec, OptimizerConfig, SFTConfig, TrainEngineConfig, _propagate_names
    from areal_b200.trainer.sl_trainer import SFTTrainer

    g = torch.Generator().manual_seed(0)
    data = []
    for _ in range(8):
        n = int(torch.randint(12, 24, (1,), generator=g))
        data.append(dict(input_ids=torch.randint(0, 1024, (n,), generator=g).tolist(), loss_mask=[0] * 4 + [1] * (n - 4)))
    cfg = SFTConfig(actor=TrainEngineConfig(
        backend="fsdp:d1", model_preset="tiny-qwen3_5", init_from_scratch=True,
        optimizer=OptimizerConfig(lr=2e-3, warmup_steps_proportion=0.0, weight_decay=0.0),
        mb_spec=MicroBatchSpec(max_tokens_per_mb=512)))
    cfg.experiment_name, cfg.trial_name = "t", "t"
    cfg.cluster.fileroot = str(tmp_path)
    cfg.train_dataset.batch_size = 8
    cfg.train_dataset.shuffle = False
    cfg.total_train_epochs = 6
    _propagate_names(cfg)
    losses = []
    with SFTTrainer(cfg, data, data) as tr:
        tr.train(max_steps=6, step_callback=lambda s, st: losses.append(st["step/loss"]))
    assert len(losses) == 6 and losses[-1] < losses[0]


@pytest.mark.gpu
def test_hybrid_model_cuda_matches_fp32_reference():
    from areal_b200.ops import _lib
    from areal_b200.ops.lm_head import lm_head_logprobs

    cfg = dataclasses.replace(CFG, hidden_size=512, intermediate_size=1024, head_dim=128, vocab_size=4096,
                              linear_key_head_dim=64, linear_value_head_dim=64)
    m = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=0)
    ref = build_model(cfg, dtype=torch.float32, device="cuda", seed=None)
    ref.load_state_dict({k: v.float() for k, v in m.state_dict().items()})
    lens = [100, 37, 260]
    T = sum(lens)
    torch.manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (T,), device="cuda")
    pos = torch.cat([torch.arange(n) for n in lens]).cuda()
    labels = torch.roll(ids, -1)
    meta = VarlenMeta([0, 100, 137, 397], "cuda")
    h = m(ids, pos, meta)
    logp, _ = lm_head_logprobs(h, m.output_weight(), labels, 1.0)
    (-logp.mean()).backward()
    assert _lib.read_status() == 0
    with torch.no_grad():
        h_ng = m(ids, pos, meta)  # no-grad path: the recurrence runs its CUDA kernel
    os.environ["AREAL_B200_FORCE_TORCH"] = "1"
    try:
        hr = ref(ids, pos, meta)
        logp_r, _ = lm_head_logprobs(hr, ref.output_weight(), labels, 1.0)
        (-logp_r.mean()).backward()
    finally:
        del os.environ["AREAL_B200_FORCE_TORCH"]
    hr = hr.detach()
    for got in (h.detach().float(), h_ng.float()):  # bf16 through 4 blocks: error relative to the activations' norm
        assert float((got - hr).norm() / hr.norm()) < 0.03
    torch.testing.assert_close(logp, logp_r, atol=0.15, rtol=0.05)
    gm = dict(m.named_parameters())
    for name, pr in ref.named_parameters():
        if pr.grad is None:
            continue
        g = gm[name].grad
        assert g is not None, name
        rel = (g.float() - pr.grad).norm().item() / (pr.grad.norm().item() + 1e-8)
        # the per-head decay parameters (4 numbers each) collect per-token terms of both signs: bf16 rounding of
        # the activations is large against their small total, so only the order of magnitude is checked
        tol = 0.75 if name.endswith(("attn.dt_bias", "attn.A_log")) else 0.1
        assert rel < tol, f"{name}: rel grad err {rel:.4f}"


def test_rollout_engine_serves_hybrid_model():
    """Greedy generation through the rollout engine (paged KV for the full-attention layers, recurrent +
    convolution state for the linear-attention layers, several sequences of different lengths at once)
    equals re-running the whole model on the growing sequence."""
    import asyncio

    from areal_b200.api.cli_args import GenerationHyperparameters, InferenceEngineConfig, NativeRolloutConfig
    from areal_b200.api.io_struct import ModelRequest
    from areal_b200.engine.rollout_engine import NativeRolloutEngine

    cfg = InferenceEngineConfig(experiment_name="e", trial_name="t", backend="native:d1", max_concurrent_rollouts=16,
                                consumer_batch_size=4,
                                native=NativeRolloutConfig(model_preset="tiny-qwen3_5", context_length=128, max_num_seqs=8,
                                                           max_num_batched_tokens=512, num_kv_blocks=64, seed=3,
                                                           cuda_graph=False))
    eng = NativeRolloutEngine(cfg).initialize(device="cpu")
    try:
        assert eng.hybrid_state is not None and eng.kv_caches[0] is None and eng.kv_caches[3] is not None
        g = torch.Generator().manual_seed(7)
        prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (5, 19, 2, 33)]
        gc = GenerationHyperparameters(max_new_tokens=9, greedy=True, ignore_eos=True)

        async def go():
            return await asyncio.gather(*[eng.agenerate(ModelRequest(rid=str(i), input_ids=p, gconfig=gc))
                                          for i, p in enumerate(prompts)])

        outs = asyncio.run(go())
        model = eng.model
        for p, r in zip(prompts, outs):
            seq = list(p)
            for _ in range(9):
                ids = torch.tensor(seq)
                meta = VarlenMeta(torch.tensor([0, len(seq)], dtype=torch.int32), "cpu")
                with torch.no_grad():
                    h = model(ids, torch.arange(len(seq)), meta)
                    seq.append(int(model.logits(h[-1:]).argmax(-1)))
            assert r.output_tokens == seq[len(p):], (r.output_tokens, seq[len(p):])
        assert not eng._state_slot and len(eng._free_state_slots) == 8  # every slot returned
    finally:
        eng.destroy()


@pytest.mark.gpu
def test_rollout_engine_serves_hybrid_model_cuda():
    """bf16 on the GPU kernels (head_dim 128 paged decode, recurrence kernel with final state): the
    log-probabilities the engine reports for its greedy tokens match a full forward over the result."""
    import asyncio

    from areal_b200.api.cli_args import GenerationHyperparameters, InferenceEngineConfig, NativeRolloutConfig
    from areal_b200.api.io_struct import ModelRequest
    from areal_b200.engine.rollout_engine import NativeRolloutEngine

    over = dict(hidden_size=512, intermediate_size=1024, head_dim=128, vocab_size=4096, linear_key_head_dim=64,
                linear_value_head_dim=64)
    cfg = InferenceEngineConfig(experiment_name="e", trial_name="t", backend="native:d1", max_concurrent_rollouts=16,
                                consumer_batch_size=4,
                                native=NativeRolloutConfig(model_preset="tiny-qwen3_5", model_overrides=over,
                                                           context_length=256, max_num_seqs=8, max_num_batched_tokens=1024,
                                                           num_kv_blocks=64, seed=3))
    eng = NativeRolloutEngine(cfg).initialize()
    try:
        g = torch.Generator().manual_seed(7)
        prompts = [torch.randint(0, 4000, (n,), generator=g).tolist() for n in (40, 150, 3)]
        gc = GenerationHyperparameters(max_new_tokens=12, greedy=True, ignore_eos=True)

        async def go():
            return await asyncio.gather(*[eng.agenerate(ModelRequest(rid=str(i), input_ids=p, gconfig=gc))
                                          for i, p in enumerate(prompts)])

        outs = asyncio.run(go())
        for p, r in zip(prompts, outs):
            seq = torch.tensor(p + r.output_tokens, device="cuda")
            meta = VarlenMeta([0, len(seq)], "cuda")
            with torch.no_grad():
                h = eng.model(seq, torch.arange(len(seq), device="cuda"), meta)
                lp = torch.log_softmax(eng.model.logits(h).float(), -1)
            want = lp[len(p) - 1:-1].gather(1, seq[len(p):, None]).squeeze(1).cpu()
            got = torch.tensor(r.output_logprobs)
            assert float((got - want).abs().max()) < 0.15
    finally:
        eng.destroy()


def test_moe_with_shared_expert_and_hybrid_moe(tmp_path):
    """Routed experts plus a sigmoid-gated shared expert (Qwen2-MoE / Qwen3.5-MoE): the block against a
    restatement from checkpoint-named tensors, and a hybrid MoE model through checkpoint round trip."""
    from areal_b200.models.qwen import MoEMLP
    from areal_b200.utils.hf_io import load_hf_weights, save_hf_checkpoint

    cfg = dataclasses.replace(CFG, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64,
                              shared_expert_intermediate_size=96, norm_topk_prob=True)
    m = build_model(cfg, dtype=torch.float32, seed=11)
    assert all(isinstance(l.mlp, MoEMLP) and l.mlp.shared_gate_up is not None for l in m.layers)
    hf = {k: v.detach() for k, v in m.to_hf()}
    p = "model.layers.1.mlp."
    x = torch.randn(13, cfg.hidden_size)
    with torch.no_grad():
        got = m.layers[1].mlp(x)
    probs = (x @ hf[p + "gate.weight"].T).softmax(-1)
    w, idx = probs.topk(2, -1)
    w = w / w.sum(-1, keepdim=True)
    want = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for j in range(2):
            e = int(idx[t, j])
            q = p + f"experts.{e}."
            h = F.silu(x[t] @ hf[q + "gate_proj.weight"].T) * (x[t] @ hf[q + "up_proj.weight"].T)
            want[t] += w[t, j] * (h @ hf[q + "down_proj.weight"].T)
    hs = F.silu(x @ hf[p + "shared_expert.gate_proj.weight"].T) * (x @ hf[p + "shared_expert.up_proj.weight"].T)
    want += torch.sigmoid(x @ hf[p + "shared_expert_gate.weight"].T) * (hs @ hf[p + "shared_expert.down_proj.weight"].T)
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-3), float((got - want).abs().max())
    # round trip of the whole hybrid MoE model
    ids = torch.randint(0, cfg.vocab_size, (30,))
    pos = torch.arange(30)
    meta = VarlenMeta(torch.tensor([0, 30], dtype=torch.int32), "cpu")
    with torch.no_grad():
        h0 = m(ids, pos, meta)
    save_hf_checkpoint(m, cfg, str(tmp_path))
    conf = json.load(open(os.path.join(tmp_path, "config.json")))
    assert conf["architectures"] == ["Qwen3_5MoeForCausalLM"] and conf["shared_expert_intermediate_size"] == 96
    cfg2 = ModelConfig.from_hf_config(str(tmp_path))
    assert cfg2.num_experts == 4 and cfg2.shared_expert_intermediate_size == 96 and cfg2.layer_types == cfg.layer_types
    m2 = build_model(cfg2, dtype=torch.float32, seed=None)
    load_hf_weights(m2, str(tmp_path))
    with torch.no_grad():
        assert torch.allclose(m2(ids, pos, meta), h0, atol=1e-5)
    # gradients reach the shared expert and its gate
    out = m(ids, pos, meta)
    out.sum().backward()
    mlp = m.layers[0].mlp
    assert mlp.shared_gate.grad is not None and float(mlp.shared_gate.grad.abs().sum()) > 0
    assert float(mlp.shared_down.grad.abs().sum()) > 0


def test_router_variants_sigmoid_scale_and_bias_balancing():
    """Sigmoid scoring with a route scale, and aux-loss-free balancing: the bias changes which experts are
    picked but not their weights, and it moves towards under-loaded experts during training."""
    from areal_b200.models.qwen import MoEMLP

    base = dataclasses.replace(PRESETS["tiny-qwen3-moe"], moe_score_func="sigmoid", moe_route_scale=2.5,
                               norm_topk_prob=True, moe_load_balance_coeff=0.01)
    torch.manual_seed(0)
    mlp = MoEMLP(base, torch.float32, "cpu")
    for p in mlp.parameters():
        torch.nn.init.normal_(p, std=0.05)
    x = torch.randn(64, base.hidden_size)
    mlp.eval()
    with torch.no_grad():
        idx, w = mlp.route(x)
    s = torch.sigmoid(x @ mlp.router.T)
    top = s.topk(base.num_experts_per_tok, -1)
    assert torch.equal(idx.long(), top.indices)
    assert torch.allclose(w, top.values / top.values.sum(-1, keepdim=True) * 2.5, atol=1e-6)
    # a large bias on expert 0 forces it into every token's selection, with its plain score as weight
    mlp.expert_bias[0] = 10.0
    with torch.no_grad():
        idx2, w2 = mlp.route(x)
    assert bool((idx2 == 0).any(-1).all())
    pos = (idx2 == 0).float().argmax(-1)
    got = w2.gather(1, pos[:, None]).squeeze(1)
    picked = s.gather(1, idx2.long())
    assert torch.allclose(got, (s[:, 0] / picked.sum(-1)) * 2.5, atol=1e-5)
    # training: the over-loaded expert's bias goes down, eval leaves it alone
    mlp.train()
    before = mlp.expert_bias.clone()
    mlp(x.requires_grad_(True)).sum().backward()
    assert float(mlp.expert_bias[0]) < float(before[0]) and mlp.router.grad is not None
    mlp.eval()
    frozen = mlp.expert_bias.clone()
    with torch.no_grad():
        mlp(x.detach())
    assert torch.equal(mlp.expert_bias, frozen)
    assert "expert_bias" in mlp.state_dict() and "expert_bias" not in dict(mlp.named_parameters())


def test_balancing_bias_update_can_be_deferred_to_the_optimizer_step():
    """Under a train engine the bias moves once per optimizer step, from the accumulated token counts (summed over
    the ranks that hold the layer), not after every forward."""
    from areal_b200.models.qwen import MoEMLP

    cfg = dataclasses.replace(PRESETS["tiny-qwen3-moe"], moe_score_func="sigmoid", moe_load_balance_coeff=0.01)
    torch.manual_seed(0)
    mlp = MoEMLP(cfg, torch.float32, "cpu")
    for p in mlp.parameters():
        torch.nn.init.normal_(p, std=0.05)
    mlp.train()
    mlp.defer_bias_update = True
    x = torch.randn(32, cfg.hidden_size)
    mlp(x).sum().backward()
    mlp(x).sum().backward()
    assert torch.equal(mlp.expert_bias, torch.zeros(cfg.num_experts))
    assert float(mlp.load_acc.sum()) == 2 * 32 * cfg.num_experts_per_tok
    load = mlp.load_acc.clone()
    mlp.update_expert_bias()
    assert torch.equal(mlp.expert_bias, 0.01 * torch.sign(load.mean() - load)) and float(mlp.load_acc.sum()) == 0
    mlp.update_expert_bias()                                   # nothing counted: nothing moves
    assert torch.equal(mlp.expert_bias, 0.01 * torch.sign(load.mean() - load))


def test_engine_updates_the_balancing_bias_per_step_and_checkpoints_it(tmp_path):
    from areal_b200.api.cli_args import OptimizerConfig, TrainEngineConfig
    from areal_b200.api.io_struct import SaveLoadMeta
    from areal_b200.engine.train_engine import B200TrainEngine

    def make(seed):
        e = B200TrainEngine(TrainEngineConfig(experiment_name="t", trial_name="t", path="", init_from_scratch=True,
                                              dtype="float32", model_preset="tiny-qwen3-moe",
                                              model_overrides={"moe_load_balance_coeff": 0.02},
                                              optimizer=OptimizerConfig(lr=1e-3, warmup_steps_proportion=0.0)))
        e.create_process_group()
        e.initialize(seed=seed)
        return e

    eng = make(1)
    mlps = [l.mlp for l in eng.model.layers]
    assert all(m.defer_bias_update and m.expert_bias is not None for m in mlps)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 1024, (4, 40), generator=g)
    batch = dict(input_ids=ids, attention_mask=torch.ones_like(ids), loss_mask=torch.ones_like(ids))
    loss = lambda lp, ent, mb: -(lp * mb["loss_mask"].float()).sum() / mb["loss_mask"].sum()  # noqa: E731
    eng.train_batch(batch, loss, lambda mb: float(mb["loss_mask"].sum()))
    b1 = [m.expert_bias.clone() for m in mlps]
    for b in b1:   # exactly one update: every entry is 0 or +-coeff
        assert b.abs().sum() > 0 and torch.all((b.abs() < 1e-9) | ((b.abs() - 0.02).abs() < 1e-6)), b
    assert all(float(m.load_acc.sum()) == 0 for m in mlps)
    path = str(tmp_path / "ck")
    eng.save(SaveLoadMeta(path=path, weight_format="dcp", with_optim=True))
    other = make(2)
    other.load(SaveLoadMeta(path=path, weight_format="dcp", with_optim=True))
    assert all(torch.equal(l.mlp.expert_bias, b) for l, b in zip(other.model.layers, b1))


def test_balancing_bias_is_the_same_on_all_data_parallel_ranks():
    import os
    import subprocess
    import sys

    from tests.conftest import free_port

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(free_port()), os.path.join(root, "tests", "torchrun", "run_moe_bias.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
