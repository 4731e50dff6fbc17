"""The Bailing hybrid family: lightning (linear) attention layers with a latent softmax-attention layer closing every
group, DeepSeek-style mixtures. No ``transformers`` class exists for it, so the oracle of the lightning layer is a
token-by-token restatement of its definition written out here, and the model-level checks are consistency checks
(checkpoint names, round trip, parallel layouts against one process)."""
import dataclasses
import math
import os
import subprocess
import sys

import pytest
import torch

from areal_b200.models.config import PRESETS, ModelConfig
from areal_b200.models.qwen import build_model
from areal_b200.ops.attention import VarlenMeta
from tests.conftest import free_port

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "torchrun", "run_model_parallel.py")


def _lightning_oracle(layer, x, cu, layer_idx, n_layers):
    """Definition of the layer, one token at a time, fp64."""
    cfg = layer.cfg
    nh, D, rot = cfg.num_attention_heads, cfg.lightning_head_dim, int(cfg.lightning_head_dim * cfg.partial_rotary_factor)
    x = x.double()
    W = {n: p.detach().double() for n, p in layer.named_parameters()}
    # ALiBi slopes written as the closed form for a power-of-two head count
    assert math.log2(nh).is_integer()
    slopes = torch.tensor([2.0 ** (-8.0 * (i + 1) / nh) for i in range(nh)], dtype=torch.float64)
    decay = torch.exp(-slopes * (1.0 - layer_idx / (n_layers - 1) + 1e-5))
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, rot, 2, dtype=torch.float64) / rot))
    G = cfg.lightning_norm_groups
    out = torch.zeros(x.shape[0], cfg.hidden_size, dtype=torch.float64)
    for s0, s1 in zip(cu[:-1], cu[1:]):
        S = torch.zeros(nh, D, D, dtype=torch.float64)
        for t in range(s0, s1):
            qkv = (W["qkv"] @ x[t]).view(3, nh, D)
            q, k, v = qkv[0], qkv[1], qkv[2]
            q = q / torch.sqrt(q.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * W["q_norm"]
            k = k / torch.sqrt(k.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * W["k_norm"]
            ang = (t - s0) * inv

            def rope(u):
                a, b = u[:, :rot // 2], u[:, rot // 2:rot]
                return torch.cat((a * ang.cos() - b * ang.sin(), b * ang.cos() + a * ang.sin(), u[:, rot:]), -1)

            q, k = rope(q), rope(k)
            S = decay[:, None, None] * S + k[:, :, None] * v[:, None, :]
            o = torch.einsum("hkv,hk->hv", S, q) / math.sqrt(D)
            og = o.view(G, -1)
            og = (og / torch.sqrt(og.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps)).view(nh, D) * W["g_norm"].view(nh, D)
            gate = torch.sigmoid(W["gate"] @ x[t]).view(nh, D)
            out[t] = W["o"] @ (og * gate).reshape(-1)
    return out


def test_lightning_layer_matches_its_definition():
    from areal_b200.models.lightning import LightningAttention

    cfg = PRESETS["tiny-bailing-hybrid"]
    torch.manual_seed(0)
    layer = LightningAttention(cfg, torch.float32, "cpu", None, layer_idx=1)
    with torch.no_grad():
        for n, p in layer.named_parameters():
            p.copy_(torch.randn_like(p) * (0.1 if "norm" not in n else 0.2) + (1.0 if "norm" in n else 0.0))
    cu = [0, 70, 75, 140]          # longer than the recurrence's chunk, one short sequence
    x = torch.randn(cu[-1], cfg.hidden_size)
    pos = torch.cat([torch.arange(b - a) for a, b in zip(cu[:-1], cu[1:])])
    meta = VarlenMeta(torch.tensor(cu, dtype=torch.int32), "cpu")
    want = _lightning_oracle(layer, x, cu, 1, cfg.num_hidden_layers)
    with torch.no_grad():
        got = layer(x, None, None, pos, meta)
    torch.testing.assert_close(got.double(), want, atol=2e-4, rtol=2e-4)
    # the differentiable (chunk-parallel) path computes the same thing
    x.requires_grad_(True)
    got2 = layer(x, None, None, pos, meta)
    torch.testing.assert_close(got2.detach().double(), want, atol=2e-4, rtol=2e-4)
    got2.sum().backward()
    assert x.grad.abs().sum() > 0 and layer.qkv.grad.abs().sum() > 0 and layer.g_norm.grad.abs().sum() > 0


def test_decay_schedule_over_layers_and_heads():
    from areal_b200.models.lightning import alibi_slopes, layer_log_decay

    s = alibi_slopes(8)
    assert torch.allclose(s, torch.tensor([2.0 ** -(i + 1) for i in range(8)]))
    assert alibi_slopes(12).shape == (12,) and torch.allclose(alibi_slopes(12)[:8], s)
    first, last = layer_log_decay(8, 0, 5), layer_log_decay(8, 4, 5)
    assert torch.all(first < last) and torch.all(last < 0)          # later layers forget more slowly
    assert torch.allclose(last, -s * 1e-5)


def test_layer_pattern_checkpoint_names_and_round_trip(tmp_path):
    from areal_b200.utils.hf_io import iter_hf_tensors, load_hf_weights, save_hf_checkpoint

    cfg = PRESETS["tiny-bailing-hybrid"]
    assert [cfg.layer_is_lightning(i) for i in range(4)] == [True, False, True, False]
    m = build_model(cfg, dtype=torch.float32, seed=1)
    assert [type(l.attn).__name__ for l in m.layers] == ["LightningAttention", "MLAttention"] * 2
    with torch.no_grad():
        for layer in m.layers:
            if getattr(layer.mlp, "expert_bias", None) is not None:
                layer.mlp.expert_bias.copy_(torch.randn(cfg.num_experts) * 0.2)
    save_hf_checkpoint(m, cfg, str(tmp_path))
    names = {n for n, _ in iter_hf_tensors(str(tmp_path))}
    for want in ("model.word_embeddings.weight", "model.layers.0.attention.query_key_value.weight",
                 "model.layers.0.attention.g_norm.weight", "model.layers.0.attention.dense.weight",
                 "model.layers.1.attention.kv_a_proj_with_mqa.weight", "model.layers.1.attention.q_b_proj.weight",
                 "model.layers.1.attention.dense.weight", "model.layers.1.mlp.gate.expert_bias",
                 "model.layers.1.mlp.shared_experts.up_proj.weight", "model.layers.1.mlp.experts.3.down_proj.weight",
                 "model.layers.0.mlp.gate_proj.weight", "model.norm.weight", "lm_head.weight"):
        assert want in names, want
    assert not any("self_attn" in n or "embed_tokens" in n for n in names)
    back = ModelConfig.from_hf_config(str(tmp_path))
    assert dataclasses.asdict(back) == dataclasses.asdict(cfg)
    m2 = load_hf_weights(build_model(back, dtype=torch.float32, seed=None), str(tmp_path))
    ids = torch.randint(0, cfg.vocab_size, (50,), generator=torch.Generator().manual_seed(3))
    meta = VarlenMeta(torch.tensor([0, 20, 50], dtype=torch.int32), "cpu")
    pos = torch.cat([torch.arange(20), torch.arange(30)])
    with torch.no_grad():
        a, b = m.logits(m(ids, pos, meta)), m2.logits(m2(ids, pos, meta))
    assert torch.equal(a, b) and torch.isfinite(a).all()
    # packed sequences do not see each other: the second sequence alone gives the same logits
    with torch.no_grad():
        alone = m.logits(m(ids[20:], torch.arange(30), VarlenMeta(torch.tensor([0, 30], dtype=torch.int32), "cpu")))
    torch.testing.assert_close(alone, a[20:], atol=1e-4, rtol=1e-4)


def _ref(tmp_path):
    f = str(tmp_path / "ref.pt")
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    r = subprocess.run([sys.executable, WORKER, "--ref", "--n-mbs", "2", "--preset", "tiny-bailing-hybrid", f],
                       env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    return f


@pytest.mark.parametrize("args", [["--sp", "2"], ["--ep", "2"], ["--pp", "2", "--n-mbs", "2"],
                                  ["--pp", "2", "--n-mbs", "4", "--schedule", "ZBVZeroBubble"]])
def test_training_step_under_parallel_layouts_matches_single_process(tmp_path, args):
    """Ulysses (the recurrence runs on heads / 2 over the whole stream after a tokens → heads exchange), expert and
    pipeline parallelism (also with one block per stage in the V-shaped placement: the per-layer decays follow the
    global layer index): loss, gradient norm and every gradient as in one process."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(free_port()), WORKER] + args + ["--preset", "tiny-bailing-hybrid",
                                                                             _ref(tmp_path)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
