"""Whole-model check: the CUDA-kernel path of a small Qwen3-shaped model against
the PyTorch reference path of the same module in fp32."""
import dataclasses
import os

import pytest
import torch

from areal_b200.models.config import PRESETS
from areal_b200.models.qwen import build_model
from areal_b200.ops import _lib
from areal_b200.ops.attention import VarlenMeta
from areal_b200.ops.lm_head import lm_head_logprobs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("preset,over", [
    ("qwen3-1.7b", dict(num_hidden_layers=2, hidden_size=512, intermediate_size=1024, num_attention_heads=4,
                        num_key_value_heads=2, vocab_size=4096)),
    ("qwen2.5-7b", dict(num_hidden_layers=2, hidden_size=512, intermediate_size=1024, num_attention_heads=4,
                        num_key_value_heads=2, vocab_size=4096)),
])
def test_model_forward_backward_matches_reference(preset, over):
    cfg = dataclasses.replace(PRESETS[preset], **over)
    m = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=0)
    ref = build_model(cfg, dtype=torch.float32, device="cuda", seed=None)
    ref.load_state_dict({k: v.float() for k, v in m.state_dict().items()})
    lens = [100, 37, 260]
    T = sum(lens)
    cu = [0, 100, 137, 397]
    ids = torch.randint(0, cfg.vocab_size, (T,), device="cuda")
    pos = torch.cat([torch.arange(n) for n in lens]).cuda()
    labels = torch.roll(ids, -1)
    meta = VarlenMeta(cu, "cuda")
    h = m(ids, pos, meta)
    logp, ent = lm_head_logprobs(h, m.output_weight(), labels, 1.0)
    loss = -(logp.mean()) + 0.01 * ent.mean()
    loss.backward()
    assert _lib.read_status() == 0
    os.environ["AREAL_B200_FORCE_TORCH"] = "1"
    try:
        hr = ref(ids, pos, meta)
        logp_r, ent_r = lm_head_logprobs(hr, ref.output_weight(), labels, 1.0)
        loss_r = -(logp_r.mean()) + 0.01 * ent_r.mean()
        loss_r.backward()
    finally:
        del os.environ["AREAL_B200_FORCE_TORCH"]
    assert abs(loss.item() - loss_r.item()) < 3e-2
    torch.testing.assert_close(logp, logp_r, atol=0.15, rtol=0.05)
    gm = dict(m.named_parameters())
    for name, pr in ref.named_parameters():
        g = gm[name].grad
        assert g is not None, name
        num = (g.float() - pr.grad).norm().item()
        den = pr.grad.norm().item() + 1e-8
        assert num / den < 0.08, f"{name}: rel grad err {num / den:.4f}"
