"""LoRA: adapter algebra on the fused projections, frozen base weights in the engine, merged weights
for the rollout engine, and the adapter checkpoint layout."""
import dataclasses
import json
import os

import pytest
import torch

from areal_b200.api.cli_args import MicroBatchSpec, OptimizerConfig, SFTConfig, TrainEngineConfig, _propagate_names
from areal_b200.api.io_struct import SaveLoadMeta
from areal_b200.models import lora
from areal_b200.models.config import PRESETS
from areal_b200.models.qwen import build_model
from areal_b200.ops.attention import VarlenMeta
from areal_b200.trainer.sl_trainer import SFTTrainer, collate_sft


def _cfg(**kw):
    return dataclasses.replace(PRESETS["tiny-qwen2"], **kw)


def _forward(model, ids, lens):
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32)
    pos = torch.cat([torch.arange(n) for n in lens])
    with torch.no_grad():
        return model(ids, pos, VarlenMeta(cu, ids.device))


def test_adapter_matches_merged_weights_and_targets():
    torch.manual_seed(0)
    base = build_model(_cfg(), dtype=torch.float32, seed=3)
    m = build_model(_cfg(lora_rank=4, lora_alpha=8.0, lora_targets=["q_proj", "v_proj", "down_proj"]),
                    dtype=torch.float32, seed=3)
    # same seed ⇒ same base weights: adapters do not consume the base model's random stream
    bp = dict(base.named_parameters())
    for n, p in m.named_parameters():
        if not lora.is_lora_param(n):
            assert torch.equal(p, bp[n]), n
    a0 = m.layers[0].attn
    assert a0.lora_o is None and m.layers[0].mlp.lora_gate_up is None
    assert list(a0.lora_qkv.lora_B.keys()) == ["q_proj", "v_proj"]
    ids = torch.randint(0, 1024, (40,))
    h0 = _forward(base, ids, [17, 23])
    assert torch.allclose(_forward(m, ids, [17, 23]), h0, atol=1e-6)  # B = 0 at initialisation
    with torch.no_grad():
        for n, p in m.named_parameters():
            if ".lora_B." in n:
                p[:, :4].normal_(0, 0.05)
    h1 = _forward(m, ids, [17, 23])
    assert (h1 - h0).abs().max() > 1e-3
    before = {n: p.detach().clone() for n, p in m.named_parameters()}
    with lora.merged(m):
        # merged base weights, adapters silenced ⇒ the same function
        k_rows = slice(_cfg().q_size, _cfg().q_size + _cfg().kv_size)
        assert torch.equal(m.layers[0].attn.qkv[k_rows], before["layers.0.attn.qkv"][k_rows])  # k_proj not targeted
        merged_sd = {n: p.detach().clone() for n, p in m.named_parameters() if not lora.is_lora_param(n)}
    for n, p in m.named_parameters():
        assert torch.equal(p, before[n]), f"{n} not restored bit-exactly"
    for n, p in base.named_parameters():
        p.data.copy_(merged_sd[n])
    assert torch.allclose(_forward(base, ids, [17, 23]), h1, atol=2e-5)


def test_adapter_gradients_and_padding():
    torch.manual_seed(1)
    ad = lora.LoRAAdapter(32, [("q_proj", 48), ("k_proj", 16), ("v_proj", 16)], ["q_proj", "v_proj"], rank=4,
                          alpha=8.0, dtype=torch.float32, device="cpu")
    with torch.no_grad():
        for p in ad.lora_B.values():
            p[:, :4].normal_()
    x = torch.randn(9, 32, requires_grad=True)
    y = ad(x)
    assert y.shape == (9, 80) and torch.all(y[:, 48:64] == 0)
    assert torch.allclose(y, x @ ad.merged_delta().T, atol=1e-5)
    y.square().sum().backward()
    # the rank padding receives exactly zero gradient, so it stays zero
    assert torch.all(ad.lora_A.grad[4:64] == 0) and torch.all(ad.lora_A.grad[68:] == 0)
    assert torch.all(ad.lora_B["q_proj"].grad[:, 4:] == 0)
    assert ad.lora_A.grad[:4].abs().max() > 0


def _engine_cfg(**kw):
    return TrainEngineConfig(backend="fsdp:d1", model_preset="tiny-qwen2", init_from_scratch=True,
                             optimizer=OptimizerConfig(lr=1e-2, warmup_steps_proportion=0.0, weight_decay=0.0),
                             mb_spec=MicroBatchSpec(max_tokens_per_mb=512), **kw)


def test_engine_trains_adapters_only(tmp_path):
    g = torch.Generator().manual_seed(0)
    data = []
    for _ in range(8):
        n = int(torch.randint(12, 24, (1,), generator=g))
        data.append(dict(input_ids=torch.randint(0, 1024, (n,), generator=g).tolist(), loss_mask=[0] * 4 + [1] * (n - 4)))
    cfg = SFTConfig(actor=_engine_cfg(use_lora=True, lora_rank=8, lora_alpha=16,
                                      target_modules=["all-linear"]))
    cfg.experiment_name, cfg.trial_name = "t", "t"
    cfg.cluster.fileroot = str(tmp_path)
    cfg.train_dataset.batch_size = 8
    cfg.train_dataset.shuffle = False
    cfg.total_train_epochs = 8
    _propagate_names(cfg)
    losses = []
    with SFTTrainer(cfg, data, data) as tr:
        eng = tr.engine
        assert eng.flat_base is not None and eng.weight_flat is eng.flat_base
        n_lora = sum(p.numel() for n, p in eng.model.named_parameters() if lora.is_lora_param(n))
        assert 0 < n_lora <= eng.flat.numel < eng.flat_base.numel
        base0 = eng.flat_base.flat.clone()
        first = tr.wrapper.evaluate_lm(collate_sft(data))
        tr.train(max_steps=8, step_callback=lambda s, st: losses.append(st["step/loss"]))
        last = tr.wrapper.evaluate_lm(collate_sft(data))
        assert torch.equal(eng.flat_base.flat, base0), "base weights must stay frozen"
        assert losses[-1] < losses[0] and last < first
        # merged view: what a rollout engine receives
        with eng._merged_weights():
            merged = eng.flat_base.flat.clone()
        assert not torch.equal(merged, base0) and torch.equal(eng.flat_base.flat, base0)
        # checkpoint: merged HF model + the adapter in the PEFT layout; the adapter round-trips
        path = str(tmp_path / "ckpt")
        eng.save(SaveLoadMeta(path=path, weight_format="hf", with_optim=False))
        conf = json.load(open(os.path.join(path, "adapter_config.json")))
        assert conf["r"] == 8 and conf["peft_type"] == "LORA" and "q_proj" in conf["target_modules"]
        from safetensors.torch import load_file

        ad = load_file(os.path.join(path, "adapter_model.safetensors"))
        key = "base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight"
        assert ad[key].shape == (8, eng.model_config.hidden_size)
        full = load_file(os.path.join(path, "model.safetensors"))
        w = full["model.layers.0.self_attn.q_proj.weight"].float()
        q0 = eng.model.layers[0].attn.qkv[:eng.model_config.q_size].float()
        delta = (ad[key.replace("lora_A", "lora_B")].float() @ ad[key].float()) * (16 / 8)
        assert torch.allclose(w, q0 + delta, atol=2e-2) and not torch.allclose(w, q0, atol=1e-4)
        saved = eng.flat.flat.clone()
        eng.flat.flat.zero_()
        eng.load(SaveLoadMeta(path=path, weight_format="hf", with_optim=False))
        assert torch.allclose(eng.flat.flat.float(), saved.float(), atol=0)


def test_rollout_engine_receives_merged_weights():
    from areal_b200.api.cli_args import InferenceEngineConfig, NativeRolloutConfig
    from areal_b200.api.io_struct import WeightUpdateMeta
    from areal_b200.engine.rollout_engine import NativeRolloutEngine
    from areal_b200.engine.train_engine import B200TrainEngine

    eng = B200TrainEngine(_engine_cfg(use_lora=True, lora_rank=4, lora_alpha=4, target_modules=["q_proj", "up_proj"]))
    eng.create_process_group()
    eng.initialize(None, None)
    rcfg = InferenceEngineConfig(experiment_name="e", trial_name="t", backend="native:d1",
                                 native=NativeRolloutConfig(model_preset="tiny-qwen2", context_length=128,
                                                            max_num_seqs=4, max_num_batched_tokens=256,
                                                            num_kv_blocks=32, seed=1, cuda_graph=False))
    ro = NativeRolloutEngine(rcfg).initialize(device="cpu")
    try:
        with torch.no_grad():
            for n, p in eng.model.named_parameters():
                if ".lora_B." in n:
                    p[:, :4].normal_(0, 0.1)
        eng.connect_engine(ro, WeightUpdateMeta(type="p2p"))
        base = eng.flat_base.flat.clone()
        eng.update_weights(WeightUpdateMeta(type="p2p", version=3))
        assert ro.get_version() == 3
        got = dict(ro.model.named_parameters())
        qs = eng.model_config.q_size
        for i, layer in enumerate(eng.model.layers):
            want = layer.attn.qkv.float() + layer.attn.lora_qkv.merged_delta()
            assert torch.allclose(got[f"layers.{i}.attn.qkv"].float(), want, atol=1e-2)
            assert not torch.allclose(got[f"layers.{i}.attn.qkv"][:qs].float(), layer.attn.qkv[:qs].float(), atol=1e-3)
            assert torch.equal(got[f"layers.{i}.attn.o"], layer.attn.o)  # not targeted
        assert torch.equal(eng.flat_base.flat, base)
    finally:
        ro.destroy()
        eng.destroy()


def test_disk_weight_update_of_a_lora_engine_ignores_the_adapter_file(tmp_path):
    """``update_weights(type="disk")`` writes the merged model and, beside it, ``adapter_model.safetensors``; the
    rollout engine must read only the model's weight files (twice in a row: the second save clears the first
    one's files before writing)."""
    from areal_b200.api.cli_args import InferenceEngineConfig, NativeRolloutConfig
    from areal_b200.api.io_struct import WeightUpdateMeta
    from areal_b200.engine.rollout_engine import NativeRolloutEngine
    from areal_b200.engine.train_engine import B200TrainEngine
    from areal_b200.utils.hf_io import weight_files

    eng = B200TrainEngine(_engine_cfg(use_lora=True, lora_rank=4, lora_alpha=4, target_modules=["q_proj"]))
    eng.create_process_group()
    eng.initialize(None, None)
    rcfg = InferenceEngineConfig(experiment_name="e", trial_name="t", backend="native:d1",
                                 native=NativeRolloutConfig(model_preset="tiny-qwen2", context_length=128,
                                                            max_num_seqs=4, max_num_batched_tokens=256,
                                                            num_kv_blocks=32, seed=1, cuda_graph=False))
    ro = NativeRolloutEngine(rcfg).initialize(device="cpu")
    try:
        with torch.no_grad():
            for n, p in eng.model.named_parameters():
                if ".lora_B." in n:
                    p.normal_(0, 0.1)
        meta = WeightUpdateMeta(type="disk", path=str(tmp_path / "wu"))
        eng.connect_engine(ro, meta)
        for version in (1, 2):
            eng.update_weights(meta.with_version(version))
            assert ro.get_version() == version
            vdir = os.path.join(meta.path, f"weight_update_v{version}")
            assert os.path.exists(os.path.join(vdir, "adapter_model.safetensors"))
            assert [f.name for f in weight_files(vdir)] == ["model.safetensors"]
        got = dict(ro.model.named_parameters())
        want = eng.model.layers[0].attn.qkv.float() + eng.model.layers[0].attn.lora_qkv.merged_delta()
        assert torch.allclose(got["layers.0.attn.qkv"].float(), want, atol=1e-2)
    finally:
        ro.destroy()
        eng.destroy()


@pytest.mark.gpu
def test_adapter_cuda_matches_fp32_reference():
    """bf16 adapter on the tcgen05 GEMMs (rank padded to 64, strided slices of the stacked
    down-projection as GEMM operands) against the same algebra in fp32."""
    torch.manual_seed(0)
    ad = lora.LoRAAdapter(1024, [("q_proj", 1024), ("k_proj", 256), ("v_proj", 256)], lora.ALL_LINEAR, rank=16,
                          alpha=32.0, dtype=torch.bfloat16, device="cuda")
    with torch.no_grad():
        for p in ad.lora_B.values():
            p[:, :16].normal_(0, 0.05)
    x = torch.randn(777, 1024, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = ad(x)
    gy = torch.randn_like(y)
    y.backward(gy)
    W = ad.merged_delta()
    xr = x.detach().float().requires_grad_(True)
    A = ad.lora_A.detach().float().requires_grad_(True)
    Bs = [ad.lora_B[n].detach().float().requires_grad_(True) for n in ("q_proj", "k_proj", "v_proj")]
    u = xr @ A.T
    yr = torch.cat([u[:, i * 64:(i + 1) * 64] @ Bs[i].T for i in range(3)], -1) * ad.scale
    yr.backward(gy.float())
    assert torch.allclose(y.float(), xr.detach() @ W.T, atol=2e-2, rtol=2e-2)
    assert torch.allclose(y.float(), yr, atol=2e-2, rtol=2e-2)
    def close(a, b, rel=2e-2):  # bf16 intermediates: error relative to the tensor's scale
        return float((a.float() - b).abs().max()) <= rel * float(b.abs().max())

    assert close(x.grad, xr.grad)
    assert close(ad.lora_A.grad, A.grad)
    for i, n in enumerate(("q_proj", "k_proj", "v_proj")):
        assert close(ad.lora_B[n].grad, Bs[i].grad)
    assert torch.all(ad.lora_A.grad[16:64] == 0)
