"""Vision-language model (Qwen2.5-VL): parity with transformers, position triples, engine path."""

import dataclasses

import pytest
import torch

from areal_b200.models.config import PRESETS, ModelConfig
from areal_b200.models.qwen import build_model
from areal_b200.models.qwen_vl import QwenVLModel, mrope_position_ids, mrope_tables
from areal_b200.ops.attention import VarlenMeta
from areal_b200.utils.hf_io import load_hf_weights, save_hf_checkpoint

CFG = PRESETS["tiny-qwen2_5-vl"]
IMG = CFG.image_token_id


def _model(seed=0, cfg=CFG):
    m = build_model(cfg, dtype=torch.float32, seed=seed)
    g = torch.Generator().manual_seed(seed + 100)
    with torch.no_grad():  # biases and norm weights start at 0 / 1: perturb them so that parity exercises them
        for n, p in m.named_parameters():
            if n.endswith(("bias", "norm", "shift")):
                p.add_(torch.randn(p.shape, generator=g) * 0.05)
    return m


def _sample(grids, texts, seed=0):
    """One sequence: text run, image, text run, image, ... → ids, pixel rows."""
    g = torch.Generator().manual_seed(seed)
    ids = []
    for i, n in enumerate(texts):
        ids += torch.randint(0, 900, (n,), generator=g).tolist()
        if i < len(grids):
            t, h, w = grids[i]
            ids += [CFG.vision_start_token_id] + [IMG] * (t * h * w // 4) + [CFG.vision_end_token_id]
    n_patch = sum(t * h * w for t, h, w in grids)
    pix = torch.randn(n_patch, 3 * 2 * 14 * 14, generator=g)
    return ids, pix


def test_position_triples():
    ids, _ = _sample([(1, 4, 6)], [3, 2])
    pos, deltas = mrope_position_ids(ids, [0, len(ids)], [(1, 4, 6)], CFG)
    # 3 text + start marker → 0..3; image 2×3 merged grid at offset 4; end marker + 2 text after max+1 = 7
    assert pos[:, :4].tolist() == [[0, 1, 2, 3]] * 3
    assert pos[0, 4:10].tolist() == [4] * 6
    assert pos[1, 4:10].tolist() == [4, 4, 4, 5, 5, 5]
    assert pos[2, 4:10].tolist() == [4, 5, 6, 4, 5, 6]
    assert pos[:, 10:].tolist() == [[7, 8, 9]] * 3
    assert deltas == [10 - len(ids)]
    with pytest.raises(ValueError):
        mrope_position_ids(ids, [0, len(ids)], [(1, 4, 8)], CFG)
    with pytest.raises(ValueError):
        mrope_position_ids(ids, [0, len(ids)], [], CFG)
    # text-only tables equal the ordinary rotary tables
    from areal_b200.ops.fused import rope_tables
    p = torch.arange(7)[None].expand(3, -1)
    cos, sin = mrope_tables(p, 64, 1e4, [8, 12, 12])
    c0, s0 = rope_tables(7, 64, 1e4, "cpu")
    assert torch.allclose(cos, c0) and torch.allclose(sin, s0)


@pytest.mark.parametrize("preset,hf_cls", [("tiny-qwen2_5-vl", "Qwen2_5_VLForConditionalGeneration"),
                                           ("tiny-qwen2-vl", "Qwen2VLForConditionalGeneration"),
                                           ("tiny-qwen3-vl", "Qwen3VLForConditionalGeneration"),
                                           ("tiny-qwen3-vl-moe", "Qwen3VLMoeForConditionalGeneration")])
def test_matches_transformers(tmp_path, preset, hf_cls):
    transformers = pytest.importorskip("transformers")
    CFG = PRESETS[preset]
    m = _model(cfg=CFG)
    assert isinstance(m, QwenVLModel)
    save_hf_checkpoint(m, CFG, str(tmp_path))
    hf = getattr(transformers, hf_cls).from_pretrained(str(tmp_path), torch_dtype=torch.float32)
    hf.eval()
    grids = [(1, 6, 8), (1, 4, 4)]  # 3×4 merged units (ragged 2×2 windows) and 2×2
    ids, pix = _sample(grids, [5, 4, 6], seed=3)
    ids_t = torch.tensor(ids)
    meta = VarlenMeta(torch.tensor([0, len(ids)], dtype=torch.int32), "cpu")
    grid_t = torch.tensor(grids)
    with torch.no_grad():
        feats = m.visual(pix, grid_t)
        theirs_feats = hf.model.visual(pix, grid_thw=grid_t).pooler_output
        assert float((feats - theirs_feats).abs().max()) < 1e-4
        mine = m.logits(m(ids_t, torch.arange(len(ids)), meta, pixel_values=pix, image_grid_thw=grid_t))
        pos, _ = m.positions(ids_t, meta, grid_t)
        hf_pos, _ = hf.model.get_rope_index(ids_t[None], mm_token_type_ids=(ids_t == IMG).long()[None],
                                            image_grid_thw=grid_t)
        assert torch.equal(hf_pos[:, 0], pos)
        theirs = hf(input_ids=ids_t[None], pixel_values=pix, image_grid_thw=grid_t,
                    position_ids=pos[:, None, :]).logits[0]
    assert float((mine - theirs).abs().max()) < 5e-4
    # text-only input: same as the text path of transformers with ordinary positions
    txt = torch.randint(0, 900, (17,), generator=torch.Generator().manual_seed(9))
    meta2 = VarlenMeta(torch.tensor([0, 17], dtype=torch.int32), "cpu")
    with torch.no_grad():
        a = m.logits(m(txt, torch.arange(17), meta2))
        b = hf(input_ids=txt[None]).logits[0]
    assert float((a - b).abs().max()) < 5e-4
    # round trip through the checkpoint (and the older `visual.*` / `model.*` naming)
    m2 = build_model(ModelConfig.from_hf_config(str(tmp_path)), dtype=torch.float32, seed=7)
    load_hf_weights(m2, str(tmp_path))
    for (n1, p1), (n2, p2) in zip(m.named_parameters(), m2.named_parameters()):
        assert n1 == n2 and torch.equal(p1, p2), n1
    old = [((n[len("model."):] if n.startswith("model.visual.") else n.replace("model.language_model.", "model.")), t)
           for n, t in m.to_hf()]
    m3 = build_model(CFG, dtype=torch.float32, seed=8).load_hf(old)
    assert all(torch.equal(p1, p3) for p1, p3 in zip(m.parameters(), m3.parameters()))


def _vl_items(n=6, seed=0):
    g = torch.Generator().manual_seed(seed)
    items = []
    for i in range(n):
        if i % 3 == 2:  # a text-only sample in the mix
            ids = torch.randint(0, 900, (14,), generator=g).tolist()
            items.append(dict(input_ids=ids, loss_mask=[0] * 8 + [1] * 6))
            continue
        grid = [(1, 4, 4), (1, 4, 6)][i % 2]
        ids, pix = _sample([grid], [4, 6], seed=seed * 100 + i)
        items.append(dict(input_ids=ids, loss_mask=[0] * (len(ids) - 6) + [1] * 6,
                          multi_modal_input=[dict(pixel_values=pix, image_grid_thw=torch.tensor([grid]))]))
    return items


def test_engine_trains_on_images(tmp_path):
    """SFT through the trainer: micro-batches keep each sequence's images, the loss falls, the tower gets
    gradients, and the engine's logprobs equal a direct model call."""
    from areal_b200.api.cli_args import MicroBatchSpec, OptimizerConfig, SFTConfig, TrainEngineConfig, _propagate_names
    from areal_b200.trainer.sl_trainer import SFTTrainer, collate_sft

    data = _vl_items()
    cfg = SFTConfig(actor=TrainEngineConfig(
        backend="fsdp:d1", model_preset="tiny-qwen2_5-vl", init_from_scratch=True, dtype="float32",
        optimizer=OptimizerConfig(lr=2e-3, warmup_steps_proportion=0.0, weight_decay=0.0),
        mb_spec=MicroBatchSpec(max_tokens_per_mb=40)))  # several micro-batches per step
    cfg.experiment_name, cfg.trial_name = "t", "t"
    cfg.cluster.fileroot = str(tmp_path)
    cfg.train_dataset.batch_size = 6
    cfg.train_dataset.shuffle = False
    cfg.total_train_epochs = 6
    _propagate_names(cfg)
    losses = []
    with SFTTrainer(cfg, data, data) as tr:
        eng = tr.engine
        assert isinstance(eng.model, QwenVLModel)
        batch = collate_sft(data)
        assert len(batch["multi_modal_input"]) == 6 and batch["multi_modal_input"][2] == {}
        w0 = eng.model.visual.patch_proj.detach().clone()
        logp = eng.forward(batch)  # [B, L] padded next-token logprobs
        ids, pix = data[1]["input_ids"], data[1]["multi_modal_input"][0]
        meta = VarlenMeta(torch.tensor([0, len(ids)], dtype=torch.int32), "cpu")
        with torch.no_grad():
            h = eng.model(torch.tensor(ids), torch.arange(len(ids)), meta, pixel_values=pix["pixel_values"],
                          image_grid_thw=pix["image_grid_thw"])
            ref = torch.log_softmax(eng.model.logits(h), -1)[:-1].gather(1, torch.tensor(ids)[1:, None])[:, 0]
        assert torch.allclose(logp[1, :len(ids) - 1], ref, atol=1e-4)
        tr.train(max_steps=6, step_callback=lambda s, st: losses.append(st["step/loss"]))
        assert losses[-1] < losses[0]
        assert not torch.equal(eng.model.visual.patch_proj, w0), "the vision tower must train"


def _rollout_engine(device="cpu", preset="tiny-qwen2_5-vl", **over):
    from areal_b200.api.cli_args import InferenceEngineConfig, NativeRolloutConfig
    from areal_b200.engine.rollout_engine import NativeRolloutEngine

    cfg = InferenceEngineConfig(experiment_name="e", trial_name="t", backend="native:d1", max_concurrent_rollouts=16,
                                consumer_batch_size=4,
                                native=NativeRolloutConfig(model_preset=preset, context_length=128,
                                                           max_num_seqs=8, max_num_batched_tokens=512,
                                                           num_kv_blocks=64, seed=3, **over))
    return NativeRolloutEngine(cfg).initialize(**({"device": device} if device == "cpu" else {}))


@pytest.mark.parametrize("preset", ["tiny-qwen2_5-vl", "tiny-qwen3-vl"])
def test_rollout_engine_serves_image_prompts(preset):
    """Greedy generation for a mix of image and text prompts equals re-running the whole model on the growing
    sequence (image features in the prefill, deep-stack features after the first blocks for Qwen3-VL, positions
    after an image offset by the prompt's delta)."""
    import asyncio

    from areal_b200.api.cli_args import GenerationHyperparameters
    from areal_b200.api.io_struct import ModelRequest

    eng = _rollout_engine(preset=preset)
    try:
        assert eng.supports_images
        reqs = []
        for i, grid in enumerate([(1, 4, 6), None, (1, 4, 4), (1, 6, 8)]):
            if grid is None:
                reqs.append((torch.randint(0, 900, (11,), generator=torch.Generator().manual_seed(i)).tolist(), None))
            else:
                ids, pix = _sample([grid], [3 + i, 2], seed=20 + i)
                reqs.append((ids, dict(pixel_values=pix, image_grid_thw=torch.tensor([grid]))))
        gc = GenerationHyperparameters(max_new_tokens=7, greedy=True, ignore_eos=True)

        async def go():
            return await asyncio.gather(*[
                eng.agenerate(ModelRequest(rid=str(i), input_ids=ids, gconfig=gc,
                                           metadata={"multi_modal_input": [mm]} if mm else {}))
                for i, (ids, mm) in enumerate(reqs)])

        outs = asyncio.run(go())
        model = eng.model
        for (p, mm), r in zip(reqs, outs):
            seq = list(p)
            for _ in range(7):
                ids = torch.tensor(seq)
                meta = VarlenMeta(torch.tensor([0, len(seq)], dtype=torch.int32), "cpu")
                with torch.no_grad():
                    h = model(ids, torch.arange(len(seq)), meta, **(mm or {}))
                    seq.append(int(model.logits(h[-1:]).argmax(-1)))
            assert r.output_tokens == seq[len(p):], (r.output_tokens, seq[len(p):])
        assert not eng._mm
        # encoded images need the request's processor
        with pytest.raises(ValueError):
            asyncio.run(eng.agenerate(ModelRequest(rid="x", input_ids=reqs[0][0], gconfig=gc, image_data=["AAAA"])))
    finally:
        eng.destroy()


class _ToyTok:
    eos_token_id = 1023
    pad_token_id = 0

    def decode(self, ids, **kw):
        return " ".join(str(int(i)) for i in ids)


class _ToyVLProcessor:
    """Stands in for the HF processor: the "image" is bytes naming its patch grid (``b"4x6"``), the text is a
    string of token ids in which ``<img>`` marks where the image goes."""

    def __init__(self):
        self.tokenizer = _ToyTok()

    def __call__(self, images=None, text=None, padding=False, return_tensors="pt"):
        ids, grids, pix = [], [], []
        it = iter(images or [])
        for w in text.split():
            if w == "<img>":
                h, wd = (int(x) for x in next(it).decode().split("x"))
                grids.append([1, h, wd])
                g = torch.Generator().manual_seed(h * 100 + wd)
                pix.append(torch.randn(h * wd, 3 * 2 * 14 * 14, generator=g))
                ids += [CFG.vision_start_token_id] + [IMG] * (h * wd // 4) + [CFG.vision_end_token_id]
            else:
                ids.append(int(w))
        out = {"input_ids": torch.tensor([ids]), "attention_mask": torch.ones(1, len(ids), dtype=torch.long)}
        if grids:
            out["pixel_values"] = torch.cat(pix, 0)
            out["image_grid_thw"] = torch.tensor(grids)
        return out


def _even_reward(prompt, completion, prompt_ids, completion_ids, **kw):
    return 1.0 if sum(1 for t in completion_ids if t % 2 == 0) > len(completion_ids) / 2 else 0.0


def test_grpo_step_with_images(tmp_path):
    """Rollout → logprob recomputation → PPO update → weight push, with image prompts, in one process: the
    trajectories keep each sample's images through batching and micro-batch splitting, the recomputed
    logprobs agree with the rollout's, and the rollout engine ends up with the trained vision tower."""
    from areal_b200.api.cli_args import (GenerationHyperparameters, GRPOConfig, InferenceEngineConfig, MicroBatchSpec,
                                         NativeRolloutConfig, NormConfig, OptimizerConfig, PPOActorConfig,
                                         _propagate_names)
    from areal_b200.trainer.rl_trainer import PPOTrainer
    from areal_b200.workflow.vision_rlvr import VisionRLVRWorkflow

    cfg = GRPOConfig(experiment_name="vl", trial_name="t")
    cfg.seed = 0
    cfg.cluster.fileroot = str(tmp_path)
    cfg.train_dataset.batch_size = 4
    cfg.train_dataset.shuffle = False
    cfg.gconfig = GenerationHyperparameters(n_samples=2, max_new_tokens=8, temperature=1.0, ignore_eos=True)
    cfg.actor = PPOActorConfig(backend="fsdp:d1", model_preset="tiny-qwen2_5-vl", init_from_scratch=True,
                               dtype="float32", optimizer=OptimizerConfig(lr=1e-3, warmup_steps_proportion=0.0),
                               mb_spec=MicroBatchSpec(max_tokens_per_mb=64), ppo_n_minibatches=1,
                               reward_norm=NormConfig(mean_level="group", std_level="group", group_size=2),
                               kl_ctl=0.0, use_decoupled_loss=True, recompute_logprob=True)
    cfg.rollout = InferenceEngineConfig(backend="native:d1", max_head_offpolicyness=0, max_concurrent_rollouts=16,
                                        native=NativeRolloutConfig(model_preset="tiny-qwen2_5-vl", context_length=128,
                                                                   max_num_seqs=8, max_num_batched_tokens=512,
                                                                   num_kv_blocks=64, seed=0, dtype="float32"))
    _propagate_names(cfg)
    ds = [dict(prompt=f"{3 + i} 17 <img> 5 {40 + i}", images=[b"4x6" if i % 2 else b"4x4"]) for i in range(7)]
    ds.append(dict(prompt="9 8 7 6 5", images=[]))  # one text-only prompt
    seen = []
    with PPOTrainer(cfg, ds) as tr:
        w0 = tr.actor_engine.model.visual.patch_proj.detach().clone()
        tr.train(workflow=VisionRLVRWorkflow,
                 workflow_kwargs=dict(reward_fn=_even_reward, gconfig=cfg.gconfig, tokenizer=_ToyTok(),
                                      processor=_ToyVLProcessor(), reward_in_process=True),
                 max_steps=2, step_callback=lambda s, st: seen.append(st))
        assert len(seen) == 2 and all(s["step/grad_norm"] > 0 for s in seen)
        assert not torch.equal(tr.actor_engine.model.visual.patch_proj, w0)
        assert torch.equal(tr.rollout.model.visual.patch_proj, tr.actor_engine.model.visual.patch_proj)
        # behaviour logprobs (rollout engine: prefill with image features + decode at offset positions) equal the
        # train engine's recomputation on the finished trajectory
        import asyncio

        wf = VisionRLVRWorkflow(_even_reward, cfg.gconfig.new(n_samples=1), _ToyTok(), _ToyVLProcessor(),
                                reward_in_process=True)
        traj = asyncio.run(wf.arun_episode(tr.rollout, ds[1]))
        n_in = int((traj["loss_mask"][0] == 0).sum())
        logp = tr.actor_engine.forward({k: v for k, v in traj.items() if k != "rewards"})
        L = traj["input_ids"].shape[1]
        assert torch.allclose(logp[0, n_in - 1:L - 1], traj["logprobs"][0, n_in:], atol=1e-4)


def _png(h, w, seed=0):
    import io

    import numpy as np
    from PIL import Image

    rng = np.random.default_rng(seed)
    buf = io.BytesIO()
    Image.fromarray((rng.random((h, w, 3)) * 255).astype("uint8")).save(buf, format="PNG")
    return buf.getvalue()


def test_encoded_images_through_the_hf_image_processor():
    """A request that carries base64 PNGs (what a remote caller sends) is decoded and run through the
    request's processor; the result equals handing over the processor's tensors directly."""
    import asyncio
    import base64
    import io

    transformers = pytest.importorskip("transformers")
    from PIL import Image

    from areal_b200.api.cli_args import GenerationHyperparameters
    from areal_b200.api.io_struct import ModelRequest

    ip = transformers.Qwen2VLImageProcessor(min_pixels=28 * 28, max_pixels=112 * 112)
    png = _png(70, 90)
    direct = ip(images=[Image.open(io.BytesIO(png))], return_tensors="pt")
    t, h, w = direct["image_grid_thw"][0].tolist()
    assert direct["pixel_values"].shape == (t * h * w, 1176)
    ids = [5, 6, CFG.vision_start_token_id] + [IMG] * (t * h * w // 4) + [CFG.vision_end_token_id, 7]
    gc = GenerationHyperparameters(max_new_tokens=5, greedy=True, ignore_eos=True)
    eng = _rollout_engine()
    try:
        a = asyncio.run(eng.agenerate(ModelRequest(rid="a", input_ids=ids, gconfig=gc, processor=ip,
                                                   image_data=[base64.b64encode(png).decode()])))
        b = asyncio.run(eng.agenerate(ModelRequest(rid="b", input_ids=ids, gconfig=gc,
                                                   metadata={"multi_modal_input": [dict(direct)]})))
        assert a.output_tokens == b.output_tokens and a.output_logprobs == pytest.approx(b.output_logprobs, abs=1e-6)
    finally:
        eng.destroy()


def test_clevr_sft_builder(tmp_path):
    """Dataset builder: placeholder expansion by the processor, loss on the answer tokens, pixel tensors kept."""
    import json

    from areal_b200.dataset import get_custom_dataset

    class Tok:
        eos_token = "<eos>"

        def encode(self, text, add_special_tokens=False):
            return [int(w) for w in text.split()]

    class Proc(_ToyVLProcessor):
        def __init__(self):
            self.tokenizer = Tok()

        def __call__(self, text=None, images=None, **kw):
            text = text[0].replace("<|vision_start|><|image_pad|><|vision_end|>", " <img> ").replace("<eos>", " 1023")
            return super().__call__(images=[im.encode() for im in images] if images else None, text=text)

    d = tmp_path / "clevr_count_70k"
    d.mkdir()
    rows = [dict(problem="<image>4 5 6 ", answer="3", images=["4x6"]), dict(problem="7 8 ", answer="2 2", images=[])]
    (d / "train.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    items = get_custom_dataset(path=str(d), type="sft", split="train", processor=Proc())
    a, b = items
    assert a["input_ids"][0] == CFG.vision_start_token_id and a["input_ids"].count(IMG) == 6
    assert a["loss_mask"] == [0] * (len(a["input_ids"]) - 2) + [1, 1] and a["input_ids"][-2:] == [3, 1023]
    assert a["multi_modal_input"][0]["pixel_values"].shape == (24, 1176)
    assert "multi_modal_input" not in b and b["loss_mask"] == [0, 0, 1, 1, 1]
    from areal_b200.trainer.sl_trainer import collate_sft

    batch = collate_sft(items)
    assert batch["input_ids"].shape[0] == 2 and batch["multi_modal_input"][1] == {}


def test_image_prompt_over_http():
    """The HTTP front takes SGLang-style ``image_data`` and the client engine forwards it: same tokens as the
    in-process call."""
    import asyncio
    import base64
    import io
    import socket
    import threading

    transformers = pytest.importorskip("transformers")
    uvicorn = pytest.importorskip("uvicorn")
    from PIL import Image

    from areal_b200.api.cli_args import GenerationHyperparameters, InferenceEngineConfig
    from areal_b200.api.io_struct import ModelRequest
    from areal_b200.engine.native_server import create_app
    from areal_b200.infra.remote_inf_engine import RemoteInfEngine

    ip = transformers.Qwen2VLImageProcessor(min_pixels=28 * 28, max_pixels=112 * 112)
    png = _png(60, 60, seed=2)
    direct = ip(images=[Image.open(io.BytesIO(png))], return_tensors="pt")
    t, h, w = direct["image_grid_thw"][0].tolist()
    ids = [9, CFG.vision_start_token_id] + [IMG] * (t * h * w // 4) + [CFG.vision_end_token_id, 11, 12]
    gc = GenerationHyperparameters(max_new_tokens=6, greedy=True, ignore_eos=True)
    eng = _rollout_engine()
    eng.image_processor = ip
    sock = socket.socket()
    sock.bind(("127.0.0.1", 0))
    port = sock.getsockname()[1]
    sock.close()
    server = uvicorn.Server(uvicorn.Config(create_app(eng), host="127.0.0.1", port=port, log_level="error"))
    th = threading.Thread(target=server.run, daemon=True)
    th.start()
    client = None
    try:
        cfg = InferenceEngineConfig(experiment_name="e", trial_name="t", backend="native:d1", max_concurrent_rollouts=4,
                                    consumer_batch_size=1, setup_timeout=30.0, request_timeout=60.0)
        client = RemoteInfEngine(cfg).initialize(addr=[f"127.0.0.1:{port}"])
        assert client.supports_images
        req = ModelRequest(rid="r", input_ids=ids, gconfig=gc, image_data=[base64.b64encode(png).decode()])
        remote = client.generate(req)
        local = asyncio.run(eng.agenerate(ModelRequest(rid="l", input_ids=ids, gconfig=gc,
                                                       metadata={"multi_modal_input": [dict(direct)]})))
        assert remote.output_tokens == local.output_tokens
    finally:
        if client is not None:
            client.destroy()
        server.should_exit = True
        th.join(timeout=10)
        eng.destroy()


def test_openai_client_with_image_messages():
    """``image_url`` parts of chat messages: the client swaps them for the template's image marker, lets the
    processor expand the placeholders, hands the pixel tensors to the engine and keeps them in the exported
    interaction; batches mix image and text interactions."""
    import asyncio
    import base64

    from areal_b200.api.cli_args import GenerationHyperparameters
    from areal_b200.openai.client import ArealOpenAI, extract_images
    from areal_b200.utils.data import concat_padded_tensors

    png = _png(28, 28)
    uri = "data:image/png;base64," + base64.b64encode(png).decode()
    msgs = [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": uri}},
                                         {"type": "text", "text": "5 6 7"}]}]
    data, tmpl = extract_images(msgs)
    assert data == [base64.b64encode(png).decode()] and tmpl[0]["content"][0] == {"type": "image"}
    assert msgs[0]["content"][0]["type"] == "image_url"  # the caller's messages are not modified

    class Tok(_ToyTok):
        def apply_chat_template(self, messages, tokenize=True, add_generation_prompt=True, **kw):
            return [int(w) for m in messages for w in str(m["content"]).split()]

    class Proc(_ToyVLProcessor):
        def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=True, **kw):
            words = []
            for m in messages:
                for part in m["content"] if isinstance(m["content"], list) else [{"type": "text", "text": m["content"]}]:
                    words.append("<img>" if part["type"] == "image" else part["text"])
            return " ".join(words)

        def __call__(self, text=None, images=None, **kw):
            assert all(im.size == (28, 28) for im in images)  # decoded PIL images arrive here
            return super().__call__(images=[b"4x4"] * len(images), text=text[0])

    eng = _rollout_engine()
    try:
        client = ArealOpenAI(eng, Tok(), GenerationHyperparameters(max_new_tokens=4, greedy=True), processor=Proc())

        async def go():
            a = await client.chat.completions.create(messages=msgs)
            b = await client.chat.completions.create(messages=[{"role": "user", "content": "8 9"}])
            return a, b

        a, b = asyncio.run(go())
        client.set_reward(a.id, 1.0)
        client.set_reward(b.id, 0.0)
        inter = client.export_interactions()
        ta, tb = inter[a.id].to_tensor_dict(), inter[b.id].to_tensor_dict()
        assert ta["multi_modal_input"][0]["pixel_values"].shape == (16, 1176) and "multi_modal_input" not in tb
        assert int((ta["input_ids"] == IMG).sum()) == 4
        for batch in (concat_padded_tensors([ta, tb]), concat_padded_tensors([tb, ta])):
            assert len(batch["multi_modal_input"]) == 2 and sum(bool(d) for d in batch["multi_modal_input"]) == 1
    finally:
        eng.destroy()


def test_load_image_forms(tmp_path):
    from areal_b200.workflow.vision_rlvr import image_to_base64, load_image

    png = _png(20, 30)
    (tmp_path / "a.png").write_bytes(png)
    for obj in (png, {"bytes": png, "path": None}, {"bytes": None, "path": str(tmp_path / "a.png")}, str(tmp_path / "a.png")):
        im = load_image(obj)
        assert im.size == (30, 20) and im.mode == "RGB"
    assert load_image(im) is im and load_image(b"not an image") == b"not an image"
    assert load_image(image_to_base64(im).encode(), decode_bytes=False) == image_to_base64(im).encode()


def test_group_samples_share_one_tower_pass():
    """The samples of a group carry the same image: the rollout engine runs the vision tower once per distinct
    image set (keyed by content) and drops the cached features when the weights change."""
    import asyncio

    from areal_b200.api.cli_args import GenerationHyperparameters
    from areal_b200.api.io_struct import ModelRequest

    eng = _rollout_engine(preset="tiny-qwen3-vl")
    try:
        ids, pix = _sample([(1, 4, 6)], [3, 2], seed=5)
        ids2, pix2 = _sample([(1, 4, 4)], [2, 2], seed=6)
        gc = GenerationHyperparameters(max_new_tokens=4, greedy=True, ignore_eos=True)

        def req(i, ids, pix, grid):
            # every request gets its own copy of the tensors, as separate processor calls produce
            return ModelRequest(rid=str(i), input_ids=ids, gconfig=gc, metadata={"multi_modal_input": [
                dict(pixel_values=pix.clone(), image_grid_thw=torch.tensor([grid]))]})

        async def go():
            return await asyncio.gather(*[eng.agenerate(req(i, ids, pix, (1, 4, 6))) for i in range(4)],
                                        eng.agenerate(req(9, ids2, pix2, (1, 4, 4))))

        outs = asyncio.run(go())
        assert eng.vision_tower_images == 2 and len(eng._vis_cache) == 2
        assert all(o.output_tokens == outs[0].output_tokens for o in outs[:4])
        again = asyncio.run(eng.agenerate(req(10, ids, pix, (1, 4, 6))))
        assert eng.vision_tower_images == 2 and again.output_tokens == outs[0].output_tokens
        eng.pause_generation()
        eng.continue_generation()
        assert not eng._vis_cache
        asyncio.run(eng.agenerate(req(11, ids, pix, (1, 4, 6))))
        assert eng.vision_tower_images == 3
    finally:
        eng.destroy()


def test_trainer_checkpoint_carries_tokenizer_and_processor(tmp_path):
    """A saved vision-language checkpoint is complete: weights, composite config, and the tokenizer's and
    processor's own files."""
    import os

    from areal_b200.api.cli_args import MicroBatchSpec, OptimizerConfig, SFTConfig, TrainEngineConfig, _propagate_names
    from areal_b200.trainer.sl_trainer import SFTTrainer

    class Saves:
        def __init__(self, fname):
            self.fname = fname

        def save_pretrained(self, path):
            open(os.path.join(path, self.fname), "w").write("{}")

    cfg = SFTConfig(actor=TrainEngineConfig(backend="fsdp:d1", model_preset="tiny-qwen2_5-vl", init_from_scratch=True,
                                            dtype="float32", optimizer=OptimizerConfig(lr=1e-3),
                                            mb_spec=MicroBatchSpec(max_tokens_per_mb=128)))
    cfg.experiment_name, cfg.trial_name = "t", "t"
    cfg.cluster.fileroot = str(tmp_path)
    cfg.train_dataset.batch_size = 6
    cfg.total_train_epochs = 1
    cfg.saver.freq_steps = 1
    _propagate_names(cfg)
    with SFTTrainer(cfg, _vl_items(), None, tokenizer=Saves("tokenizer_config.json"),
                    processor=Saves("preprocessor_config.json")) as tr:
        tr.train(max_steps=1)
    found = [os.path.join(d, f) for d, _, fs in os.walk(tmp_path) for f in fs]
    names = {os.path.basename(f) for f in found}
    assert {"model.safetensors", "config.json", "tokenizer_config.json", "preprocessor_config.json"} <= names
    ckpt = os.path.dirname(next(f for f in found if f.endswith("model.safetensors")))
    assert ModelConfig.from_hf_config(ckpt).is_vl


@pytest.mark.parametrize("preset", ["tiny-qwen2_5-vl", "tiny-qwen2-vl", "tiny-qwen3-vl", "tiny-qwen3-vl-moe"])
def test_parameter_count_includes_the_tower(preset):
    cfg = PRESETS[preset]
    m = build_model(cfg, dtype=torch.float32, seed=None)
    assert cfg.num_params() == sum(p.numel() for p in m.parameters()) and cfg.vision_params() > 0


def test_lora_on_the_decoder_of_a_vision_language_model(tmp_path):
    """Adapters on the decoder's projections, tower and base weights frozen; the adapter checkpoint names the
    decoder where PEFT finds it in a vision-language model."""
    import json
    import os

    from safetensors.torch import load_file

    from areal_b200.api.cli_args import MicroBatchSpec, OptimizerConfig, SFTConfig, TrainEngineConfig, _propagate_names
    from areal_b200.api.io_struct import SaveLoadMeta
    from areal_b200.trainer.sl_trainer import SFTTrainer

    cfg = SFTConfig(actor=TrainEngineConfig(backend="fsdp:d1", model_preset="tiny-qwen2_5-vl", init_from_scratch=True,
                                            dtype="float32", use_lora=True, lora_rank=4, lora_alpha=8,
                                            target_modules=["q_proj", "v_proj", "down_proj"],
                                            optimizer=OptimizerConfig(lr=1e-2, warmup_steps_proportion=0.0,
                                                                      weight_decay=0.0),
                                            mb_spec=MicroBatchSpec(max_tokens_per_mb=128)))
    cfg.experiment_name, cfg.trial_name = "t", "t"
    cfg.cluster.fileroot = str(tmp_path)
    cfg.train_dataset.batch_size = 6
    cfg.train_dataset.shuffle = False
    cfg.total_train_epochs = 5
    _propagate_names(cfg)
    losses = []
    with SFTTrainer(cfg, _vl_items(), None) as tr:
        eng = tr.engine
        tower0 = eng.model.visual.patch_proj.detach().clone()
        tr.train(max_steps=5, step_callback=lambda s, st: losses.append(st["step/loss"]))
        assert losses[-1] < losses[0]
        assert torch.equal(eng.model.visual.patch_proj, tower0), "the tower is part of the frozen base"
        path = str(tmp_path / "ckpt")
        eng.save(SaveLoadMeta(path=path, weight_format="hf", with_optim=False))
        ad = load_file(os.path.join(path, "adapter_model.safetensors"))
        assert "base_model.model.model.language_model.layers.0.self_attn.q_proj.lora_A.weight" in ad
        assert json.load(open(os.path.join(path, "adapter_config.json")))["r"] == 4
        assert ModelConfig.from_hf_config(path).is_vl  # the merged model next to it is a full VL checkpoint
