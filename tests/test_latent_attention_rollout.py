"""The rollout engine serves latent-attention (DeepSeek-V3 family) models (expanded keys and padded values in the
paged cache, grouped sigmoid routing in its MoE layers) and the Bailing hybrid (a recurrent state per sequence for
the lightning layers). Greedy continuations must be the ones a full forward of the same model picks token by
token."""
import asyncio

import pytest
import torch

from areal_b200.ops.attention import VarlenMeta


def test_rollout_engine_serves_the_deepseek_v3_family_on_cpu():
    from areal_b200.api.cli_args import GenerationHyperparameters, InferenceEngineConfig, NativeRolloutConfig
    from areal_b200.api.io_struct import ModelRequest
    from areal_b200.engine.rollout_engine import NativeRolloutEngine

    cfg = InferenceEngineConfig(experiment_name="e", trial_name="t", backend="native:d1", max_concurrent_rollouts=16,
                                consumer_batch_size=4,
                                native=NativeRolloutConfig(model_preset="tiny-deepseek-v3", context_length=128,
                                                           max_num_seqs=8, max_num_batched_tokens=512,
                                                           num_kv_blocks=64, seed=3, cuda_graph=False))
    eng = NativeRolloutEngine(cfg).initialize(device="cpu")
    try:
        mc = eng.model_config
        # the cache holds full-width keys / padded values of every head
        assert tuple(eng.kv_caches[0][0].shape[1::2]) == (mc.num_attention_heads, mc.qk_nope_head_dim + mc.qk_rope_head_dim)
        with torch.no_grad():   # a selection bias that changes which experts win
            for layer in eng.model.layers:
                if getattr(layer.mlp, "expert_bias", None) is not None:
                    layer.mlp.expert_bias.copy_(torch.randn(mc.num_experts, generator=torch.Generator().manual_seed(1)) * 0.2)
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
            # and the reported log-probabilities are those of the full forward
            ids = torch.tensor(seq)
            with torch.no_grad():
                h = model(ids, torch.arange(len(seq)), VarlenMeta(torch.tensor([0, len(seq)], dtype=torch.int32), "cpu"))
                lp = torch.log_softmax(model.logits(h).float(), -1)
            want = lp[len(p) - 1:-1].gather(1, ids[len(p):, None]).squeeze(1)
            assert float((torch.tensor(r.output_logprobs) - want).abs().max()) < 1e-3
    finally:
        eng.destroy()


def test_rollout_engine_serves_the_bailing_hybrid_on_cpu():
    """Lightning layers keep a recurrent state per running sequence (left by the prefill, advanced by every decode
    step), latent-attention layers use the paged cache; sequences join and leave the batch at different times."""
    from areal_b200.api.cli_args import GenerationHyperparameters, InferenceEngineConfig, NativeRolloutConfig
    from areal_b200.api.io_struct import ModelRequest
    from areal_b200.engine.rollout_engine import NativeRolloutEngine

    cfg = InferenceEngineConfig(experiment_name="e", trial_name="t", backend="native:d1", max_concurrent_rollouts=16,
                                consumer_batch_size=4,
                                native=NativeRolloutConfig(model_preset="tiny-bailing-hybrid", context_length=160,
                                                           max_num_seqs=4, max_num_batched_tokens=512,
                                                           num_kv_blocks=64, seed=3, cuda_graph=False))
    eng = NativeRolloutEngine(cfg).initialize(device="cpu")
    try:
        assert eng.kv_caches[0] is None and eng.kv_caches[1] is not None           # lightning, latent, ...
        assert eng.hybrid_state.rec[0].shape[1:] == (4, 32, 32) and eng.hybrid_state.rec[1] is None
        g = torch.Generator().manual_seed(7)
        # six requests through four state slots: slots are reused, and one prompt is longer than the
        # recurrence's chunk
        prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (5, 19, 2, 33, 70, 11)]
        lens = [9, 4, 12, 6, 5, 9]

        async def go():
            return await asyncio.gather(*[eng.agenerate(ModelRequest(
                rid=str(i), input_ids=p, gconfig=GenerationHyperparameters(max_new_tokens=n, greedy=True, ignore_eos=True)))
                for i, (p, n) in enumerate(zip(prompts, lens))])

        outs = asyncio.run(go())
        model = eng.model
        for p, n, r in zip(prompts, lens, outs):
            seq = list(p)
            for _ in range(n):
                ids = torch.tensor(seq)
                meta = VarlenMeta(torch.tensor([0, len(seq)], dtype=torch.int32), "cpu")
                with torch.no_grad():
                    h = model(ids, torch.arange(len(seq)), meta)
                    seq.append(int(model.logits(h[-1:]).argmax(-1)))
            assert r.output_tokens == seq[len(p):], (r.output_tokens, seq[len(p):])
        assert not eng._state_slot and len(eng._free_state_slots) == 4
    finally:
        eng.destroy()
