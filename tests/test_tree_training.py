"""Tree training in the engine: trie-packed forward/backward equals the packed varlen path."""
import pytest
import torch

from areal_b200.api.cli_args import MicroBatchSpec, OptimizerConfig, TrainEngineConfig
from areal_b200.engine.train_engine import B200TrainEngine
from areal_b200.utils import stats_tracker


def _engine(tree: bool, device="cpu", dtype="float32"):
    cfg = TrainEngineConfig(backend="fsdp:d1", model_preset="tiny-qwen2", init_from_scratch=True, dtype=dtype,
                            optimizer=OptimizerConfig(type="sgd", lr=0.1, warmup_steps_proportion=0.0, weight_decay=0.0,
                                                      gradient_clipping=0.0),  # weights move by lr * grad: compares gradients
                            mb_spec=MicroBatchSpec(max_tokens_per_mb=4096), enable_tree_training=tree)
    eng = B200TrainEngine(cfg)
    eng.create_process_group()
    eng.initialize(None, None, **({"device": device} if device != "cpu" else {}))
    return eng


def _batch(seed=0, n_prompts=3, group=4, plen=20, rlen=(5, 30)):
    """GRPO-shaped batch: `group` responses per prompt share the prompt and often a few more tokens."""
    g = torch.Generator().manual_seed(seed)
    seqs, masks = [], []
    for _ in range(n_prompts):
        prompt = torch.randint(0, 1024, (plen,), generator=g).tolist()
        common = torch.randint(0, 1024, (4,), generator=g).tolist()
        for k in range(group):
            n = int(torch.randint(rlen[0], rlen[1], (1,), generator=g))
            resp = (common if k % 2 == 0 else []) + torch.randint(0, 1024, (n,), generator=g).tolist()
            seqs.append(prompt + resp)
            masks.append([0] * plen + [1] * len(resp))
    L = max(map(len, seqs))
    B = len(seqs)
    ids = torch.zeros(B, L, dtype=torch.long)
    am = torch.zeros(B, L, dtype=torch.bool)
    lm = torch.zeros(B, L, dtype=torch.long)
    for i, (s, m) in enumerate(zip(seqs, masks)):
        ids[i, :len(s)] = torch.tensor(s)
        am[i, :len(s)] = True
        lm[i, :len(s)] = torch.tensor(m)
    return dict(input_ids=ids, attention_mask=am, loss_mask=lm)


def _loss(logp, ent, mb):
    m = torch.roll(mb["loss_mask"], -1, 0).float()
    return -(logp * m).sum() / m.sum().clamp(min=1) + 0.01 * (ent * m).sum() / m.sum().clamp(min=1)


def _weight(mb):
    return torch.roll(mb["loss_mask"], -1, 0).float().sum()


def _compare(device, dtype, tol):
    batch = _batch()
    plain, tree = _engine(False, device, dtype), _engine(True, device, dtype)
    try:
        lp0, e0 = plain.forward_batch(batch, return_entropy=True)
        lp1, e1 = tree.forward_batch(batch, return_entropy=True)
        # compare where a label exists: every position but the last of each sequence
        valid = batch["attention_mask"].clone()
        lens = valid.sum(1)
        valid[torch.arange(valid.shape[0]), lens - 1] = False
        assert float((lp0 - lp1)[valid].abs().max()) < tol
        assert float((e0 - e1)[valid].abs().max()) < tol
        assert float(lp1[~valid].abs().max()) == 0.0
        ratio = stats_tracker.export().get("tree/node_ratio")
        assert ratio is not None and ratio < 0.75  # 3 prompts x 4 samples share 20-token prompts
        plain_w0 = plain.flat.flat.float().clone()
        s0 = plain.train_batch(batch, _loss, _weight)
        s1 = tree.train_batch(batch, _loss, _weight)
        assert s0["grad_norm"] == pytest.approx(s1["grad_norm"], rel=max(tol, 1e-4))
        w0, w1 = plain.flat.flat.float(), tree.flat.flat.float()
        assert float((w0 - w1).abs().max()) < (2e-2 if dtype == "bfloat16" else 1e-5)
        assert float((w0 - plain_w0).abs().max()) > 1e-3  # the step did move the weights
    finally:
        plain.destroy()
        tree.destroy()


def test_tree_training_matches_packed_cpu():
    _compare("cpu", "float32", 2e-4)


@pytest.mark.gpu
def test_tree_training_matches_packed_cuda():
    _compare("cuda", "bfloat16", 0.08)
