"""Smaller components that the larger tests only touch indirectly: the asynchronous reward wrapper
(timeouts, exceptions, a dying worker), the frequency-gated evaluator, the preference / tool-reasoning
dataset builders (jsonl, json and parquet sources), and the installation validator."""
import asyncio
import json
import os
import time

import pytest

from areal_b200.api.cli_args import EvaluatorConfig
from areal_b200.api.io_struct import FinetuneSpec
from areal_b200.api.reward_api import AsyncRewardWrapper
from areal_b200.dataset import get_custom_dataset
from areal_b200.utils.evaluator import Evaluator


def _ok(a, b=1):
    return a * b


def _slow(x):
    time.sleep(5)
    return x


def _raises(x):
    raise ValueError("bad sample")


def _dies(flag_path):
    """Kills its worker process the first time, answers the second time (pool rebuilt in between)."""
    if not os.path.exists(flag_path):
        open(flag_path, "w").close()
        os._exit(1)
    return 7.0


def test_async_reward_wrapper_ok_timeout_exception_and_broken_pool(tmp_path):
    async def go():
        assert await AsyncRewardWrapper(_ok, max_workers=2)(3, b=2) == 6.0
        t0 = time.time()
        assert await AsyncRewardWrapper(_slow, timeout_seconds=0.3, max_workers=2, default=-1.0)(1) == -1.0
        assert time.time() - t0 < 4
        assert await AsyncRewardWrapper(_raises, max_workers=2, default=0.5)(1) == 0.5
        assert await AsyncRewardWrapper(_dies, max_workers=3, max_retries=2)(str(tmp_path / "flag")) == 7.0

    asyncio.run(go())


def test_evaluator_frequency_and_state():
    calls = []
    ev = Evaluator(EvaluatorConfig(freq_steps=3), FinetuneSpec(total_train_epochs=2, dataset_size=40, train_batch_size=4))
    fired = [ev.evaluate(lambda: calls.append(1), 0, s, s) for s in range(7)]
    assert fired == [False, False, True, False, False, True, False] and len(calls) == 2
    ev2 = Evaluator(EvaluatorConfig(freq_steps=3))
    ev2.load_state_dict(ev.state_dict())
    assert [ev2.evaluate(lambda: None, 0, 7, 7), ev2.evaluate(lambda: None, 0, 8, 8)] == [False, True]
    ev3 = Evaluator(EvaluatorConfig(freq_epochs=1), FinetuneSpec(total_train_epochs=2, dataset_size=8, train_batch_size=4))
    assert [ev3.evaluate(lambda: None, 0, s, s) for s in range(2)] == [False, True]  # last step of the epoch


class _Tok:
    eos_token_id = 2

    def encode(self, text, add_special_tokens=True):
        return [3 + (ord(c) % 50) for c in text]


def test_preference_and_tool_datasets(tmp_path):
    d = tmp_path / "hh-rlhf"
    d.mkdir()
    rows = [dict(chosen="\n\nHuman: hi\n\nAssistant: hello there", rejected="\n\nHuman: hi\n\nAssistant: go away"),
            dict(chosen="\n\nHuman: 2+2?\n\nAssistant: 4", rejected="\n\nHuman: 2+2?\n\nAssistant: 5" + "!" * 400)]
    with open(d / "train.jsonl", "w") as f:
        f.writelines(json.dumps(r) + "\n" for r in rows)
    pairs = get_custom_dataset(str(d), type="dpo", tokenizer=_Tok())
    assert len(pairs) == 2
    p = pairs[0]
    n_prompt = p["chosen_loss_mask"].index(1)
    assert p["chosen_ids"][:n_prompt] == p["rejected_ids"][:n_prompt]  # shared prompt, masked out
    assert p["chosen_ids"][-1] == p["rejected_ids"][-1] == 2 and sum(p["rejected_loss_mask"]) == len("go away") + 2
    assert len(get_custom_dataset(str(d), type="rw", tokenizer=_Tok(), max_length=100)) == 1  # the long pair is dropped
    # ToRL-style records from a json file with a split key, and from parquet
    t = tmp_path / "torl"
    t.mkdir()
    recs = [dict(prompt=[{"role": "user", "content": "1+1"}], reward_model={"ground_truth": "2"}),
            dict(question="3*3", answer="9")]
    json.dump({"train": recs}, open(t / "train.json", "w"))
    out = get_custom_dataset(str(t), type="rl")
    assert out[0]["answer"] == "2" and out[1]["messages"][0]["content"] == "3*3" and out[1]["answer"] == "9"
    import pyarrow as pa
    import pyarrow.parquet as pq

    os.remove(t / "train.json")
    pq.write_table(pa.Table.from_pylist([dict(question="5-1", answer="4")]), t / "train.parquet")
    assert get_custom_dataset(str(t), type="rl")[0]["answer"] == "4"
    with pytest.raises(ValueError):
        get_custom_dataset(str(tmp_path / "unknown-set"), type="rl")


def test_validate_installation_reports_success_on_cpu(capsys):
    from areal_b200.tools import validate_installation

    rc = validate_installation.main(["--no-build"])
    out = capsys.readouterr().out
    assert rc == 0, out
    assert "import torch" in out


def test_determinism_switches_set_and_clear():
    """``megatron.use_deterministic_algorithms``: fixed NCCL algorithm, cuBLAS workspace, PyTorch's deterministic
    operators, and the library's flag that routes the two atomically-summing kernels to ordered paths."""
    import os

    import torch

    from areal_b200.utils import determinism

    old = {k: os.environ.get(k) for k in ("NCCL_ALGO", "CUBLAS_WORKSPACE_CONFIG")}
    try:
        os.environ.pop("NCCL_ALGO", None)
        determinism.set_deterministic_algorithms(True)
        assert determinism.deterministic_mode() and torch.are_deterministic_algorithms_enabled()
        assert os.environ["NCCL_ALGO"] == "Ring" and os.environ["CUBLAS_WORKSPACE_CONFIG"] in (":4096:8", ":16:8")
    finally:
        determinism.set_deterministic_algorithms(False)
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
    assert not determinism.deterministic_mode() and not torch.are_deterministic_algorithms_enabled()


def test_activation_checkpoint_policies_keep_gradients_identical():
    """none / full / selective (every N-th block, or the MLP half of every block) / memory budget: the same
    gradients, bit for bit on CPU, whichever parts are recomputed."""
    import torch

    from areal_b200.models.activation_checkpoint import apply_activation_checkpointing, make_policy
    from areal_b200.models.config import PRESETS
    from areal_b200.models.qwen import build_model
    from areal_b200.ops.attention import VarlenMeta

    assert make_policy(6, "selective", 2).full_layers == {0, 2, 4}
    assert make_policy(6, "selective", "op").mlp_only and not make_policy(6, "selective", "op").full_layers
    assert make_policy(8, "memory_budget", budget=0.25).full_layers == set(range(6))
    assert not make_policy(8, "memory_budget", budget=1.0).active and make_policy(4, "full").full_layers == {0, 1, 2, 3}
    import pytest

    with pytest.raises(ValueError):
        make_policy(4, "sometimes")
    model = build_model(PRESETS["tiny-qwen2-4l"], dtype=torch.float32, device="cpu", seed=1)
    ids = torch.randint(0, 1000, (50,))
    pos = torch.cat([torch.arange(30), torch.arange(20)])
    meta = VarlenMeta([0, 30, 50], torch.device("cpu"))
    grads = {}
    for mode, opt, budget in (("none", "op", 0.5), ("full", "op", 0.5), ("selective", 2, 0.5), ("selective", "op", 0.5),
                              ("memory_budget", "op", 0.4)):
        apply_activation_checkpointing(model, mode, opt, budget)
        model.zero_grad()
        model.train()
        h = model(ids, pos, meta)
        model.logits(h).float().square().mean().backward()
        grads[(mode, opt)] = torch.cat([p.grad.flatten() for p in model.parameters() if p.grad is not None])
    base = grads[("none", "op")]
    assert base.abs().sum() > 0
    for k, g in grads.items():
        assert torch.equal(g, base), k


def test_kv_name_resolve_against_a_fake_etcd_client():
    """The etcd3 / Ray repositories speak to their service through five calls; a fake with those calls stands in."""
    import pytest

    from areal_b200.utils import name_resolve as nr

    class Meta:
        def __init__(self, key):
            self.key = key.encode()

    class Lease:
        def __init__(self):
            self.refreshed, self.revoked = 0, False

        def refresh(self):
            self.refreshed += 1

        def revoke(self):
            self.revoked = True

    class FakeEtcd:
        def __init__(self):
            self.d, self.leases = {}, []

        def put(self, k, v, lease=None):
            self.d[k] = v.encode()

        def get(self, k):
            return self.d.get(k), None

        def get_prefix(self, p):
            return [(v, Meta(k)) for k, v in self.d.items() if k.startswith(p)]

        def delete(self, k):
            self.d.pop(k, None)

        def lease(self, ttl):
            self.leases.append(Lease())
            return self.leases[-1]

    client = FakeEtcd()
    repo = nr.KVNameRecordRepository(client, keepalive_interval=0.01)
    repo.add("exp/trial/servers/a", "host:1", keepalive_ttl=2)
    repo.add("exp/trial/servers/b", "host:2")
    repo.add("exp/trial/serversX", "other")
    with pytest.raises(nr.NameEntryExistsError):
        repo.add("exp/trial/servers/a", "again")
    repo.add("exp/trial/servers/a", "host:9", replace=True)
    assert repo.get("exp/trial/servers/a") == "host:9"
    assert repo.get_subtree("exp/trial/servers") == ["host:9", "host:2"]          # the sibling prefix is not a child
    assert repo.find_subtree("exp/trial/servers") == ["exp/trial/servers/a", "exp/trial/servers/b"]
    import time

    time.sleep(0.05)
    assert client.leases[0].refreshed > 0
    repo.delete("exp/trial/servers/b")
    with pytest.raises(nr.NameEntryNotFoundError):
        repo.get("exp/trial/servers/b")
    repo.reset()
    assert client.d == {} and all(l.revoked for l in client.leases)
    with pytest.raises(ImportError):
        nr.Etcd3NameRecordRepository("localhost:2379")
