"""Async task runner and workflow executor (staleness gate, accept/reject, ordering)."""
import asyncio
import threading
import time

import pytest
import torch

from areal_b200.api.cli_args import InferenceEngineConfig
from areal_b200.api.workflow_api import RolloutWorkflow
from areal_b200.infra.async_task_runner import AsyncTaskRunner, TaskQueueFullError
from areal_b200.infra.workflow_executor import (GroupedRolloutWorkflow, WorkflowExecutor, check_trajectory_format,
                                                resolve_workflow)


def test_runner_submit_wait_pause_and_failures():
    r = AsyncTaskRunner(max_queue_size=4)
    r.initialize()

    async def work(x, delay=0.0):
        await asyncio.sleep(delay)
        if x < 0:
            raise ValueError("boom")
        return x * 2

    ids = [r.submit(work, i) for i in range(3)]
    got = sorted(x.data for x in r.wait(3, timeout=5))
    assert got == [0, 2, 4] and len(set(ids)) == 3
    r.pause()
    r.submit(work, 5)
    time.sleep(0.1)
    assert r.get_output_queue_size() == 0 and r.get_input_queue_size() == 1
    with pytest.raises(TimeoutError):
        r.wait(1, timeout=0.1)
    r.resume()
    assert r.wait(1, timeout=5)[0].data == 10
    r.submit(work, -1)
    res = r.wait(1, timeout=5)[0]
    assert res.data is None and isinstance(res.error, ValueError)
    r.pause()
    for i in range(4):
        r.submit(work, i)
    with pytest.raises(TaskQueueFullError):
        r.submit(work, 9)
    r.destroy()
    with pytest.raises(RuntimeError):
        r.submit(work, 1)


class FakeEngine:
    def __init__(self):
        self.version = 0

    def get_version(self):
        return self.version


class CountingWorkflow(RolloutWorkflow):
    started = 0
    lock = threading.Lock()

    def __init__(self, reject_odd=False, delay=0.01):
        self.reject_odd, self.delay = reject_odd, delay

    async def arun_episode(self, engine, data):
        with CountingWorkflow.lock:
            CountingWorkflow.started += 1
        await asyncio.sleep(self.delay)
        if self.reject_odd and data["i"] % 2:
            return None
        n = 3 + data["i"] % 3
        return dict(input_ids=torch.full((1, n), data["i"]), attention_mask=torch.ones(1, n, dtype=torch.bool),
                    rewards=torch.tensor([float(data["i"])]), versions=torch.full((1, n), engine.get_version()))


def _executor(bs=4, eta=0, conc=64):
    eng = FakeEngine()
    cfg = InferenceEngineConfig(backend="native:d1", consumer_batch_size=bs, max_head_offpolicyness=eta,
                                max_concurrent_rollouts=conc)
    ex = WorkflowExecutor(cfg, eng).initialize()
    return eng, ex


def test_executor_staleness_gate_blocks_until_version_advances():
    CountingWorkflow.started = 0
    eng, ex = _executor(bs=4, eta=1)
    for i in range(20):
        ex.submit({"i": i}, CountingWorkflow)
    b1 = ex.wait(4, timeout=10)
    b2 = ex.wait(4, timeout=10)
    assert b1["input_ids"].shape[0] == 4 and b2["rewards"].shape == (4,)
    time.sleep(0.2)
    # (eta + version + 1) * bs = 8 episodes may start at version 0
    assert CountingWorkflow.started == 8
    assert ex.wait(1, timeout=0.2, raise_timeout=False) is None
    eng.version = 1
    b3 = ex.wait(4, timeout=10)
    assert (b3["versions"].max() == 1) and CountingWorkflow.started == 12
    st = ex.export_stats()
    assert st["rollout/accepted"] == 12 and st["rollout/enqueued"] == 8
    ex.destroy()


def test_executor_rejection_and_should_accept():
    eng, ex = _executor(bs=2, eta=100)
    for i in range(8):
        ex.submit({"i": i}, CountingWorkflow, workflow_kwargs=dict(reject_odd=True),
                  should_accept_fn=lambda t: float(t["rewards"][0]) != 4.0)
    out = ex.wait(3, timeout=10)
    assert sorted(out["rewards"].tolist()) == [0.0, 2.0, 6.0]
    time.sleep(0.1)
    st = ex.export_stats()
    assert st["rollout/accepted"] == 3 and st["rollout/rejected"] == 5 and st["rollout/running"] == 0
    ex.destroy()


def test_rollout_batch_group_and_wait_for_task():
    eng, ex = _executor(bs=2, eta=100)
    out = ex.rollout_batch([{"i": 1}, {"i": 2}], CountingWorkflow, group_size=3)
    assert out["input_ids"].shape[0] == 6 and out["attention_mask"].shape == out["input_ids"].shape
    tid = ex.submit({"i": 5}, CountingWorkflow())
    assert ex.wait_for_task(tid, timeout=5)["rewards"].tolist() == [5.0]
    ex.destroy()


def test_workflow_resolution_forms():
    wf = resolve_workflow("tests.test_async_runtime.CountingWorkflow", dict(delay=0.0))
    assert isinstance(wf, CountingWorkflow)
    assert isinstance(resolve_workflow(CountingWorkflow, None, group_size=2), GroupedRolloutWorkflow)
    inst = CountingWorkflow()
    assert resolve_workflow(inst, None) is inst
    with pytest.raises(TypeError):
        resolve_workflow(object(), None)


def test_trajectory_format_checks():
    ok = dict(input_ids=torch.zeros(2, 5, dtype=torch.long), attention_mask=torch.ones(2, 5, dtype=torch.bool),
              rewards=torch.zeros(2))
    assert check_trajectory_format(ok) and check_trajectory_format(None)
    with pytest.raises(ValueError):
        check_trajectory_format({"input_ids": torch.zeros(2, 5)})
    with pytest.raises(ValueError):
        check_trajectory_format(dict(ok, rewards=torch.zeros(3)))
    with pytest.raises(ValueError):
        check_trajectory_format(dict(ok, logprobs=torch.zeros(2, 4)))
    with pytest.raises(ValueError):
        check_trajectory_format([1, 2])


def test_scheduler_shares_prompt_pages_between_identical_prompts():
    """n samples of one prompt: the first prefills, the others reference its full prompt pages, get
    a private copy of the tail page and start decoding from the last prompt token."""
    import numpy as np

    from areal_b200.engine.rollout_engine import PagedScheduler

    bs = 16
    s = PagedScheduler(num_blocks=64, block_size=bs, max_num_seqs=16, max_batched_tokens=4096, max_blocks_per_seq=8)
    prompt = list(range(100, 140))  # 40 tokens: 2 full pages + 8 tokens in the third
    other = list(range(500, 520))
    ids = [s.add(prompt, 4, 0, [], True) for _ in range(3)] + [s.add(other, 4, 0, [], True)]
    free0 = s.stats()["free_blocks"]
    assert s.plan() == 1  # prefill: the leader and the unrelated prompt; the two followers wait one step
    assert s.hdr.n_seqs == 2 and s.hdr.n_tokens == 60 and s.hdr.n_copies == 0
    s.commit(np.array([7, 8], dtype=np.int32), np.zeros(2, dtype=np.float32))
    assert s.plan() == 2  # decode: the followers forked in, no second prefill
    assert s.hdr.n_copies == 2 and s.hdr.n_seqs == 4
    st = s.stats()
    assert st["prompt_forks"] == 2 and st["shared_pages"] == 4
    n = s.hdr.n_seqs
    rows = s.block_table[: n * 8].reshape(n, 8)
    order = s.seq_ids[:n].tolist()
    lead, f1, f2 = (rows[order.index(i)] for i in ids[:3])
    assert (lead[:2] == f1[:2]).all() and (lead[:2] == f2[:2]).all()       # full prompt pages are shared
    assert len({int(lead[2]), int(f1[2]), int(f2[2])}) == 3                 # the tail page is private
    pairs = s.copy_pairs[:4].reshape(2, 2)
    assert set(pairs[:, 0].tolist()) == {int(lead[2])} and set(pairs[:, 1].tolist()) == {int(f1[2]), int(f2[2])}
    # followers decode the LAST PROMPT TOKEN at position 39 with a context of 40; the leader is one token ahead
    for i, want_tok, want_pos in ((ids[0], 7, 40), (ids[1], 139, 39), (ids[2], 139, 39)):
        j = order.index(i)
        assert int(s.tokens[j]) == want_tok and int(s.positions[j]) == want_pos and int(s.seq_lens[j]) == want_pos + 1
        assert int(s.slots[j]) == int(rows[j][want_pos // bs]) * bs + want_pos % bs
    # run everything to completion: every page comes back exactly once
    for _ in range(6):
        k = s.plan()
        if k == 0:
            break
        s.commit(np.full(s.hdr.n_seqs, 9, dtype=np.int32), np.zeros(s.hdr.n_seqs, dtype=np.float32))
    while s.pop_finished() is not None:
        pass
    assert s.stats()["free_blocks"] == free0 and s.stats()["live"] == 0
    # sharing can be switched off
    s.set_prompt_sharing(False)
    for _ in range(2):
        s.add(prompt, 1, 0, [], True)
    assert s.plan() == 1 and s.hdr.n_seqs == 2
    s.close()


def test_engine_prompt_sharing_does_not_change_greedy_outputs():
    """Greedy decoding of several copies of two prompts: with prompt sharing (followers skip their
    prefill and read the leader's pages) every copy must produce exactly the tokens it produces with
    sharing switched off, and the same logprobs."""
    import asyncio

    from areal_b200.api.cli_args import GenerationHyperparameters, InferenceEngineConfig, NativeRolloutConfig
    from areal_b200.api.io_struct import ModelRequest
    from areal_b200.engine.rollout_engine import NativeRolloutEngine

    def run(share: bool):
        cfg = InferenceEngineConfig(experiment_name="e", trial_name="t", backend="native:d1", max_concurrent_rollouts=64,
                                    consumer_batch_size=8,
                                    native=NativeRolloutConfig(model_preset="tiny-qwen2", context_length=128, max_num_seqs=16,
                                                               max_num_batched_tokens=1024, num_kv_blocks=128, seed=0,
                                                               cuda_graph=False))
        eng = NativeRolloutEngine(cfg).initialize(device="cpu")
        eng.sched.set_prompt_sharing(share)
        g = torch.Generator().manual_seed(5)
        prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (37, 16)]
        gc = GenerationHyperparameters(max_new_tokens=12, greedy=True, temperature=0.0, ignore_eos=True)

        async def go():
            reqs = [ModelRequest(rid=f"{p}-{i}", input_ids=prompts[p], gconfig=gc) for p in range(2) for i in range(3)]
            return await asyncio.gather(*[eng.agenerate(r) for r in reqs])

        out = asyncio.run(go())
        stats = eng.sched.stats()
        eng.destroy()
        return [(r.output_tokens, r.output_logprobs) for r in out], stats

    shared, st_on = run(True)
    plain, st_off = run(False)
    assert st_on["prompt_forks"] == 4 and st_off["prompt_forks"] == 0
    for (ta, la), (tb, lb) in zip(shared, plain):
        assert ta == tb
        assert max(abs(x - y) for x, y in zip(la, lb)) < 1e-4
    # and all copies of one prompt agree with each other
    assert shared[0][0] == shared[1][0] == shared[2][0] and shared[3][0] == shared[4][0] == shared[5][0]


def test_scheduler_keeps_a_group_prefix_shared_across_resubmission():
    """After an interruption the samples of a group come back as prompt + partial output (different requests,
    same leading tokens). Each is prefilled whole; the first becomes the holder of the group's full prefix
    pages, the others adopt them and give their own copies back."""
    import numpy as np

    from areal_b200.engine.rollout_engine import PagedScheduler

    bs = 16
    s = PagedScheduler(num_blocks=64, block_size=bs, max_num_seqs=16, max_batched_tokens=4096, max_blocks_per_seq=8)
    prompt = list(range(100, 140))  # 40 tokens: 2 full pages + 8 tokens
    parts = [[900 + i] * (5 + 7 * i) for i in range(3)]  # partial outputs of different lengths
    free0 = s.stats()["free_blocks"]
    ids = [s.add(prompt + part, 4, 0, [], True, share_len=len(prompt)) for part in parts]
    solo = s.add(list(range(300, 350)), 4, 0, [], True)  # unrelated request: keeps its own pages
    assert s.plan() == 1 and s.hdr.n_seqs == 4  # different prompts: everyone prefills
    used_before = free0 - s.stats()["free_blocks"]
    s.commit(np.full(4, 7, dtype=np.int32), np.zeros(4, dtype=np.float32))
    st = s.stats()
    assert st["dedup_pages"] == 4  # two followers x two full prefix pages
    assert free0 - st["free_blocks"] == used_before - 4
    assert s.plan() == 2
    n = s.hdr.n_seqs
    rows = s.block_table[: n * 8].reshape(n, 8)
    order = s.seq_ids[:n].tolist()
    a, b, c = (rows[order.index(i)] for i in ids)
    assert (a[:2] == b[:2]).all() and (a[:2] == c[:2]).all() and len({int(a[2]), int(b[2]), int(c[2])}) == 3
    # the group's sequences are adjacent in the decode batch (sorted by their first page)
    pos = sorted(order.index(i) for i in ids)
    assert pos[2] - pos[0] == 2 and order.index(solo) not in range(pos[0], pos[2] + 1)
    for _ in range(8):
        if s.plan() == 0:
            break
        s.commit(np.full(s.hdr.n_seqs, 9, dtype=np.int32), np.zeros(s.hdr.n_seqs, dtype=np.float32))
    while s.pop_finished() is not None:
        pass
    assert s.stats()["free_blocks"] == free0 and s.stats()["live"] == 0  # every page came back exactly once
    s.close()


def test_engine_outputs_do_not_change_when_resubmitted_groups_share_their_prefix():
    """Greedy continuation of three requests that start with the same 40 tokens and continue differently: with
    the prefix pages shared after prefill the tokens and logprobs equal those with sharing switched off."""
    import asyncio

    from areal_b200.api.cli_args import GenerationHyperparameters, InferenceEngineConfig, NativeRolloutConfig
    from areal_b200.engine.rollout_engine import NativeRolloutEngine

    def run(share: bool):
        cfg = InferenceEngineConfig(experiment_name="e", trial_name="t", backend="native:d1", max_concurrent_rollouts=64,
                                    consumer_batch_size=8,
                                    native=NativeRolloutConfig(model_preset="tiny-qwen2", context_length=128, max_num_seqs=16,
                                                               max_num_batched_tokens=1024, num_kv_blocks=128, seed=0,
                                                               cuda_graph=False))
        eng = NativeRolloutEngine(cfg).initialize(device="cpu")
        eng.sched.set_prompt_sharing(share)
        g = torch.Generator().manual_seed(9)
        prefix = torch.randint(0, 1000, (40,), generator=g).tolist()
        tails = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (3, 11, 20)]
        gc = GenerationHyperparameters(max_new_tokens=10, greedy=True, temperature=0.0, ignore_eos=True)

        async def go():
            return await asyncio.gather(*[eng._generate_once(prefix + t, gc, 10, share_len=len(prefix)) for t in tails])

        out = asyncio.run(go())
        st = eng.sched.stats()
        eng.destroy()
        return [(toks, lps) for _, toks, lps in out], st

    shared, st_on = run(True)
    plain, st_off = run(False)
    assert st_on["dedup_pages"] == 4 and st_off["dedup_pages"] == 0
    for (ta, la), (tb, lb) in zip(shared, plain):
        assert ta == tb and max(abs(x - y) for x, y in zip(la, lb)) < 1e-4


def test_evaluation_episodes_bypass_the_staleness_gate_and_the_training_queue():
    CountingWorkflow.started = 0
    eng, ex = _executor(bs=4, eta=0)
    try:
        for i in range(12):
            ex.submit({"i": i}, CountingWorkflow)
        assert ex.wait(4, timeout=10)["rewards"].shape == (4,)
        time.sleep(0.1)
        assert ex.get_capacity() <= 0 and CountingWorkflow.started == 4       # training is gated at version 0
        # evaluation goes through although 8 training episodes wait for capacity in front of it
        ev = ex.rollout_batch([{"i": 100 + i} for i in range(5)], CountingWorkflow, is_eval=True)
        assert sorted(ev["rewards"].tolist()) == [100.0, 101.0, 102.0, 103.0, 104.0]
        st = ex.export_stats()
        assert st["rollout/accepted"] == 4 and st["rollout/enqueued"] == 8    # untouched by the evaluation samples
        assert ex.wait(1, timeout=0.2, raise_timeout=False) is None           # and none of them leaked into a batch
        eng.version = 1
        nxt = ex.wait(4, timeout=10)
        assert nxt["rewards"].max() < 100
    finally:
        ex.destroy()


def test_native_engine_stop_strings_and_unsupported_sampling_options():
    """Stop strings cut the output at the first token that completes one (matched on decoded text, so a string
    may span tokens); options the engine does not implement are refused, not ignored."""
    import asyncio

    from areal_b200.api.cli_args import GenerationHyperparameters, InferenceEngineConfig, NativeRolloutConfig
    from areal_b200.api.io_struct import ModelRequest
    from areal_b200.engine.rollout_engine import NativeRolloutEngine, stop_string_cut

    class Tok:  # token i decodes to one letter; "cd" spans two tokens
        def decode(self, ids, skip_special_tokens=True):
            return "".join("abcdefghij"[i % 10] for i in ids)

    assert stop_string_cut([0, 1, 2, 3, 4], Tok(), ["cd"]) == 4
    assert stop_string_cut([0, 1, 2, 3, 4], Tok(), ["zz", "e"]) == 5
    assert stop_string_cut([0, 1, 2], Tok(), ["cd"]) is None and stop_string_cut([], Tok(), ["a"]) is None
    assert stop_string_cut([2, 3, 2, 3], Tok(), ["cd"]) == 2          # the first occurrence wins

    cfg = InferenceEngineConfig(experiment_name="e", trial_name="t", backend="native:d1", max_concurrent_rollouts=8,
                                consumer_batch_size=4,
                                native=NativeRolloutConfig(model_preset="tiny-qwen2", context_length=128, max_num_seqs=8,
                                                           max_num_batched_tokens=512, num_kv_blocks=64, seed=0,
                                                           cuda_graph=False))
    eng = NativeRolloutEngine(cfg).initialize(device="cpu")
    try:
        prompt = list(range(20, 40))
        base = GenerationHyperparameters(max_new_tokens=12, greedy=True, temperature=0.0, ignore_eos=True)
        full = asyncio.run(eng.agenerate(ModelRequest(input_ids=prompt, gconfig=base, tokenizer=Tok())))
        assert len(full.output_tokens) == 12 and full.stop_reason == "length"
        text = Tok().decode(full.output_tokens)
        stop = text[4:6]                                              # a two-letter string inside the output
        first = text.index(stop) + 2
        cut = asyncio.run(eng.agenerate(ModelRequest(input_ids=prompt, gconfig=base.new(stop=[stop]), tokenizer=Tok())))
        assert cut.stop_reason == "stop" and cut.output_tokens == full.output_tokens[:first]
        assert len(cut.output_logprobs) == len(cut.output_versions) == first
        same = asyncio.run(eng.agenerate(ModelRequest(input_ids=prompt, gconfig=base.new(stop=["#nothing#"]), tokenizer=Tok())))
        assert same.output_tokens == full.output_tokens and same.stop_reason == "length"
        with pytest.raises(ValueError, match="tokenizer"):
            asyncio.run(eng.agenerate(ModelRequest(input_ids=prompt, gconfig=base.new(stop=["x"]))))
        # frequency penalty: a huge penalty forbids any repeated output token (greedy decoding of a random tiny
        # model repeats itself quickly without it)
        free = asyncio.run(eng.agenerate(ModelRequest(input_ids=prompt, gconfig=base.new(max_new_tokens=40))))
        pen = asyncio.run(eng.agenerate(ModelRequest(input_ids=prompt, gconfig=base.new(max_new_tokens=40,
                                                                                         frequency_penalty=1e4))))
        assert len(set(pen.output_tokens)) == 40 and pen.output_tokens[0] == free.output_tokens[0]
        assert len(set(free.output_tokens)) < 40 or free.output_tokens == pen.output_tokens
        assert not eng._hist                                             # the history is dropped with the request
        with pytest.raises(NotImplementedError):
            asyncio.run(eng.agenerate(ModelRequest(input_ids=prompt, gconfig=base.new(use_beam_search=True))))
    finally:
        eng.destroy()
