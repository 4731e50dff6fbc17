"""Chrome-trace JSONL tracer, session tracer and converter."""
import asyncio
import json
import os

from areal_b200.api.cli_args import PerfTracerConfig, SessionTracerConfig
from areal_b200.utils import perf_tracer as pt


def _cfg(tmp_path, **kw):
    return PerfTracerConfig(experiment_name="e", trial_name="t", fileroot=str(tmp_path), enabled=True, **kw)


def test_scopes_instants_decorators_and_conversion(tmp_path):
    tr = pt.configure(_cfg(tmp_path, save_interval=2), rank=3, role="actor")

    @pt.trace_perf("work", pt.Category.COMPUTE)
    def work(x):
        return x + 1

    @pt.trace_perf(category=pt.Category.IO)
    async def awork():
        await asyncio.sleep(0)
        return 7

    with pt.trace_scope("outer", pt.Category.SCHEDULER, {"k": 1}):
        assert work(1) == 2
        assert asyncio.run(awork()) == 7
        pt.instant("mark", pt.Category.MISC)
    pt.save(step=0)            # (0 + 1) % 2 != 0: nothing written yet
    assert not os.path.exists(tr.path)
    pt.save(step=1)
    lines = [json.loads(l) for l in open(tr.path)]
    names = [e["name"] for e in lines]
    assert {"outer", "work", "mark"} <= set(names) and any("awork" in n for n in names)
    outer = next(e for e in lines if e["name"] == "outer")
    inner = next(e for e in lines if e["name"] == "work")
    assert outer["ph"] == "X" and outer["pid"] == 3 and outer["cat"] == "scheduler" and outer["args"]["k"] == 1
    assert outer["ts"] <= inner["ts"] and inner["ts"] + inner["dur"] <= outer["ts"] + outer["dur"] + 1
    out = pt.convert_jsonl_to_chrome_trace(os.path.dirname(tr.path))
    merged = json.load(open(out))
    assert len(merged["traceEvents"]) == len(lines)
    pt.configure(None)
    with pt.trace_scope("noop"):
        pass


def test_session_tracer(tmp_path):
    tr = pt.configure(_cfg(tmp_path, session_tracer=SessionTracerConfig(enabled=True, flush_threshold=2)), rank=0)
    st = pt.get_session_tracer()
    a = st.start_session(task_id=11, prompt_len=5)
    with st.phase(a, "generate", tokens=9):
        pass
    with st.phase(a, "reward"):
        pass
    b = st.start_session(task_id=12)
    st.end_session(a, "accepted", reward=1.0)
    st.end_session(b, "rejected")        # second finished session reaches the flush threshold
    recs = [json.loads(l) for l in open(st.path)]
    assert [r["status"] for r in recs] == ["accepted", "rejected"]
    assert [p["name"] for p in recs[0]["phases"]] == ["generate", "reward"] and recs[0]["meta"]["reward"] == 1.0
    pt.configure(None)


def test_trace_converter_cli_and_engine_profiler(tmp_path, capsys):
    """The converter tool merges rank files and summarises; the engine profiler runs on the CPU path."""
    import json

    from areal_b200.tools import perf_trace_converter, profile_engines

    for r in range(2):
        with open(tmp_path / f"traces-r{r}.jsonl", "w") as f:
            f.write(json.dumps(dict(name="fwd", cat="compute", ph="X", ts=10 + r, dur=2000, pid=r, tid=0)) + "\n")
            f.write(json.dumps(dict(name="allreduce", cat="comm", ph="X", ts=5000, dur=500, pid=r, tid=1)) + "\n")
    out = str(tmp_path / "merged.json")
    assert perf_trace_converter.main([str(tmp_path), "-o", out, "--summary"]) == 0
    ev = json.load(open(out))["traceEvents"]
    assert len(ev) == 4 and [e["ts"] for e in ev] == sorted(e["ts"] for e in ev)
    rows = perf_trace_converter.summarize(out)
    assert rows[0][:3] == ("compute", "fwd", 2) and rows[0][3] == 4.0 and rows[1][3] == 1.0
    capsys.readouterr()
    assert profile_engines.main(["--preset", "tiny-qwen2", "--device", "cpu", "--tokens", "256", "--seq-len", "64",
                                 "--steps", "1", "--warmup", "1"]) == 0
    text = capsys.readouterr().out
    rep = json.loads(text[text.index("{"):])
    assert rep["tokens_per_step"] == 256 and rep["train"]["tokens_per_s"] > 0 and rep["forward"]["ms_per_step"] > 0


def test_session_trace_summary_and_timeline(tmp_path, capsys):
    import json

    from areal_b200.tools import plot_session_trace
    from areal_b200.utils.perf_tracer import SessionTracer

    tr = SessionTracer(None, str(tmp_path), rank=0)
    for k in range(3):
        sid = tr.start_session(task_id=k)
        with tr.phase(sid, "generate"):
            pass
        with tr.phase(sid, "reward"):
            pass
        tr.end_session(sid, status="accepted" if k < 2 else "rejected")
    tr.flush(force=True)
    recs = plot_session_trace.load(str(tmp_path))
    s = plot_session_trace.summarize(recs)
    assert s["sessions"] == 3 and s["status"] == {"accepted": 2, "rejected": 1}
    assert set(s["phases"]) == {"generate", "reward"} and s["phases"]["generate"]["n"] == 3
    assert plot_session_trace.main([str(tmp_path)]) == 0
    page = open(tmp_path / "sessions.html").read()
    assert page.count("<rect") == 9 and "generate" in page and "#d00" in page


def test_trainer_writes_perf_trace_sessions_and_torch_profile(tmp_path):
    """With `perf_tracer.enabled`, a trainer run leaves a per-rank trace with its timed phases, a torch
    profile for the configured step, and (with rollout tracing on) one session per episode."""
    import glob
    import json
    import math

    import torch

    from areal_b200.api.cli_args import (MicroBatchSpec, OptimizerConfig, PerfTracerConfig, SFTConfig,
                                         TrainEngineConfig, _propagate_names)
    from areal_b200.trainer.sl_trainer import SFTTrainer

    g = torch.Generator().manual_seed(0)
    data = [dict(input_ids=torch.randint(0, 1024, (16,), generator=g).tolist(), loss_mask=[0] * 4 + [1] * 12)
            for _ in range(8)]
    cfg = SFTConfig(actor=TrainEngineConfig(backend="fsdp:d1", model_preset="tiny-qwen2", init_from_scratch=True,
                                            optimizer=OptimizerConfig(lr=1e-3, warmup_steps_proportion=0.0),
                                            mb_spec=MicroBatchSpec(max_tokens_per_mb=512)))
    cfg.experiment_name, cfg.trial_name = "pt", "t"
    cfg.cluster.fileroot = str(tmp_path)
    cfg.train_dataset.batch_size = 4
    cfg.total_train_epochs = 2
    cfg.perf_tracer = PerfTracerConfig(enabled=True, save_interval=1, profile_steps=[1])
    _propagate_names(cfg)
    with SFTTrainer(cfg, data) as tr:
        tr.train(max_steps=3)
    traces = glob.glob(str(tmp_path / "**" / "traces-r0.jsonl"), recursive=True)
    assert len(traces) == 1
    events = [json.loads(line) for line in open(traces[0])]
    names = {e["name"] for e in events}
    assert {"train_step", "train_step_0", "train_step_2"} <= names
    assert all(math.isfinite(e.get("dur", 0.0)) for e in events)
    profs = glob.glob(str(tmp_path / "**" / "torch_profile_step1_r0.json"), recursive=True)
    assert len(profs) == 1 and os.path.getsize(profs[0]) > 1000


def test_task_and_session_ids_follow_the_coroutine_context(tmp_path):
    """Two episodes run concurrently; each binds its task and session to its own context, and phases traced deep
    inside (no ids passed around) land in the right session."""
    pt.reset()
    assert not pt.is_configured() and pt.register_session() is None
    with pt.trace_session_phase("ignored"):          # outside a configured tracer: a no-op
        pass
    pt.configure(_cfg(tmp_path, session_tracer=SessionTracerConfig(enabled=True, flush_threshold=100)), rank=0, role="rollout")
    assert pt.is_configured()

    async def reward(name):
        async with pt.atrace_session_phase("reward", who=name):
            await asyncio.sleep(0.001)

    async def episode(name, reject):
        tid = pt.register_task()
        with pt.session_context(who=name) as ctx:
            assert pt.get_task_id() == tid and pt.get_session_id() == ctx["session_id"]
            with pt.trace_session_phase("generate", who=name):
                await asyncio.sleep(0.002)
            await reward(name)
            pt.trace_session_event("scored", who=name)
            if reject:
                ctx["status"] = "rejected"
        assert pt.get_session_id() is None or pt.get_session_id() != ctx["session_id"]
        return tid

    async def boom():
        pt.register_task()
        with pt.trace_session():
            raise ValueError("x")

    async def main():
        tids = await asyncio.gather(episode("a", False), episode("b", True))
        try:
            await boom()
        except ValueError:
            pass
        return tids

    tids = asyncio.run(main())
    assert tids[0] != tids[1]
    pt.save(force=True)
    path = pt.get_session_tracer().path
    recs = [json.loads(line) for line in open(path)]
    by = {r["meta"].get("who"): r for r in recs}
    assert by["a"]["status"] == "accepted" and by["b"]["status"] == "rejected" and by[None]["status"] == "failed"
    for who in ("a", "b"):
        assert [p["name"] for p in by[who]["phases"]] == ["generate", "reward", "scored"]
        assert all(p["who"] == who for p in by[who]["phases"]) and by[who]["task_id"] in tids
    pt.reset()
    assert pt.get_tracer() is None and pt.get_task_id() is None
