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
