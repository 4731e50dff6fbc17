"""Search and terminal agents: retrieval, scoring, the tool loops against a scripted chat client, datasets."""
import asyncio
import json
import types

import pytest

from areal_b200.dataset import get_custom_dataset
from areal_b200.infra.sandbox import ShellWorkspace
from areal_b200.workflow.agents import HttpSearch, LocalCorpus, ReActSearchAgent, TerminalAgent, qa_reward
from areal_b200.workflow.agents.search_agent import extract_final_answer, normalize_answer, qa_f1, run_search_tool
from areal_b200.workflow.agents.terminal_agent import run_terminal_tool, score_checks

DOCS = [
    {"id": "d1", "title": "Eiffel Tower", "text": "The Eiffel Tower is a wrought-iron lattice tower in Paris, France. "
                                                    "It was completed in 1889 by Gustave Eiffel's company."},
    {"id": "d2", "title": "Statue of Liberty", "text": "The Statue of Liberty stands in New York Harbor. It was a gift "
                                                         "from France, dedicated in 1886."},
    {"id": "d3", "title": "Great Wall", "text": "The Great Wall of China is a series of fortifications built across "
                                                 "the northern borders of ancient Chinese states."},
]


class ScriptedClient:
    """Stands in for the chat client: returns the next scripted assistant message and records the requests."""

    def __init__(self, script):
        self.script, self.requests = list(script), []
        self.chat = types.SimpleNamespace(completions=types.SimpleNamespace(create=self._create))

    async def _create(self, **kw):
        self.requests.append(dict(kw, messages=list(kw["messages"])))   # the agent keeps appending to its list
        msg = self.script.pop(0)
        calls = [types.SimpleNamespace(id=f"call{i}", function=types.SimpleNamespace(name=n, arguments=json.dumps(a)))
                 for i, (n, a) in enumerate(msg.get("tool_calls", []))]
        message = types.SimpleNamespace(content=msg.get("content"), tool_calls=calls or None)
        return types.SimpleNamespace(id=f"cmpl{len(self.requests)}", choices=[types.SimpleNamespace(message=message)])


def test_bm25_ranks_the_matching_passage_first():
    corpus = LocalCorpus(DOCS)
    hits = corpus.search("who built the tower in Paris", top_k=2)
    assert hits[0]["id"] == "d1" and len(hits) <= 2
    assert corpus.search("zebra quantum")[:1] == []
    assert corpus.search("France")[0]["id"] in ("d1", "d2")
    assert "New York Harbor" in corpus.visit("d2") and corpus.visit("nope") is None


def test_bm25_prefers_rare_terms_and_from_jsonl(tmp_path):
    p = tmp_path / "corpus.jsonl"
    p.write_text("\n".join(json.dumps(d) for d in DOCS))
    corpus = LocalCorpus.from_jsonl(str(p))
    # "fortifications" occurs in one passage only, "the" in all: the rare term decides
    assert corpus.search("the fortifications")[0]["id"] == "d3"


def test_answer_scoring():
    assert normalize_answer("The  Eiffel-Tower!") == "eiffeltower"
    assert qa_f1("Gustave Eiffel", "gustave eiffel") == 1.0
    assert 0 < qa_f1("Gustave Eiffel company", "Gustave Eiffel") < 1
    assert qa_f1("Paris", "London") == 0.0
    assert extract_final_answer("a <answer>x</answer> b <answer> 1889 </answer>") == "1889"
    assert qa_reward("I think <answer>1889</answer>", ["1889", "in 1889"]) == 1.0
    assert qa_reward("1889 without tags", "1889") == 0.0
    assert qa_reward("<answer>the year 1889</answer>", "1889", metric="em") == 0.0


def test_search_tool_reports_errors_as_text():
    corpus = LocalCorpus(DOCS)
    assert "[d1]" in run_search_tool(corpus, "search", {"query": "Eiffel"})
    assert run_search_tool(corpus, "visit", '{"doc_id": "zzz"}') == "error: unknown doc_id"
    assert run_search_tool(corpus, "search", "{not json").startswith("error:")
    assert run_search_tool(corpus, "fly", {}).startswith("error: unknown tool")


def test_http_backend_uses_the_service_protocol():
    seen = []

    def post(url, payload):
        seen.append((url, payload))
        return {"results": [{"id": "x", "title": "t", "snippet": "s"}]} if url.endswith("/search") else {"text": "full"}

    b = HttpSearch("http://svc:1/", post=post)
    assert b.search("q", 3)[0]["id"] == "x" and b.visit("x") == "full"
    assert seen == [("http://svc:1/search", {"query": "q", "top_k": 3}), ("http://svc:1/visit", {"id": "x"})]


def test_react_agent_loop_feeds_tool_results_back():
    client = ScriptedClient([
        {"tool_calls": [("search", {"query": "Eiffel Tower completed"})]},
        {"tool_calls": [("visit", {"doc_id": "d1"})]},
        {"content": "It was finished in <answer>1889</answer>."},
    ])
    agent = ReActSearchAgent(LocalCorpus(DOCS), max_turns=5, temperature=1.0, max_tokens=5)
    data = {"messages": [{"role": "user", "content": "When was the Eiffel Tower completed?"}], "answer": ["1889"]}
    assert asyncio.run(agent.run(data, client=client)) == 1.0
    assert len(client.requests) == 3 and "max_tokens" not in client.requests[0]
    last = client.requests[-1]["messages"]
    assert [m["role"] for m in last] == ["system", "user", "assistant", "tool", "assistant", "tool"]
    assert "[d1]" in last[3]["content"] and "wrought-iron" in last[5]["content"]


def test_react_agent_without_answer_gets_penalty_and_respects_max_turns():
    client = ScriptedClient([{"tool_calls": [("search", {"query": "x"})]}] * 3)
    agent = ReActSearchAgent(LocalCorpus(DOCS), max_turns=3, invalid_penalty=0.5)
    r = asyncio.run(agent.run({"messages": [{"role": "user", "content": "q"}], "answer": "a"}, client=client))
    assert r == -0.5 and len(client.requests) == 3


def test_shell_workspace_keeps_state_and_fences_paths():
    with ShellWorkspace(files={"src/a.txt": "hello\n"}) as ws:
        assert ws.run("cat src/a.txt").stdout == "hello\n"
        assert ws.run("echo more > b.txt && ls").ok
        assert ws.read_file("b.txt") == "more\n"
        assert ws.run("exit 3").exit_code == 3
        r = ws.run("sleep 30", timeout=0.5)
        assert r.timed_out and not r.ok
        with pytest.raises(ValueError):
            ws.write_file("../escape.txt", "x")
        root = ws.root
    import os

    assert not os.path.exists(root)


def test_terminal_tools_and_checks():
    with ShellWorkspace() as ws:
        assert run_terminal_tool(ws, "write_file", {"path": "f.py", "content": "print(6*7)\n"}) == "ok"
        out = run_terminal_tool(ws, "bash", {"command": "python3 f.py"})
        assert out.startswith("exit code 0") and "42" in out
        assert run_terminal_tool(ws, "read_file", {"path": "f.py"}) == "print(6*7)\n"
        assert run_terminal_tool(ws, "read_file", {"path": "missing"}).startswith("error:")
        assert score_checks(ws, ["test -f f.py", "test -f g.py"]) == 0.5
        assert score_checks(ws, ["test -f f.py", "test -f g.py"], all_or_nothing=True) == 0.0
        assert score_checks(ws, []) == 0.0


def test_terminal_agent_episode_is_rewarded_by_the_checks():
    client = ScriptedClient([
        {"tool_calls": [("read_file", {"path": "calc.py"})]},
        {"tool_calls": [("write_file", {"path": "calc.py", "content": "def add(a, b):\n    return a + b\n"})]},
        {"tool_calls": [("bash", {"command": "python3 -c 'import calc; print(calc.add(2, 3))'"})]},
        {"content": "Fixed the add function."},
    ])
    task = {"instruction": "calc.add returns the wrong result; fix it.",
            "files": {"calc.py": "def add(a, b):\n    return a - b\n"},
            "checks": ["python3 -c 'import calc, sys; sys.exit(calc.add(2, 3) != 5)'", "test -f calc.py"]}
    assert asyncio.run(TerminalAgent(max_turns=6).run(task, client=client)) == 1.0
    assert "5" in client.requests[-1]["messages"][-1]["content"]
    # an agent that does nothing passes only the second check
    lazy = ScriptedClient([{"content": "done"}])
    assert asyncio.run(TerminalAgent().run(task, client=lazy)) == 0.5


def test_agent_datasets(tmp_path):
    qa = tmp_path / "hotpot_qa.jsonl"
    qa.write_text(json.dumps({"question": "q1", "answer": "a1"}) + "\n" +
                  json.dumps({"question": "q2", "answers": ["a2", "b2"]}) + "\n" + json.dumps({"question": "q3"}) + "\n")
    items = get_custom_dataset(path=str(qa), type="rl")
    assert [i["answer"] for i in items] == [["a1"], ["a2", "b2"]]
    tasks = tmp_path / "terminal_tasks.jsonl"
    tasks.write_text(json.dumps({"instruction": "do", "files": {"a": "b"}, "checks": ["true"]}) + "\n" +
                     json.dumps({"instruction": "no checks"}) + "\n")
    items = get_custom_dataset(path=str(tasks), type="rl")
    assert len(items) == 1 and items[0]["checks"] == ["true"] and items[0]["messages"][0]["content"] == "do"


def test_code_reward_runs_the_last_code_block_in_the_sandbox(tmp_path):
    from areal_b200.reward.code import code_reward_fn, extract_program

    tests = [{"input": "2 3\n", "output": "5"}, {"input": "10 -4\n", "output": "6"}]
    good = "First idea:\n```python\nprint(1)\n```\nBetter:\n```python\na, b = map(int, input().split())\nprint(a + b)\n```"
    assert extract_program(good).startswith("a, b")
    assert code_reward_fn(None, good, None, None, tests=tests) == 1.0
    half = "```python\nprint(5)\n```"
    assert code_reward_fn(None, half, None, None, tests=tests) == 0.5
    assert code_reward_fn(None, half, None, None, tests=tests, all_or_nothing=True) == 0.0
    assert code_reward_fn(None, "```python\nwhile True: pass\n```", None, None, tests=tests[:1], timeout=0.5) == 0.0
    assert code_reward_fn(None, "", None, None, tests=tests) == 0.0 and code_reward_fn(None, good, None, None) == 0.0
    path = tmp_path / "code_tasks.jsonl"
    path.write_text(json.dumps({"question": "Add two integers.", "tests": tests}) + "\n" + json.dumps({"question": "x"}) + "\n")
    items = get_custom_dataset(path=str(path), type="rl")
    assert len(items) == 1 and items[0]["tests"] == tests and "```python" in items[0]["messages"][0]["content"]


def test_external_user_lifecycle_against_a_gateway():
    """The user-side example script drives one episode through an in-process gateway and proxy worker."""
    import importlib.util
    import os

    import httpx

    from areal_b200.openai.proxy.online_agent import OnlineAgent
    from areal_b200.openai.proxy.proxy_gateway import create_gateway_app
    from areal_b200.openai.proxy.proxy_rollout_server import create_proxy_app
    from tests.test_openai_proxy import Engine, Tok

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("external_user", os.path.join(root, "examples", "online_proxy",
                                                                               "external_user.py"))
    user = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(user)
    worker = create_proxy_app(Engine(), Tok(), admin_api_key="adm")

    async def forward(method, url, body, headers):
        async with httpx.AsyncClient(transport=httpx.ASGITransport(app=worker), base_url="http://w") as c:
            r = await c.request(method, "/" + url.split("//", 1)[1].split("/", 1)[1], json=body, headers=headers)
            return r.status_code, r.content, r.headers.get("content-type", "application/json")

    gw = create_gateway_app(admin_api_key="adm", forward=forward)

    async def scenario():
        async with httpx.AsyncClient(transport=httpx.ASGITransport(app=gw), base_url="http://gw") as c:
            async def apost(url, body, headers):
                r = await c.post(url.replace("http://gw", ""), json=body, headers=headers)
                r.raise_for_status()
                return r.json()

            wait = asyncio.create_task(OnlineAgent("http://gw", "w:1", admin_api_key="adm", timeout=30, post=apost).run({}))
            while (await c.get("/health")).json()["ready_workers"] < 1:
                await asyncio.sleep(0.01)
            loop = asyncio.get_running_loop()

            def post(url, body, headers):  # the script is synchronous: hop back onto the loop from its thread
                return asyncio.run_coroutine_threadsafe(apost(url, body, headers), loop).result(30)

            result = await loop.run_in_executor(None, lambda: user.run_episode("http://gw/", "adm", "hi", "zzz", post, 4))
            return result, await wait

    result, done = asyncio.run(scenario())
    assert result["reward"] in (0.0, 1.0) and done["session_id"] == result["session_id"]


def test_remote_sandbox_service_and_client():
    from fastapi.testclient import TestClient

    from areal_b200.infra.sandbox import code_reward
    from areal_b200.infra.sandbox.remote import RemoteSandbox, create_runner_app
    from areal_b200.reward.code import code_reward_fn

    srv = TestClient(create_runner_app(token="tok", max_timeout=2.0))
    assert srv.post("/run", json={"code": "print(1)"}).status_code == 401

    def post(url, body, headers):
        r = srv.post(url.replace("http://sb", ""), json=body, headers=headers)
        r.raise_for_status()
        return r.json()

    sb = RemoteSandbox("http://sb/", "tok", post=post)
    r = sb.run("import sys\nprint(int(sys.stdin.read()) * 2)", stdin="21")
    assert r.ok and r.stdout.strip() == "42"
    assert sb.run("raise SystemExit(3)").exit_code == 3
    slow = sb.run("while True: pass", timeout=30.0)                 # the service caps the time-out at 2 s
    assert slow.timed_out and not slow.ok
    rs = sb.run_batch([{"code": "print('a')"}, {"code": "print('b')"}, {"code": "1/0"}])
    assert [x.stdout.strip() for x in rs[:2]] == ["a", "b"] and not rs[2].ok
    assert srv.get("/health").json()["runs"] == 6
    assert code_reward(sb, "print(input()[::-1])", [("abc", "cba"), ("xy", "yx")]) == 1.0
    tests = [{"input": "2 3\n", "output": "5"}]
    good = "```python\na, b = map(int, input().split())\nprint(a + b)\n```"
    assert code_reward_fn(None, good, None, None, tests=tests, sandbox=sb) == 1.0
    down = RemoteSandbox("http://sb", "wrong", post=post)            # a refused request is a failed run, not an exception
    bad = down.run("print(1)")
    assert not bad.ok and "sandbox service error" in bad.stderr and code_reward_fn(None, good, None, None, tests=tests, sandbox=down) == 0.0
    assert asyncio.run(sb.arun("print(7)")).stdout.strip() == "7"


def test_service_desk_domain_policy_and_reward():
    """The tools keep the data consistent but do not enforce the policy; the reward compares the final database with
    what the task's reference actions produce and checks what the agent told the customer."""
    from areal_b200.workflow.agents.service_desk_agent import (DeskDB, ScriptedUser, STOP, desk_reward,
                                                               expected_state, make_desk_tasks)

    tasks = make_desk_tasks(8, seed=3)
    assert [t["kind"] for t in tasks[:4]] == ["cancel_ok", "cancel_refuse", "change", "bags"]
    assert make_desk_tasks(8, seed=3) == tasks and make_desk_tasks(8, seed=4) != tasks
    ok, refuse, change, bags = tasks[:4]
    rid = next(iter(refuse["db"]["reservations"]))
    db = DeskDB(refuse["db"])
    seats = db.data["flights"][db.data["reservations"][rid]["flight_number"]]["seats"]
    assert desk_reward(refuse, db.data, ["I am sorry, this reservation cannot be cancelled."]) == 1.0
    assert json.loads(db.call("get_reservation_details", {"reservation_id": rid}))["insurance"] is False
    assert json.loads(db.call("cancel_reservation", json.dumps({"reservation_id": rid}))) == {"status": "cancelled"}
    assert db.data["flights"][db.data["reservations"][rid]["flight_number"]]["seats"] == seats + 1
    assert desk_reward(refuse, db.data, []) == 0.0                      # the forbidden cancellation went through
    assert db.call("cancel_reservation", {"reservation_id": rid}).startswith("error:")
    assert db.call("get_user_details", {"user_id": "nobody"}).startswith("error:") and \
        db.call("drop_tables", {}).startswith("error:")
    # the reference actions reach the reference state; the required information must have been said
    db = DeskDB(change["db"])
    a = change["expected_actions"][0]
    assert "price_difference" in json.loads(db.call(a["name"], a["arguments"]))
    assert db.data == expected_state(change)
    assert desk_reward(change, db.data, [f"Done, you are now on {change['outputs'][0]}."]) == 1.0
    assert desk_reward(change, db.data, ["Done."]) == 0.0
    assert db.call("change_flight", {"reservation_id": a["arguments"]["reservation_id"], "flight_number": "ZZ1"}).startswith("error:")
    user = ScriptedUser(bags)
    assert asyncio.run(user.respond("May I have your user id?")).startswith("My user id is user_")
    assert "reservation is R" in asyncio.run(user.respond("Thanks. Which reservation is it about?"))
    assert "in total" in asyncio.run(user.respond("How many bags do you need?"))
    assert asyncio.run(user.respond("I will set it to that. Do you confirm?")) == "Yes, please go ahead."
    assert asyncio.run(user.respond("Done. Goodbye!")) == STOP


def test_service_desk_agent_episodes_against_a_scripted_client():
    from areal_b200.workflow.agents import ServiceDeskAgent, make_desk_tasks

    ok, refuse, change, bags = make_desk_tasks(4, seed=5)
    rid = next(iter(ok["db"]["reservations"]))
    good = ScriptedClient([
        {"content": "Sure. May I have your user id?"},
        {"tool_calls": [("get_user_details", {"user_id": ok["user_id"]})]},
        {"content": "Thank you. Which reservation would you like to cancel?"},
        {"tool_calls": [("get_reservation_details", {"reservation_id": rid})]},
        {"content": "This reservation can be cancelled. Shall I proceed?"},
        {"tool_calls": [("cancel_reservation", {"reservation_id": rid})]},
        {"content": "It is cancelled. Goodbye!"},
    ])
    assert asyncio.run(ServiceDeskAgent().run(ok, client=good)) == 1.0
    # the customer's answers reached the agent, and the tool result followed the call
    seen = [m for m in good.requests[-1]["messages"] if m["role"] == "user"]
    assert [m["content"] for m in seen][1:] == [ok["facts"]["user id"], ok["facts"]["reservation"], "Yes, please go ahead."]
    assert good.requests[-1]["messages"][-1]["role"] == "tool" and good.requests[0]["tools"]
    # cancelling where the policy forbids it costs the reward; refusing earns it
    rid2 = next(iter(refuse["db"]["reservations"]))
    bad = ScriptedClient([{"tool_calls": [("cancel_reservation", {"reservation_id": rid2})]}, {"content": "Done, goodbye."}])
    assert asyncio.run(ServiceDeskAgent().run(refuse, client=bad)) == 0.0
    polite = ScriptedClient([{"content": "I am sorry: economy without insurance, booked more than a day ago, cannot be "
                                         "cancelled. Goodbye."}])
    assert asyncio.run(ServiceDeskAgent().run(refuse, client=polite)) == 1.0
    # an agent that never finishes is cut off at max_turns with the database untouched
    looping = ScriptedClient([{"tool_calls": [("get_user_details", {"user_id": bags["user_id"]})]}] * 5)
    assert asyncio.run(ServiceDeskAgent(max_turns=5).run(bags, client=looping)) == 0.0
    items = get_custom_dataset(path="generate:desk:6:1", type="rl")
    assert len(items) == 6 and items[0]["messages"][0]["content"] == items[0]["opening"]
    assert get_custom_dataset(path="generate:desk:6:1", type="rl", split="test") != items
