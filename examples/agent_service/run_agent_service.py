"""Starts an agent service on this machine (workers + gateway, each a FastAPI app under uvicorn in a thread) and
talks to it over the OpenAI Responses protocol.

    python examples/agent_service/run_agent_service.py --base-url http://127.0.0.1:8000/v1 [--workers 2]
    python examples/agent_service/run_agent_service.py --base-url ... --once "What is 17 * 23?"

``--base-url`` is the chat endpoint the agent thinks with: the proxy rollout server of a training job (then every
conversation is recorded for training), an inference gateway (``services/inference_service.py``) or any other
OpenAI-compatible server. Requests can also be sent directly:

    curl -X POST http://127.0.0.1:<port>/v1/responses -H 'Authorization: Bearer areal-agent-admin' \\
         -H 'Content-Type: application/json' \\
         -d '{"input": [{"type": "message", "content": "Explain GRPO in two sentences"}], "user": "my-session"}'

Reference: examples/agent_service/run_agent_service.py."""

from __future__ import annotations

import argparse
import os
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from areal_b200.infra.utils.http import request_with_retry  # noqa: E402
from areal_b200.services import agent_service  # noqa: E402
from areal_b200.utils.network import find_free_ports  # noqa: E402


def serve(app, port: int) -> threading.Thread:
    import uvicorn

    server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="warning"))
    t = threading.Thread(target=server.run, daemon=True)
    t.start()
    return t


def wait_ready(url: str, timeout: float = 30.0):
    t0 = time.time()
    while time.time() - t0 < timeout:
        try:
            if request_with_retry("GET", url, max_retries=0, timeout=2).status_code == 200:
                return
        except Exception:
            time.sleep(0.2)
    raise TimeoutError(url)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--base-url", required=True, help="OpenAI-compatible endpoint the agent calls (…/v1)")
    ap.add_argument("--api-key", default=os.environ.get("OPENAI_API_KEY"))
    ap.add_argument("--model", default="default")
    ap.add_argument("--workers", type=int, default=2)
    ap.add_argument("--token", default="areal-agent-admin")
    ap.add_argument("--once", default=None, help="ask one question and exit instead of the interactive prompt")
    args = ap.parse_args()

    ports = find_free_ports(args.workers + 1)
    for p in ports[:-1]:
        serve(agent_service.create_worker_app(), p)
        wait_ready(f"http://127.0.0.1:{p}/health")
    gw_port = ports[-1]
    serve(agent_service.create_gateway_app(token=args.token, agent="examples.agent_service.agent.ChatAgent",
                                           agent_kwargs={"model": args.model}, base_url=args.base_url,
                                           api_key=args.api_key), gw_port)
    gw = f"http://127.0.0.1:{gw_port}"
    headers = {"Authorization": f"Bearer {args.token}"}
    time.sleep(0.5)
    for i, p in enumerate(ports[:-1]):
        request_with_retry("POST", gw + "/register", json={"worker_id": f"w{i}", "addr": f"127.0.0.1:{p}"},
                           headers=headers, max_retries=20, timeout=5)
    print(f"agent service ready: {gw}/v1/responses ({args.workers} workers)")

    def ask(text: str, user: str) -> str:
        r = request_with_retry("POST", gw + "/v1/responses", headers=headers, max_retries=0, timeout=900,
                               json={"input": [{"type": "message", "role": "user", "content": text}], "user": user,
                                     "model": args.model})
        return r.json()["output_text"]

    if args.once is not None:
        print(ask(args.once, "once"))
        return
    while True:
        try:
            line = input("you> ").strip()
        except (EOFError, KeyboardInterrupt):
            break
        if line in ("", "exit", "quit"):
            break
        print("agent>", ask(line, "interactive"))


if __name__ == "__main__":
    main()
