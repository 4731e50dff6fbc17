"""What an EXTERNAL user of online training runs: any program that speaks the OpenAI API against the
gateway of a training job whose rollout workflow is in `online` mode.

Life cycle of one episode:

1. `POST {gateway}/rl/start_session` with the admin key → `{"session_id", "api_key"}`; the gateway binds the
   session to the rollout worker that has waited longest.
2. Chat with `base_url={gateway}/v1` and that `api_key` (OpenAI SDKs, curl, agent frameworks): every
   completion is recorded with token ids, log-probs and weight versions on the worker.
3. `POST {gateway}/rl/set_reward {"reward": r}` (optionally `"interaction_id"` for one completion).
4. `POST {gateway}/rl/end_session`: the worker's workflow exports the trajectory into the training batch.

    python examples/online_proxy/external_user.py http://gateway:8000 --admin-key areal-admin-key \
        --question "What is 6 times 7?" --answer 42

The functions take a `post(url, json, headers) -> dict` so that tests (and other HTTP stacks) can inject theirs.
"""
import argparse
import sys


def _requests_post(url, body, headers):
    import requests

    r = requests.post(url, json=body, headers=headers, timeout=600)
    r.raise_for_status()
    return r.json()


def start_session(gateway: str, admin_key: str, post=_requests_post) -> dict:
    return post(f"{gateway}/rl/start_session", {}, {"Authorization": f"Bearer {admin_key}"})


def chat(gateway: str, api_key: str, messages: list[dict], post=_requests_post, **sampling) -> dict:
    return post(f"{gateway}/v1/chat/completions", dict(messages=messages, model="default", **sampling),
                {"Authorization": f"Bearer {api_key}"})


def set_reward(gateway: str, api_key: str, reward: float, interaction_id: str | None = None, post=_requests_post):
    body = {"reward": float(reward)}
    if interaction_id is not None:
        body["interaction_id"] = interaction_id
    return post(f"{gateway}/rl/set_reward", body, {"Authorization": f"Bearer {api_key}"})


def end_session(gateway: str, api_key: str, post=_requests_post):
    return post(f"{gateway}/rl/end_session", {}, {"Authorization": f"Bearer {api_key}"})


def run_episode(gateway: str, admin_key: str, question: str, answer: str, post=_requests_post, max_tokens: int = 256):
    """One rewarded question: 1.0 if the reply contains the expected answer."""
    gateway = gateway.rstrip("/")
    sess = start_session(gateway, admin_key, post)
    try:
        reply = chat(gateway, sess["api_key"], [{"role": "user", "content": question}], post, max_tokens=max_tokens)
        text = reply["choices"][0]["message"].get("content") or ""
        reward = float(str(answer) in text)
        set_reward(gateway, sess["api_key"], reward, reply["id"], post)
    finally:
        end_session(gateway, sess["api_key"], post)
    return {"session_id": sess["session_id"], "reward": reward, "text": text}


def main(argv):
    ap = argparse.ArgumentParser()
    ap.add_argument("gateway")
    ap.add_argument("--admin-key", default="areal-admin-key")
    ap.add_argument("--question", default="What is 6 times 7?")
    ap.add_argument("--answer", default="42")
    ap.add_argument("--episodes", type=int, default=1)
    args = ap.parse_args(argv)
    for _ in range(args.episodes):
        print(run_episode(args.gateway, args.admin_key, args.question, args.answer))


if __name__ == "__main__":
    main(sys.argv[1:])
