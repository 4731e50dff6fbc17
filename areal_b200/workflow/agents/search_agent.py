"""Question answering with a search tool: a ReAct-style agent on the chat-completions protocol.

The policy may call ``search(query)`` (ranked snippets) and ``visit(doc_id)`` (one document's text) any
number of times within ``max_turns`` requests and must finish with ``<answer>...</answer>``. The reward is
the token-level F1 (or exact match) between the normalised final answer and the gold answers; an episode
that never answers gets 0.

Retrieval backends:

* :class:`LocalCorpus` – BM25 over a local ``.jsonl`` corpus (``{"id", "title", "text"}`` per line), built
  in process; enough for offline corpora of a few hundred thousand passages and for tests.
* :class:`HttpSearch` – ``POST {url}/search {"query", "top_k"}`` and ``POST {url}/visit {"id"}`` against a
  retrieval service that the user runs (dense retriever, web search bridge).

Reference behaviour: examples/search_agent/tongyi_deepresearch/{react_agent.py, tool_search.py,
tool_visit.py, train.py} (multi-turn tool loop whose every completion is a training sample, answer
judged against the gold answer).
"""

from __future__ import annotations

import json
import math
import re
import string
from collections import Counter
from typing import Any, Protocol

from .math_agent import _client, _get, _message_dict

_WORD = re.compile(r"[a-z0-9]+")
_ANSWER = re.compile(r"<answer>(.*?)</answer>", re.S | re.I)

SEARCH_INSTRUCTIONS = (
    "You answer questions by looking things up. Use the `search` tool to find passages and the `visit` tool to "
    "read a passage in full; search again with other words when the results do not help. When you know the "
    "answer, reply with the shortest exact answer inside <answer></answer> tags.")


def _tool(name: str, doc: str, params: dict[str, str]) -> dict[str, Any]:
    return {"type": "function", "function": {
        "name": name, "description": doc,
        "parameters": {"type": "object", "properties": {p: {"type": t} for p, t in params.items()},
                       "required": list(params)}}}


SEARCH_TOOLS = [
    _tool("search", "Search the corpus; returns the best passages with their ids.", {"query": "string"}),
    _tool("visit", "Return the full text of the passage with this id.", {"doc_id": "string"}),
]


# --------------------------------------------------------------------------------------- scoring
def normalize_answer(s: str) -> str:
    """Lower case, no punctuation, no articles, single spaces (the usual open-domain QA normalisation)."""
    s = "".join(ch for ch in s.lower() if ch not in set(string.punctuation))
    s = re.sub(r"\b(a|an|the)\b", " ", s)
    return " ".join(s.split())


def qa_f1(prediction: str, gold: str) -> float:
    p, g = normalize_answer(prediction).split(), normalize_answer(gold).split()
    if not p or not g:
        return float(p == g)
    common = sum((Counter(p) & Counter(g)).values())
    if common == 0:
        return 0.0
    precision, recall = common / len(p), common / len(g)
    return 2 * precision * recall / (precision + recall)


def extract_final_answer(text: str | None) -> str | None:
    found = _ANSWER.findall(text or "")
    return found[-1].strip() if found else None


def qa_reward(completion: str | None, answers: str | list[str], metric: str = "f1") -> float:
    """Best score of the tagged final answer over the gold answers; 0 without a tagged answer."""
    pred = extract_final_answer(completion)
    if pred is None:
        return 0.0
    golds = [answers] if isinstance(answers, str) else list(answers)
    if metric == "em":
        return float(any(normalize_answer(pred) == normalize_answer(g) for g in golds))
    return max((qa_f1(pred, g) for g in golds), default=0.0)


# --------------------------------------------------------------------------------------- retrieval
class SearchBackend(Protocol):
    def search(self, query: str, top_k: int = 5) -> list[dict[str, Any]]: ...

    def visit(self, doc_id: str) -> str | None: ...


class LocalCorpus:
    """Okapi BM25 over an in-memory corpus with an inverted index (term → postings)."""

    def __init__(self, docs: list[dict[str, Any]], k1: float = 1.5, b: float = 0.75, snippet_chars: int = 240):
        self.docs = {str(d.get("id", i)): d for i, d in enumerate(docs)}
        self.k1, self.b, self.snippet_chars = k1, b, snippet_chars
        self.postings: dict[str, list[tuple[str, int]]] = {}
        self.length: dict[str, int] = {}
        for doc_id, d in self.docs.items():
            toks = _WORD.findall((d.get("title", "") + " " + d.get("text", "")).lower())
            self.length[doc_id] = len(toks)
            for term, tf in Counter(toks).items():
                self.postings.setdefault(term, []).append((doc_id, tf))
        self.avg_len = (sum(self.length.values()) / len(self.length)) if self.length else 0.0

    @classmethod
    def from_jsonl(cls, path: str, **kw) -> "LocalCorpus":
        with open(path) as f:
            return cls([json.loads(line) for line in f if line.strip()], **kw)

    def search(self, query: str, top_k: int = 5) -> list[dict[str, Any]]:
        n = len(self.docs)
        scores: dict[str, float] = {}
        for term in set(_WORD.findall(query.lower())):
            post = self.postings.get(term)
            if not post:
                continue
            idf = math.log(1.0 + (n - len(post) + 0.5) / (len(post) + 0.5))
            for doc_id, tf in post:
                norm = tf + self.k1 * (1 - self.b + self.b * self.length[doc_id] / max(self.avg_len, 1e-9))
                scores[doc_id] = scores.get(doc_id, 0.0) + idf * tf * (self.k1 + 1) / norm
        best = sorted(scores.items(), key=lambda kv: (-kv[1], kv[0]))[:top_k]
        return [{"id": i, "title": self.docs[i].get("title", ""), "score": round(s, 4),
                 "snippet": self.docs[i].get("text", "")[: self.snippet_chars]} for i, s in best]

    def visit(self, doc_id: str) -> str | None:
        d = self.docs.get(str(doc_id))
        return None if d is None else d.get("text", "")


class HttpSearch:
    """Client of a retrieval service: ``/search`` → ``{"results": [{"id","title","snippet"}...]}``,
    ``/visit`` → ``{"text": ...}``. ``post`` is injectable (tests; other HTTP stacks)."""

    def __init__(self, url: str, timeout: float = 30.0, post=None):
        self.url, self.timeout = url.rstrip("/"), timeout
        self._post = post or self._requests_post

    def _requests_post(self, url: str, payload: dict) -> dict:
        import requests

        r = requests.post(url, json=payload, timeout=self.timeout)
        r.raise_for_status()
        return r.json()

    def search(self, query: str, top_k: int = 5) -> list[dict[str, Any]]:
        return list(self._post(f"{self.url}/search", {"query": query, "top_k": top_k}).get("results", []))

    def visit(self, doc_id: str) -> str | None:
        return self._post(f"{self.url}/visit", {"id": doc_id}).get("text")


def run_search_tool(backend: SearchBackend, name: str, arguments: str | dict, top_k: int = 5,
                    max_chars: int = 4000) -> str:
    """Executes one tool call; every failure comes back as text so the policy can react to it."""
    try:
        args = json.loads(arguments) if isinstance(arguments, str) else dict(arguments)
        if name == "search":
            hits = backend.search(str(args["query"]), top_k)
            if not hits:
                return "no results"
            return "\n".join(f"[{h['id']}] {h.get('title', '')}: {h.get('snippet', '')}" for h in hits)[:max_chars]
        if name == "visit":
            text = backend.visit(str(args["doc_id"]))
            return "error: unknown doc_id" if text is None else text[:max_chars]
        return f"error: unknown tool {name!r}"
    except Exception as e:  # noqa: BLE001 - reported back to the model
        return f"error: {type(e).__name__}: {e}"


# --------------------------------------------------------------------------------------- agent
class ReActSearchAgent:
    """``data = {"messages": [...], "answer": str | [str]}``. Stops at the first completion without tool
    calls (its text is judged) or after ``max_turns`` requests. ``invalid_penalty`` is subtracted when the
    episode ends without a tagged answer, which teaches the format early in training."""

    def __init__(self, backend: SearchBackend, max_turns: int = 6, top_k: int = 5, metric: str = "f1",
                 invalid_penalty: float = 0.0, **sampling):
        self.backend, self.max_turns, self.top_k, self.metric = backend, max_turns, top_k, metric
        self.invalid_penalty = invalid_penalty
        self.sampling = {k: v for k, v in sampling.items() if k != "max_tokens"}

    async def run(self, data: dict, **extra) -> float:
        client = _client(extra)
        messages = [{"role": "system", "content": SEARCH_INSTRUCTIONS}] + list(data["messages"])
        final = None
        for _ in range(self.max_turns):
            comp = await client.chat.completions.create(messages=messages, model="default", tools=SEARCH_TOOLS,
                                                        **self.sampling)
            message = comp.choices[0].message
            messages.append(_message_dict(message))
            calls = _get(message, "tool_calls") or []
            if not calls:
                final = _get(message, "content")
                break
            for c in calls:
                fn = _get(c, "function")
                messages.append({"role": "tool", "tool_call_id": _get(c, "id"),
                                 "content": run_search_tool(self.backend, _get(fn, "name"), _get(fn, "arguments"),
                                                            self.top_k)})
        if extract_final_answer(final) is None:
            return -self.invalid_penalty
        return qa_reward(final, data["answer"], self.metric)
