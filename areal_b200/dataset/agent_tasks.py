"""Prompts for the tool-using agent examples.

* ``qa`` (paths containing ``qa``: HotpotQA / NQ / TriviaQA style files): records with ``question`` and
  ``answer`` or ``answers`` become ``{"messages", "answer"}`` with the gold answers as a list.
* ``terminal`` (paths containing ``terminal``): records ``{"instruction", "files", "checks"}`` become
  ``{"messages", "instruction", "files", "checks"}`` for :class:`~areal_b200.workflow.agents.TerminalAgent`.

Role in the reference: the dataset preparation inside examples/search_agent/tongyi_deepresearch/train.py
and examples/terminal_bench/train.py.
"""
from .loaders import load_records


def qa_rl(path, split="train", tokenizer=None, max_length=None, **kw):
    out = []
    for r in load_records(path, split):
        answers = r.get("answers", r.get("answer"))
        if answers is None:
            continue
        answers = [answers] if isinstance(answers, str) else [str(a) for a in answers]
        if tokenizer is not None and max_length is not None and len(tokenizer.encode(r["question"])) > max_length:
            continue
        out.append(dict(messages=[{"role": "user", "content": r["question"]}], answer=answers))
    return out


def terminal_rl(path, split="train", tokenizer=None, max_length=None, **kw):
    out = []
    for r in load_records(path, split):
        if not r.get("checks"):
            continue  # a task without checks cannot be rewarded
        out.append(dict(messages=[{"role": "user", "content": r["instruction"]}], instruction=r["instruction"],
                        files=dict(r.get("files") or {}), checks=list(r["checks"])))
    return out


BUILDERS = {("qa", "rl"): qa_rl, ("terminal", "rl"): terminal_rl}
