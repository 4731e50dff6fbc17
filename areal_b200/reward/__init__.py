"""Rule-based reward functions. Signature used by the workflows:
``reward_fn(prompt, completion, prompt_ids, completion_ids, **dataset_fields) -> float``."""

from .math_parser import extract_answer, math_equal  # noqa: F401
from .gsm8k import gsm8k_reward_fn  # noqa: F401
from .geometry3k import geometry3k_reward_fn  # noqa: F401
from .clevr_count_70k import clevr_count_70k_reward_fn  # noqa: F401


def get_custom_reward_fn(path: str, **kwargs):
    """Dataset path/name → reward function (areal/reward/__init__.py)."""
    p = path.lower()
    if "gsm8k" in p:
        return gsm8k_reward_fn
    if "geometry3k" in p:
        return geometry3k_reward_fn
    if "clevr_count_70k" in p:
        return clevr_count_70k_reward_fn
    raise ValueError(f"no reward function registered for dataset {path!r}")


class MathVerifyWorker:
    """Answer checker with the interface of the reference's math-verify worker (areal/reward/__init__.py):
    ``verify(response, ground_truth) -> 0.0 | 1.0``. Uses the ``math_verify`` package when it is installed
    (LaTeX-aware parsing and symbolic comparison); otherwise this package's own parser (last ``\\boxed{}`` /
    ``####`` / number, numeric and normalised-string equality). Never raises: a response that cannot be parsed
    scores 0."""

    def __init__(self, try_extract_without_anchor: bool = True, precision: int = 6):
        self.precision = precision
        self.try_extract_without_anchor = try_extract_without_anchor
        try:
            import math_verify  # noqa: F401

            self._mv = math_verify
        except ImportError:
            self._mv = None

    def verify(self, response: str, ground_truth: str) -> float:
        try:
            if self._mv is not None:
                gold = self._mv.parse(ground_truth if "$" in ground_truth or "\\boxed" in ground_truth
                                      else f"${ground_truth}$")
                pred = self._mv.parse(response)
                return float(bool(self._mv.verify(gold, pred, float_rounding=self.precision)))
            ref = extract_answer(ground_truth) or ground_truth
            return float(math_equal(extract_answer(response), ref, rel_tol=10.0 ** -self.precision))
        except Exception:  # noqa: BLE001 - a malformed response is a wrong answer, not an error
            return 0.0


_MATH_VERIFY_WORKER: MathVerifyWorker | None = None


def get_math_verify_worker() -> MathVerifyWorker:
    """One checker per process (reward functions run in pool workers: each builds its own on first use)."""
    global _MATH_VERIFY_WORKER
    if _MATH_VERIFY_WORKER is None:
        _MATH_VERIFY_WORKER = MathVerifyWorker()
    return _MATH_VERIFY_WORKER
