"""Structured errors that carry a category, a sub-category and a reason (areal/utils/errors.py): RPC layers
serialise the three fields and rebuild the exception on the caller's side."""


class _Structured(Exception):
    def __init__(self, error_type: str, sub_error: str, reason: str):
        self.error_type, self.sub_error, self.reason = error_type, sub_error, reason
        super().__init__(f"error_type: {error_type}, sub_error: {sub_error}, reason: {reason}")

    def to_dict(self) -> dict[str, str]:
        return {"kind": type(self).__name__, "error_type": self.error_type, "sub_error": self.sub_error,
                "reason": self.reason}

    @classmethod
    def from_dict(cls, d: dict[str, str]) -> "_Structured":
        kinds = {c.__name__: c for c in (EngineError, FrameworkError)}
        return kinds.get(d.get("kind", ""), cls)(d["error_type"], d["sub_error"], d["reason"])


class EngineError(_Structured):
    """Raised by a train or inference engine (bad request, failed update, lost worker)."""


class FrameworkError(_Structured):
    """Raised by the orchestration around the engines (configuration, scheduling, data flow)."""
