"""Typed scheduler errors (areal/infra/scheduler/exceptions.py)."""


class SchedulerError(Exception):
    pass


class WorkerCreationError(SchedulerError):
    def __init__(self, role: str, reason: str, detail: str = ""):
        super().__init__(f"failed to create worker(s) for role {role!r}: {reason}. {detail}".strip())
        self.role, self.reason, self.detail = role, reason, detail


class WorkerFailedError(SchedulerError):
    def __init__(self, worker_id: str, exit_code: int | None, stderr: str = ""):
        super().__init__(f"worker {worker_id} exited with code {exit_code}. {stderr[-2000:]}")
        self.worker_id, self.exit_code, self.stderr = worker_id, exit_code, stderr


class WorkerNotFoundError(SchedulerError):
    def __init__(self, worker_id: str):
        super().__init__(f"worker {worker_id} is not known to the scheduler")
        self.worker_id = worker_id


class WorkerTimeoutError(SchedulerError):
    def __init__(self, role: str, timeout: float):
        super().__init__(f"workers of role {role!r} were not ready within {timeout}s")
        self.role, self.timeout = role, timeout


class EngineCreationError(SchedulerError):
    def __init__(self, worker_id: str, detail: str, status: int | None = None):
        super().__init__(f"engine creation on {worker_id} failed ({status}): {detail}")
        self.worker_id, self.detail, self.status = worker_id, detail, status


class EngineCallError(SchedulerError):
    def __init__(self, worker_id: str, method: str, detail: str, attempt: int = 1):
        super().__init__(f"{method} on {worker_id} failed after {attempt} attempt(s): {detail}")
        self.worker_id, self.method, self.detail, self.attempt = worker_id, method, detail, attempt


class RPCConnectionError(SchedulerError):
    def __init__(self, worker_id: str, addr: str, detail: str):
        super().__init__(f"cannot reach worker {worker_id} at {addr}: {detail}")
        self.worker_id, self.addr = worker_id, addr


class GPUAllocationError(SchedulerError):
    pass


class PortAllocationError(SchedulerError):
    pass
