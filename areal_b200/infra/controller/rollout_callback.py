"""Trainer-side handle of a rollout controller that lives in another process: the train engine's
weight-update path calls ``pause_generation`` / ``continue_generation`` / ``set_version`` /
``update_weights_from_disk`` on it and the handle POSTs them to the controller's callback server.
Reference: areal/infra/controller/rollout_callback.py."""

from __future__ import annotations

from concurrent.futures import Future, ThreadPoolExecutor

from ...api.io_struct import WeightUpdateMeta
from ..rpc.serialization import deserialize_value, serialize_value
from ..utils.http import request_with_retry


class RolloutCallback:
    def __init__(self, controller_addr: str, timeout: float = 3600.0, max_retries: int = 3):
        self.addr, self.timeout, self.max_retries = controller_addr.rstrip("/"), timeout, max_retries
        if not self.addr.startswith("http"):
            self.addr = "http://" + self.addr
        self._pool = ThreadPoolExecutor(max_workers=2, thread_name_prefix="rollout-cb")

    def _post(self, route: str, **payload):
        r = request_with_retry("POST", f"{self.addr}/callback/{route}", json=serialize_value(payload),
                               timeout=self.timeout, max_retries=self.max_retries)
        body = r.json()
        return deserialize_value(body.get("result")) if isinstance(body, dict) else None

    def pause_generation(self):
        return self._post("pause_generation")

    def continue_generation(self):
        return self._post("continue_generation")

    def set_version(self, version: int):
        return self._post("set_version", version=version)

    def get_version(self) -> int:
        return int(self._post("get_version"))

    def update_weights_from_disk(self, meta: WeightUpdateMeta) -> Future:
        return self._pool.submit(self._post, "update_weights_from_disk", meta=meta)

    def init_weights_update_group(self, meta: WeightUpdateMeta) -> Future:
        return self._pool.submit(self._post, "init_weights_update_group", meta=meta)

    def update_weights_from_distributed(self, meta: WeightUpdateMeta, param_specs) -> Future:
        return self._pool.submit(self._post, "update_weights_from_distributed", meta=meta, param_specs=param_specs)
