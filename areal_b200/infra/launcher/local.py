"""SPMD launcher for one machine.

    python -m areal_b200.infra.launcher.local examples/gsm8k_grpo.py --config cfg.yaml [k=v ...]

Reads the allocation strings of the config, starts ``torchrun`` with one process
per GPU (rollout ranks first, trainer ranks after, or all colocated), sets
``AREAL_SPMD_MODE=1`` and relaunches the job up to ``recover.retries`` times when
it dies and recovery is enabled (the next attempt resumes from the last recover
checkpoint). Counterpart of areal/infra/launcher/local.py:87-440 in the
reference, where the inference servers are separate processes; here they are
ranks of the same world.
"""

from __future__ import annotations

import os
import signal
import subprocess
import sys
import time

from ...api.alloc_mode import ModelAllocation
from ...api.cli_args import BaseExperimentConfig, PPOConfig, load_expr_config
from ...utils import logging
from ..rpc.rpc_server import find_free_ports

logger = logging.getLogger("LocalLauncher")


def world_size_of(config) -> int:
    """GPUs (ranks) the experiment needs according to its allocation strings."""
    actor = getattr(config, "actor", None)
    n_train = ModelAllocation.from_str(actor.backend).world_size if actor is not None else 1
    rollout = getattr(config, "rollout", None)
    if rollout is None or rollout.backend in (None, "", "???"):
        return n_train
    n_gen = ModelAllocation.from_str(rollout.backend).world_size
    colocated = getattr(config, "allocation_mode", "") == "colocated" or \
        rollout.scheduling_strategy.type == "colocation"
    return max(n_train, n_gen) if colocated else n_train + n_gen


class LocalLauncher:
    def __init__(self, experiment_name: str, trial_name: str, fileroot: str):
        self.experiment_name, self.trial_name, self.fileroot = experiment_name, trial_name, fileroot
        self.proc: subprocess.Popen | None = None

    def log_path(self) -> str:
        d = os.path.join(self.fileroot, "logs", os.environ.get("USER", "user"), self.experiment_name, self.trial_name)
        os.makedirs(d, exist_ok=True)
        return os.path.join(d, "launcher.log")

    def submit(self, script_args: list[str], nproc: int, env: dict[str, str] | None = None) -> subprocess.Popen:
        port = find_free_ports(1)[0]
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), *script_args]
        full_env = dict(os.environ, AREAL_SPMD_MODE="1", **(env or {}))
        logger.info("launching: " + " ".join(cmd))
        self.proc = subprocess.Popen(cmd, env=full_env, start_new_session=True)
        return self.proc

    def wait(self, poll: float = 1.0) -> int:
        assert self.proc is not None
        try:
            while self.proc.poll() is None:
                time.sleep(poll)
        except KeyboardInterrupt:
            self.stop()
            raise
        return self.proc.returncode

    def stop(self):
        if self.proc is not None and self.proc.poll() is None:
            os.killpg(os.getpgid(self.proc.pid), signal.SIGTERM)
            try:
                self.proc.wait(timeout=15)
            except subprocess.TimeoutExpired:
                os.killpg(os.getpgid(self.proc.pid), signal.SIGKILL)


def local_main(argv: list[str]) -> int:
    if not argv:
        raise SystemExit("usage: python -m areal_b200.infra.launcher.local <script.py> --config cfg.yaml [overrides]")
    script, rest = argv[0], argv[1:]
    try:
        config, _ = load_expr_config(rest, PPOConfig)
    except (KeyError, TypeError):
        config, _ = load_expr_config(rest, BaseExperimentConfig)
    nproc = world_size_of(config)
    launcher = LocalLauncher(config.experiment_name, config.trial_name, config.cluster.fileroot)
    retries = config.recover.retries if config.recover.mode in ("auto", "fault") else 0
    attempt = 0
    while True:
        launcher.submit([script, *rest], nproc, env={"AREAL_RECOVER_RUN": str(attempt)})
        rc = launcher.wait()
        if rc == 0:
            return 0
        attempt += 1
        if attempt > retries:
            logger.error(f"job failed with exit code {rc} after {attempt} attempt(s)")
            return rc
        logger.warning(f"job exited with {rc}; relaunching for recovery ({attempt}/{retries})")
        time.sleep(2.0)


if __name__ == "__main__":
    sys.exit(local_main(sys.argv[1:]))
