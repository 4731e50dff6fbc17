"""SPMD launcher for Slurm clusters.

    python -m areal_b200.infra.launcher.slurm train.py --config cfg.yaml [k=v ...]

Writes one batch script that starts ``torchrun`` on every node of the allocation (``srun``, one
launcher task per node, ``nproc-per-node`` = GPUs per node, rendezvous on the first node) and
submits it with ``sbatch``; ``--wait`` follows the job until it ends and resubmits it for
recovery like the local launcher does. Rollout and trainer ranks share the one world, so unlike
the reference (areal/infra/launcher/slurm.py, separate server and trainer job arrays) there is a
single job. Commands go through ``run_cmd`` for testability.
"""

from __future__ import annotations

import os
import shlex
import subprocess
import sys
import time

from ...api.cli_args import BaseExperimentConfig, PPOConfig, load_expr_config
from ...utils import logging
from .local import world_size_of

logger = logging.getLogger("SlurmLauncher")


def render_job(script_args: list[str], nproc: int, gpus_per_node: int, job_name: str, log_path: str,
               cpus_per_gpu: int = 12, mem_per_gpu_gb: int = 100, partition: str | None = None,
               account: str | None = None, time_limit: str | None = None, env: dict[str, str] | None = None,
               port: int = 29500) -> str:
    nodes = -(-nproc // gpus_per_node)
    per_node = min(gpus_per_node, nproc)
    lines = ["#!/bin/bash", f"#SBATCH --job-name={job_name}", f"#SBATCH --output={log_path}",
             f"#SBATCH --nodes={nodes}", "#SBATCH --ntasks-per-node=1", f"#SBATCH --gres=gpu:{per_node}",
             f"#SBATCH --cpus-per-task={cpus_per_gpu * per_node}", f"#SBATCH --mem={mem_per_gpu_gb * per_node}G"]
    for flag, val in (("partition", partition), ("account", account), ("time", time_limit)):
        if val:
            lines.append(f"#SBATCH --{flag}={val}")
    lines += ["", "export AREAL_SPMD_MODE=1",
              "MASTER=$(scontrol show hostnames $SLURM_JOB_NODELIST | head -n 1)"]
    for k, v in (env or {}).items():
        lines.append(f"export {k}={shlex.quote(str(v))}")
    torchrun = (f"{sys.executable} -m torch.distributed.run --nnodes={nodes} --nproc-per-node={per_node} "
                f"--rdzv-backend=c10d --rdzv-endpoint=$MASTER:{port} --rdzv-id=$SLURM_JOB_ID "
                + " ".join(shlex.quote(a) for a in script_args))
    lines.append(f"srun --unbuffered --kill-on-bad-exit=1 bash -c {shlex.quote(torchrun)}")
    return "\n".join(lines) + "\n"


class SlurmLauncher:
    def __init__(self, experiment_name: str, trial_name: str, fileroot: str, run_cmd=None):
        self.experiment_name, self.trial_name, self.fileroot = experiment_name, trial_name, fileroot
        self.run_cmd = run_cmd or (lambda cmd: subprocess.run(cmd, check=True, capture_output=True, text=True).stdout)
        self.job_id: str | None = None

    def log_dir(self) -> str:
        d = os.path.join(self.fileroot, "logs", os.environ.get("USER", "user"), self.experiment_name, self.trial_name)
        os.makedirs(d, exist_ok=True)
        return d

    def submit(self, script_args: list[str], nproc: int, gpus_per_node: int = 8, **kw) -> str:
        path = os.path.join(self.log_dir(), "job.sbatch")
        with open(path, "w") as f:
            f.write(render_job(script_args, nproc, gpus_per_node, f"{self.experiment_name}_{self.trial_name}",
                               os.path.join(self.log_dir(), "slurm_%j.out"), **kw))
        self.job_id = self.run_cmd(["sbatch", "--parsable", path]).strip().split(";")[0]
        logger.info(f"submitted slurm job {self.job_id}")
        return self.job_id

    def state(self) -> str:
        out = self.run_cmd(["squeue", "-h", "-j", self.job_id, "-o", "%T"]).strip()
        if out:
            return out.splitlines()[0]
        out = self.run_cmd(["sacct", "-n", "-X", "-j", self.job_id, "-o", "State", "-P"]).strip()
        return out.splitlines()[0].split()[0] if out else "UNKNOWN"

    def wait(self, poll: float = 10.0) -> str:
        while True:
            st = self.state()
            if st not in ("PENDING", "RUNNING", "CONFIGURING", "COMPLETING"):
                return st
            time.sleep(poll)

    def stop(self):
        if self.job_id is not None:
            self.run_cmd(["scancel", self.job_id])


def slurm_main(argv: list[str]) -> int:
    wait = "--wait" in argv
    argv = [a for a in argv if a != "--wait"]
    if not argv:
        raise SystemExit("usage: python -m areal_b200.infra.launcher.slurm [--wait] <script.py> --config cfg.yaml [overrides]")
    script, rest = argv[0], argv[1:]
    try:
        config, _ = load_expr_config(rest, PPOConfig)
    except (KeyError, TypeError):
        config, _ = load_expr_config(rest, BaseExperimentConfig)
    launcher = SlurmLauncher(config.experiment_name, config.trial_name, config.cluster.fileroot)
    retries = config.recover.retries if config.recover.mode in ("auto", "fault") else 0
    attempt = 0
    while True:
        launcher.submit([script, *rest], world_size_of(config), gpus_per_node=config.cluster.n_gpus_per_node,
                        env={"AREAL_RECOVER_RUN": str(attempt)})
        if not wait:
            print(launcher.job_id)
            return 0
        st = launcher.wait()
        if st == "COMPLETED":
            return 0
        attempt += 1
        if attempt > retries:
            logger.error(f"job ended in state {st} after {attempt} attempt(s)")
            return 1


if __name__ == "__main__":
    sys.exit(slurm_main(sys.argv[1:]))
