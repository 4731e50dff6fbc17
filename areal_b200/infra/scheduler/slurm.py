"""Slurm scheduler: every role becomes one ``sbatch`` array-like job whose tasks run the worker
RPC server under ``srun``; workers publish ``host:port`` through ``name_resolve`` (NFS), the
scheduler discovers them there, checks job state with ``squeue`` / ``sacct`` and cancels with
``scancel``. Engine calls reuse the HTTP client logic of the local scheduler.

Counterpart of areal/infra/scheduler/slurm.py:72-1814 in the reference (sbatch script generation
:800, job status :216, network discovery :349). All Slurm commands go through ``self.run_cmd`` so
the logic is testable without a cluster.
"""

from __future__ import annotations

import os
import re
import shlex
import subprocess
import time
from dataclasses import dataclass

import requests

from ...api.cli_args import NameResolveConfig, SchedulingSpec
from ...api.scheduler_api import Job, Worker
from ...utils import logging, name_resolve
from .exceptions import WorkerCreationError, WorkerFailedError, WorkerNotFoundError, WorkerTimeoutError
from .local import LocalScheduler, _WorkerInfo

logger = logging.getLogger("SlurmScheduler")

_BAD_STATES = {"FAILED", "CANCELLED", "TIMEOUT", "NODE_FAIL", "OUT_OF_MEMORY", "BOOT_FAIL", "DEADLINE", "PREEMPTED"}


@dataclass
class SlurmJobState:
    job_id: str
    state: str  # PENDING | RUNNING | COMPLETED | FAILED | ...
    nodes: str = ""


def _default_run(cmd: list[str]) -> str:
    return subprocess.run(cmd, check=True, capture_output=True, text=True).stdout


class SlurmScheduler(LocalScheduler):
    def __init__(self, experiment_name: str, trial_name: str, fileroot: str, n_gpus_per_node: int = 8,
                 partition: str | None = None, account: str | None = None, time_limit: str | None = None,
                 startup_timeout: float = 600.0, run_cmd=None, name_resolve_root: str | None = None, **kw):
        super().__init__(gpu_devices=[], log_dir=os.path.join(fileroot, "logs", experiment_name, trial_name, "slurm"),
                         startup_timeout=startup_timeout, **kw)
        self.experiment_name, self.trial_name, self.fileroot = experiment_name, trial_name, fileroot
        self.n_gpus_per_node = n_gpus_per_node
        self.partition, self.account, self.time_limit = partition, account, time_limit
        self.run_cmd = run_cmd or _default_run
        self.nr_root = name_resolve_root or os.path.join(fileroot, "name_resolve")
        name_resolve.reconfigure(NameResolveConfig(type="nfs", nfs_record_root=self.nr_root))
        self._jobs: dict[str, str] = {}  # role -> slurm job id

    # ------------------------------------------------------------- sbatch
    def _worker_key(self, role: str, i: int) -> str:
        return f"{self.experiment_name}/{self.trial_name}/workers/{role}/{i}"

    def render_sbatch(self, job: Job) -> str:
        """The batch script of one role: ``replicas`` tasks, ``gpu`` GPUs each, packed onto nodes."""
        spec: SchedulingSpec = (job.tasks[0] if job.tasks else SchedulingSpec())
        n = job.replicas
        gpus = max(spec.gpu, 0)
        tasks_per_node = max(1, self.n_gpus_per_node // gpus) if gpus else n
        nodes = -(-n // tasks_per_node)
        lines = ["#!/bin/bash",
                 f"#SBATCH --job-name={self.experiment_name}_{self.trial_name}:{job.role}",
                 f"#SBATCH --output={os.path.join(self.log_dir, job.role.replace('/', '_'))}_%j.out",
                 f"#SBATCH --nodes={nodes}", f"#SBATCH --ntasks={n}", f"#SBATCH --ntasks-per-node={min(tasks_per_node, n)}",
                 f"#SBATCH --cpus-per-task={spec.cpu}", f"#SBATCH --mem-per-cpu={max(spec.mem * 1024 // max(spec.cpu, 1), 1)}M"]
        if gpus:
            lines.append(f"#SBATCH --gres=gpu:{min(gpus * min(tasks_per_node, n), self.n_gpus_per_node)}")
        for flag, val in (("partition", self.partition), ("account", self.account), ("time", self.time_limit),
                          ("nodelist", spec.nodelist), ("exclude", spec.exclude)):
            if val:
                lines.append(f"#SBATCH --{flag}={val}")
        lines.append("")
        for k, v in (spec.env_vars or {}).items():
            lines.append(f"export {k}={shlex.quote(str(v))}")
        lines += list(spec.additional_bash_cmds or [])
        cmd = spec.cmd or self.worker_command
        key = f"{self.experiment_name}/{self.trial_name}/workers/{job.role}/$SLURM_PROCID"
        inner = (f"{cmd} --host $(hostname -i | awk '{{print $1}}') --port 0 --name-key {key} "
                 f"--nfs-record-root {self.nr_root}")
        if gpus:
            inner = (f"CUDA_VISIBLE_DEVICES=$(seq -s, $((SLURM_LOCALID*{gpus})) $((SLURM_LOCALID*{gpus}+{gpus - 1}))) "
                     + inner)
        wrapped = f"bash -c {shlex.quote(inner)}"
        if spec.image and spec.container_type in ("apptainer", "singularity"):
            wrapped = f"{spec.container_type} exec --nv --bind {spec.mount} {spec.image} {wrapped}"
        lines.append(f"srun {spec.srun_additional_args} {wrapped}")
        return "\n".join(lines) + "\n"

    def create_workers(self, job: Job, *args, **kwargs) -> list[str]:
        role = job.role
        if role in self._workers:
            raise WorkerCreationError(role, "role already exists", "delete it first")
        if job.replicas <= 0:
            raise WorkerCreationError(role, "invalid configuration", "replicas must be positive")
        script = os.path.join(self.log_dir, f"{role.replace('/', '_')}.sbatch")
        with open(script, "w") as f:
            f.write(self.render_sbatch(job))
        try:
            out = self.run_cmd(["sbatch", "--parsable", script])
        except Exception as e:
            raise WorkerCreationError(role, "sbatch failed", str(e)) from e
        job_id = out.strip().split(";")[0]
        if not re.fullmatch(r"\d+", job_id):
            raise WorkerCreationError(role, "sbatch failed", f"unexpected output {out!r}")
        self._jobs[role] = job_id
        infos = [_WorkerInfo(Worker(id=f"{role}/{i}", ip="", worker_ports=[]), None, role) for i in range(job.replicas)]
        self._workers[role] = infos
        for info in infos:
            self._by_id[info.worker.id] = info
        logger.info(f"submitted slurm job {job_id} for role {role} ({job.replicas} tasks)")
        return [i.worker.id for i in infos]

    # -------------------------------------------------------------- status
    def job_state(self, role: str) -> SlurmJobState:
        job_id = self._jobs[role]
        out = self.run_cmd(["squeue", "-h", "-j", job_id, "-o", "%T|%N"]).strip()
        if not out:  # left the queue: ask the accounting database
            out = self.run_cmd(["sacct", "-n", "-X", "-j", job_id, "-o", "State,NodeList", "-P"]).strip()
        first = out.splitlines()[0] if out else "UNKNOWN|"
        state, _, nodes = first.partition("|")
        return SlurmJobState(job_id, state.split()[0] if state else "UNKNOWN", nodes)

    def _check_alive(self, info: _WorkerInfo):
        st = self.job_state(info.role)
        if st.state in _BAD_STATES or (st.state == "COMPLETED"):
            raise WorkerFailedError(info.worker.id, -1, f"slurm job {st.job_id} is {st.state}")

    def get_workers(self, role: str, timeout: float | None = None) -> list[Worker]:
        if role not in self._workers:
            raise WorkerNotFoundError(role)
        limit = timeout if timeout is not None else self.startup_timeout
        deadline = time.monotonic() + limit
        pending = list(enumerate(self._workers[role]))
        while pending:
            self._check_alive(pending[0][1])
            for i, info in list(pending):
                if not info.worker.worker_ports:
                    try:
                        addr = name_resolve.get(self._worker_key(role, i))
                    except Exception:
                        continue
                    host, _, port = addr.rpartition(":")
                    info.worker.ip, info.worker.worker_ports = host, [port]
                try:
                    if requests.get(f"http://{self._addr(info)}/health", timeout=2).status_code == 200:
                        pending.remove((i, info))
                except requests.RequestException:
                    pass
            if pending:
                if time.monotonic() > deadline:
                    raise WorkerTimeoutError(role, limit)
                time.sleep(self.health_interval)
        return [i.worker for i in self._workers[role]]

    def _terminate(self, info: _WorkerInfo):
        job_id = self._jobs.pop(info.role, None)
        if job_id is not None:
            try:
                self.run_cmd(["scancel", job_id])
            except Exception as e:
                logger.warning(f"scancel {job_id} failed: {e}")

    def fork_workers(self, role: str, target_role: str, command: str | None = None) -> list[str]:
        # forks are started by the parent worker's RPC server on its own node
        return super().fork_workers(role, target_role, command)
