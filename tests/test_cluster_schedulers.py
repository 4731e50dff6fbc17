"""Slurm scheduler against scripted sbatch / squeue / scancel and a real local worker process
that registers itself through name_resolve; Ray scheduler's placement logic and its import gate."""
import os
import subprocess
import sys
import time

import pytest

from areal_b200.api.cli_args import SchedulingSpec
from areal_b200.api.scheduler_api import Job
from areal_b200.infra.scheduler.exceptions import WorkerFailedError
from areal_b200.infra.scheduler.ray import placement_bundles
from areal_b200.infra.scheduler.slurm import SlurmScheduler


def test_sbatch_script_and_lifecycle(tmp_path):
    procs, calls = [], []
    state = {"s": "RUNNING"}
    sched_box = {}

    def run_cmd(cmd):
        calls.append(cmd)
        if cmd[0] == "sbatch":
            sch = sched_box["s"]
            # stand-in for the cluster: start task 0 of the job as a local process
            key = f"{sch.experiment_name}/{sch.trial_name}/workers/actor/0"
            procs.append(subprocess.Popen([sys.executable, "-m", "areal_b200.infra.rpc.rpc_server", "--host", "127.0.0.1",
                                           "--port", "0", "--name-key", key, "--nfs-record-root", sch.nr_root]))
            return "4242\n"
        if cmd[0] == "squeue":
            return f"{state['s']}|node01\n"
        if cmd[0] == "scancel":
            for p in procs:
                p.terminate()
            return ""
        raise AssertionError(cmd)

    s = SlurmScheduler("exp", "trial", str(tmp_path), n_gpus_per_node=8, partition="gpu", run_cmd=run_cmd,
                       startup_timeout=60)
    sched_box["s"] = s
    job = Job(replicas=1, role="actor", tasks=[SchedulingSpec(cpu=4, gpu=2, mem=16, env_vars={"FOO": "bar"})])
    script = s.render_sbatch(Job(replicas=6, role="actor", tasks=job.tasks))
    assert "#SBATCH --ntasks=6" in script and "#SBATCH --nodes=2" in script and "#SBATCH --gres=gpu:8" in script
    assert "#SBATCH --partition=gpu" in script and "export FOO=bar" in script and "srun " in script
    try:
        ids = s.create_workers(job)
        assert ids == ["actor/0"] and calls[0][0] == "sbatch"
        workers = s.get_workers("actor", timeout=60)
        assert workers[0].worker_ports and workers[0].ip == "127.0.0.1"
        assert s.job_state("actor").state == "RUNNING"
        state["s"] = "FAILED"
        with pytest.raises(WorkerFailedError):
            s.get_workers("actor", timeout=5)
    finally:
        s.delete_workers()
        for p in procs:
            p.terminate()
    assert any(c[0] == "scancel" for c in calls)


def test_ray_placement_bundles_and_import_gate():
    job = Job(replicas=3, role="r", tasks=[SchedulingSpec(cpu=2, gpu=1, mem=4)])
    b = placement_bundles(job)
    assert len(b) == 3 and b[0]["GPU"] == 1.0 and b[0]["CPU"] == 2.0
    try:
        import ray  # noqa: F401
    except ImportError:
        from areal_b200.infra.scheduler.ray import RayScheduler

        with pytest.raises(ImportError, match="ray"):
            RayScheduler()
