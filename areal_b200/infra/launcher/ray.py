"""SPMD launcher on a Ray cluster: one Ray task per node runs ``torchrun`` for that node's ranks
(placement group with one GPU bundle set per node). Ray is optional; without it the launcher
exits with a message. Counterpart of areal/infra/launcher/ray.py in the reference."""

from __future__ import annotations

import sys

from ...api.cli_args import BaseExperimentConfig, PPOConfig, load_expr_config
from ...utils import logging
from .local import world_size_of

logger = logging.getLogger("RayLauncher")


def node_plan(nproc: int, gpus_per_node: int) -> list[int]:
    """Ranks per node."""
    full, rest = divmod(nproc, gpus_per_node)
    return [gpus_per_node] * full + ([rest] if rest else [])


def ray_main(argv: list[str]) -> int:
    try:
        import ray
    except ImportError:
        raise SystemExit("the Ray launcher needs the 'ray' package, which is not installed; use the local or Slurm launcher")
    if not argv:
        raise SystemExit("usage: python -m areal_b200.infra.launcher.ray <script.py> --config cfg.yaml [overrides]")
    script, rest = argv[0], argv[1:]
    try:
        config, _ = load_expr_config(rest, PPOConfig)
    except (KeyError, TypeError):
        config, _ = load_expr_config(rest, BaseExperimentConfig)
    from ray.util.placement_group import placement_group
    from ray.util.scheduling_strategies import PlacementGroupSchedulingStrategy

    ray.init(ignore_reinit_error=True)
    plan = node_plan(world_size_of(config), config.cluster.n_gpus_per_node)
    pg = placement_group([{"GPU": n, "CPU": 8 * n} for n in plan], strategy="STRICT_SPREAD" if len(plan) > 1 else "PACK")
    ray.get(pg.ready())

    @ray.remote
    def node_ip():
        import socket

        return socket.gethostbyname(socket.gethostname())

    master = ray.get(node_ip.options(scheduling_strategy=PlacementGroupSchedulingStrategy(pg, 0)).remote())

    @ray.remote
    def run_node(node_rank: int, nproc: int):
        import os
        import subprocess

        cmd = [sys.executable, "-m", "torch.distributed.run", f"--nnodes={len(plan)}", f"--node-rank={node_rank}",
               f"--nproc-per-node={nproc}", "--master-addr", master, "--master-port", "29500", script, *rest]
        return subprocess.call(cmd, env=dict(os.environ, AREAL_SPMD_MODE="1"))

    rcs = ray.get([run_node.options(num_gpus=n, scheduling_strategy=PlacementGroupSchedulingStrategy(pg, i)).remote(i, n)
                   for i, n in enumerate(plan)])
    return max(rcs)


if __name__ == "__main__":
    sys.exit(ray_main(sys.argv[1:]))
