"""Worker: the data-parallel ranks hold rollout batches of very different token counts; after redistribution every
rank holds the same number of samples, groups intact, token counts close, and nothing is lost or duplicated."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from areal_b200.infra.dist_rollout import redistribute_trajectories  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    # rank r rolled out 4 samples (2 groups of 2); rank 0's are long, the others' short
    lens = [60, 58, 50, 49] if rank == 0 else [6 + rank, 5, 4, 3]
    L = max(lens)
    mask = torch.arange(L)[None, :] < torch.tensor(lens)[:, None]
    ids = (torch.arange(4)[:, None] + 100 * rank + 1).expand(-1, L) * mask
    batch = dict(input_ids=ids, attention_mask=mask, rewards=torch.arange(4).float() + 10 * rank,
                 tags=[f"r{rank}s{i}" for i in range(4)])
    for algo in ("greedy", "kk"):
        out = redistribute_trajectories(batch, dist.group.WORLD, granularity=2, algorithm=algo)
        mine = out.data
        assert mine["attention_mask"].shape[0] == 4 and len(mine["tags"]) == 4
        tags = [None] * world
        dist.all_gather_object(tags, mine["tags"])
        flat = sorted(t for ts in tags for t in ts)
        assert flat == sorted(f"r{r}s{i}" for r in range(world) for i in range(4)), flat
        for ts in tags:            # groups (s0, s1) and (s2, s3) of a source rank stay together
            for t in ts:
                r, i = t[1:].split("s")
                assert f"r{r}s{int(i) ^ 1}" in ts
        tokens = [None] * world
        dist.all_gather_object(tokens, int(mine["attention_mask"].sum()))
        assert max(tokens) - min(tokens) <= 100 and max(tokens) < 60 + 58 + 50 + 49, tokens   # the long groups were split up
        assert out.rank == rank and sorted(i for g in out.group_indices for i in g) == list(range(4 * world))
        # rewards travelled with their rows
        for t, rw in zip(mine["tags"], mine["rewards"].tolist()):
            r, i = t[1:].split("s")
            assert rw == 10 * int(r) + int(i)
    dist.barrier()
    if rank == 0:
        print("OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
