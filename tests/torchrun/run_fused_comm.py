"""Worker: symmetric-memory collectives and fused compute+collective GEMMs against NCCL /
PyTorch references on N GPUs (``areal_b200.parallel.selfcheck``). Writes timings and max errors as JSON (rank 0)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from areal_b200.parallel.selfcheck import fused_comm_check  # noqa: E402


def main(out_path):
    rank = int(os.environ["RANK"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    res = fused_comm_check()
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(res, f)
        print(json.dumps(res))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1])
