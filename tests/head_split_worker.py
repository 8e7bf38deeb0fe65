"""Child process of tests/test_head_split_prefill_gpu.py (one per GPU, started by torchrun): runs the head-split
prefill section of the benchmarks, which raises unless the fused form equals all-gather + permute."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist

from raftinfer_b200 import benchmarks


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    torch.cuda.set_stream(torch.cuda.Stream(device=dev))
    result = benchmarks.head_split_prefill(dev, torch.cuda.current_stream(), 1679.4, rank, world, dist, tokens=1024)
    if rank == 0:
        print("fused_matches_all_gather", result["fused_matches_all_gather"], flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
