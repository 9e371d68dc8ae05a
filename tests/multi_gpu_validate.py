"""Helper of test_gpu_multi.py, run under torch.distributed.run: one rank per GPU validates the
token-sharded operator chain against an unsharded run through an NCCL all-gather."""
import importlib
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = importlib.import_module("qwen3x-orin_b200")
    pkg.capi.load()
    shard = importlib.import_module("qwen3x-orin_b200.shard")
    report = shard.validate_sharded_chain(rank, world, tokens_per_rank=512, layers=4)
    ok = torch.tensor([int(report["local_equals_unsharded"] and report["gathered_equals_unsharded"])], device="cuda")
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        report["all_ranks_bit_exact"] = bool(ok.item())
        print("REPORT " + json.dumps(report), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0 if ok.item() else 1


if __name__ == "__main__":
    sys.exit(main())
