"""Multi-GPU validation (skipped on a single GPU): token-row shards on 2 GPUs, outputs all-gathered
over NCCL and compared bit for bit with an unsharded run; plus the one-GPU form of the same check."""
import importlib
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_chain_shard_of_one_equals_itself():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    pkg = importlib.import_module("qwen3x-orin_b200")
    pkg.capi.load()
    shard = importlib.import_module("qwen3x-orin_b200.shard")
    report = shard.validate_sharded_chain(0, 1, tokens_per_rank=1024, layers=4)
    assert report["local_equals_unsharded"] and report["gathered_equals_unsharded"]


def test_two_gpu_shards_gather_to_the_unsharded_result():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_DEBUG="WARN")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29533", os.path.join(ROOT, "tests", "multi_gpu_validate.py")]
    done = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-2000:]
    line = [l for l in done.stdout.splitlines() if l.startswith("REPORT ")][-1]
    report = json.loads(line[len("REPORT "):])
    assert report["all_ranks_bit_exact"] and report["gathered_bytes"] > 0
