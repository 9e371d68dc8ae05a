"""Token-row sharding (qwen3x-orin_b200/shard.py): partition arithmetic, and a world-size-2 run on
CPU (gloo) that shards a prompt by rows, runs the row-local oracle ops on each rank's rows with the
conv halo read from the raw tensor, all-gathers the outputs for validation and compares them with
the unsharded result bit for bit.  No collective is on the data path; the gather is validation only."""
import importlib
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
shard = importlib.import_module("qwen3x-orin_b200.shard")


def test_partition_is_contiguous_chunk_aligned_and_balanced():
    for total, world in [(131072, 8), (60000, 8), (60000, 4), (60000, 1), (513, 2), (512, 4), (1, 8), (0, 2), (1500, 3)]:
        parts = shard.partition(total, world)
        assert len(parts) == world and parts[0].first_token == 0
        assert sum(p.tokens for p in parts) == total
        for a, b in zip(parts, parts[1:]):
            assert a.end_token == b.first_token
        for p in parts:
            if p.tokens and p.end_token != total:
                assert p.first_token % shard.CHUNK == 0 and p.tokens % shard.CHUNK == 0
        sizes = [-(-p.tokens // shard.CHUNK) for p in parts]
        assert max(sizes) - min(sizes) <= 1
    p = shard.partition(131072, 8)
    assert all(x.tokens == 16384 for x in p)
    p = shard.partition(60000, 8)   # 117 full chunks + a 96-token tail
    assert [x.tokens for x in p][:5] == [7680] * 5 and p[-1].end_token == 60000
    assert shard.shard_for(60000, 3, 8) == p[3]
    assert shard.shard_for(2048, 1, 2).halo_first == 1021 and shard.shard_for(2048, 0, 2).halo_first == 0
    with pytest.raises(ValueError):
        shard.partition(10, 0)
    with pytest.raises(ValueError):
        shard.shard_for(10, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, total, out_dir):
    sys.path.insert(0, ROOT)
    from oracle import oracle as orc

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # every rank regenerates the same seeded prompt, then keeps only its rows
        rng = np.random.default_rng(7)
        raw = orc.bf16_encode(rng.standard_normal((total, 10240)).astype(np.float32))
        cw = orc.bf16_encode((rng.standard_normal((10240, 4)) * 0.5).astype(np.float32))
        left = orc.bf16_encode(rng.standard_normal((total, 5120)).astype(np.float32))
        right = orc.bf16_encode(rng.standard_normal((total, 5120)).astype(np.float32))
        w = orc.bf16_encode((rng.standard_normal(5120) * 0.02).astype(np.float32))
        mine = shard.shard_for(total, rank, world)
        lo, hi = mine.first_token, mine.end_token
        # conv: history = the three raw rows before the shard (zero at the start of the prompt)
        hist = np.zeros((10240, 3), dtype=np.uint16)
        n_halo = lo - mine.halo_first
        if n_halo:
            hist[:, 3 - n_halo:] = raw[mine.halo_first:lo].T
        conv, _ = orc.causal_conv1d_silu(raw[lo:hi], cw, hist)
        res, nrm = orc.residual_add_rms_norm(left[lo:hi], right[lo:hi], w, 1e-6)
        codes, scales, gs = orc.nvfp4_quantize(nrm, shard.CHUNK)   # scale groups never straddle ranks
        gathered = {}
        for name, arr in (("conv", conv), ("res", res), ("nrm", nrm), ("codes", codes), ("scales", scales)):
            t = torch.from_numpy(arr.astype(np.int32))
            gathered[name] = shard.gather_rows(t, mine, total).numpy()
        if rank == 0:
            np.savez(os.path.join(out_dir, "gathered.npz"), **gathered)
    finally:
        dist.destroy_process_group()


def test_two_rank_sharded_run_matches_unsharded(tmp_path):
    from oracle import oracle as orc

    orc.build()
    total, world = 1300, 2   # 3 chunks: ranks own 1024 and 276 rows (ragged tail on the last rank)
    port = _free_port()
    mp.start_processes(_worker, args=(world, port, total, str(tmp_path)), nprocs=world, join=True, start_method="spawn")
    got = np.load(os.path.join(str(tmp_path), "gathered.npz"))
    rng = np.random.default_rng(7)
    raw = orc.bf16_encode(rng.standard_normal((total, 10240)).astype(np.float32))
    cw = orc.bf16_encode((rng.standard_normal((10240, 4)) * 0.5).astype(np.float32))
    left = orc.bf16_encode(rng.standard_normal((total, 5120)).astype(np.float32))
    right = orc.bf16_encode(rng.standard_normal((total, 5120)).astype(np.float32))
    w = orc.bf16_encode((rng.standard_normal(5120) * 0.02).astype(np.float32))
    conv, _ = orc.causal_conv1d_silu(raw, cw, np.zeros((10240, 3), dtype=np.uint16))
    res, nrm = orc.residual_add_rms_norm(left, right, w, 1e-6)
    codes, scales, _ = orc.nvfp4_quantize(nrm, shard.CHUNK)
    for name, want in (("conv", conv), ("res", res), ("nrm", nrm), ("codes", codes), ("scales", scales)):
        assert np.array_equal(got[name], want.astype(np.int32)), name
