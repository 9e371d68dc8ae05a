"""Token-row sharding of a long prompt over the GPUs of one box.

Every operator of the path is row-local, so a prompt is cut into contiguous token ranges, one per
rank, with no exchange on the data path.  Ranges are aligned to the reference's 512-token prefill
chunk (include/q3x/runtime/request_state.h:18) so that (a) the scope of an NVFP4 global scale (one
chunk) never straddles two ranks and (b) a rank's results are bit-identical to the single-GPU run of
the same rows.  The causal conv needs the three raw rows before a range; they are read from the
(replicated or regenerated) raw tensor, never communicated.
"""
from __future__ import annotations

from dataclasses import dataclass

CHUNK = 512
CONV_HALO = 3


@dataclass(frozen=True)
class Shard:
    rank: int
    world: int
    first_token: int   # first token row owned by this rank
    tokens: int        # number of rows owned

    @property
    def end_token(self) -> int:
        return self.first_token + self.tokens

    @property
    def halo_first(self) -> int:
        """First raw row the conv of this shard reads (clamped at the start of the prompt)."""
        return max(0, self.first_token - CONV_HALO)


def partition(total_tokens: int, world: int, chunk: int = CHUNK) -> list[Shard]:
    """Splits [0,total_tokens) into `world` contiguous chunk-aligned ranges whose sizes differ by at
    most one chunk; the ragged tail (total % chunk) goes to the last non-empty rank."""
    if world <= 0 or total_tokens < 0 or chunk <= 0:
        raise ValueError("world and chunk must be positive, total_tokens non-negative")
    chunks = -(-total_tokens // chunk)
    base, extra = divmod(chunks, world)
    shards, first = [], 0
    for r in range(world):
        n_chunks = base + (1 if r < extra else 0)
        end = min(total_tokens, first + n_chunks * chunk)
        shards.append(Shard(r, world, first, end - first))
        first = end
    assert first == total_tokens
    return shards


def shard_for(total_tokens: int, rank: int, world: int, chunk: int = CHUNK) -> Shard:
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    return partition(total_tokens, world, chunk)[rank]


def gather_rows(local_rows, shard: Shard, total_tokens: int, group=None):
    """Validation only: all-gathers each rank's output rows ([tokens, width] tensor) into the full
    [total_tokens, width] tensor on every rank (NCCL over NVLink on GPUs, gloo on CPU).  Never on
    the timed path.  Ranks may own different row counts; rows are padded to the largest shard."""
    import torch
    import torch.distributed as dist

    world = shard.world
    if world == 1:
        return local_rows
    parts = partition(total_tokens, world)
    longest = max(p.tokens for p in parts)
    width = local_rows.shape[1]
    padded = torch.zeros((longest, width), dtype=local_rows.dtype, device=local_rows.device)
    padded[:shard.tokens] = local_rows
    out = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(out, padded, group=group)
    return torch.cat([o[:p.tokens] for o, p in zip(out, parts)], dim=0)


def validate_sharded_chain(rank: int, world: int, tokens_per_rank: int = 1024, layers: int = 8, group=None) -> dict:
    """Validation only (never timed): every rank runs the operator chain on its token shard of one
    shared synthetic prompt, the shards' outputs are all-gathered over NCCL / NVLink, and each rank
    compares them bit for bit with its own unsharded run of the whole prompt.  Checks the two
    cross-row dependencies of the path: the conv halo (three raw rows before the shard) and the
    NVFP4 scale groups (chunk-aligned shards never split one).  Returns a small report."""
    import importlib

    import torch

    chain = importlib.import_module(__package__ + ".chain")
    total = tokens_per_rank * world
    me = shard_for(total, rank, world)
    lo, hi = me.first_token, me.end_token
    rows = 4096  # a small embedding table is enough here
    whole = chain.LayerStack(total, first_position=0, seed=99, layers=layers, table_rows=rows)
    local = chain.LayerStack(me.tokens, first_position=lo, seed=7, layers=layers, table_rows=rows)
    # same prompt, same weights: the shard's inputs are row slices of the whole prompt's
    for name in whole.inputs:
        local.inputs[name].copy_(whole.inputs[name][lo:hi])
    local.token_ids.copy_(whole.token_ids[lo:hi])
    for name in ("table", "norm_w", "q_norm_w", "k_norm_w", "gdn_norm_w", "conv_w"):
        setattr(local, name, getattr(whole, name))
    if me.halo_first < lo:  # raw rows just before the shard become its conv history (oldest first)
        halo = whole.inputs["conv_raw"][me.halo_first:lo].t().contiguous()
        local.conv_hist[:, :, CONV_HALO - halo.shape[1]:] = halo[None]
    stream = torch.cuda.current_stream().cuda_stream
    final_whole = whole.residual[whole.enqueue_step(stream)]
    final_local = local.residual[local.enqueue_step(stream)]
    torch.cuda.synchronize()
    whole.check_error("unsharded validation run")
    local.check_error("sharded validation run")

    def same(a, b):
        return bool(torch.equal(a.contiguous().view(torch.uint8), b.contiguous().view(torch.uint8)))

    first_group = lo // CHUNK
    report = {
        "tokens": total, "layers": layers, "rank_rows": [lo, hi],
        "local_equals_unsharded": all([
            same(final_local, final_whole[lo:hi]), same(local.normalized, whole.normalized[lo:hi]),
            same(local.codes, whole.codes[lo:hi]), same(local.scales, whole.scales[lo:hi]),
            same(local.conv_out, whole.conv_out[lo:hi]), same(local.gdn_out, whole.gdn_out[lo:hi]),
            same(local.gdn_codes, whole.gdn_codes[lo:hi]), same(local.q_out, whole.q_out[lo:hi]),
            same(local.attn_out, whole.attn_out[lo:hi]), same(local.mlp_out, whole.mlp_out[lo:hi]),
            same(local.global_scales, whole.global_scales[first_group:first_group + local.groups]),
        ]),
    }
    gathered_bytes = 0
    ok = True
    for mine, full in ((final_local, final_whole), (local.codes, whole.codes), (local.scales, whole.scales)):
        gathered = gather_rows(mine, me, total, group)
        gathered_bytes += gathered.numel() * gathered.element_size()
        ok = ok and same(gathered, full)
    report["gathered_bytes"] = gathered_bytes
    report["gathered_equals_unsharded"] = ok
    return report
