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
    parts = partition(total_tokens, world)
    longest = max(p.tokens for p in parts)
    width = local_rows.shape[1]
    padded = torch.zeros((longest, width), dtype=local_rows.dtype, device=local_rows.device)
    padded[:shard.tokens] = local_rows
    out = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(out, padded, group=group)
    return torch.cat([o[:p.tokens] for o, p in zip(out, parts)], dim=0)
