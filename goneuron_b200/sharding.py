"""Batch sharding over ranks: contiguous equal shards, rank r owns samples [r*B/R, (r+1)*B/R) -- the chunking
rule of the reference's worker pool (internal/net/net.go:621-633) applied to GPUs."""


def shard_bounds(global_batch, rank, world_size):
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} / world {world_size}")
    if global_batch % world_size:
        raise ValueError(f"global batch {global_batch} is not divisible by {world_size} ranks")
    per = global_batch // world_size
    return rank * per, (rank + 1) * per
