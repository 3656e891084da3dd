"""Oracle (test infrastructure): the reference's tensor-parallel plumbing in NumPy —
sharding (src/parallel/shard.rs), the host all_reduce / all_gather
(src/parallel/comm.rs:47-62,178-193) and TpWorld's size rules
(src/parallel/world.rs:95-133)."""
from __future__ import annotations

import numpy as np

from .kernels_ref import rnd


def column_shard(weight: np.ndarray, rank: int, world_size: int) -> np.ndarray:
    """narrow(0, rank*chunk, chunk) with chunk = rows/world_size (shard.rs:46-54)."""
    rows = weight.shape[0]
    if rows % world_size != 0:
        raise ValueError(f"column_shard: out_features ({rows}) is not divisible by world_size ({world_size})")
    chunk = rows // world_size
    return weight[rank * chunk:(rank + 1) * chunk]


def row_shard(weight: np.ndarray, rank: int, world_size: int) -> np.ndarray:
    """narrow(1, rank*chunk, chunk) with chunk = cols/world_size (shard.rs:66-74)."""
    cols = weight.shape[1]
    if cols % world_size != 0:
        raise ValueError(f"row_shard: in_features ({cols}) is not divisible by world_size ({world_size})")
    chunk = cols // world_size
    return weight[:, rank * chunk:(rank + 1) * chunk]


def bias_shard(bias: np.ndarray, rank: int, world_size: int) -> np.ndarray:
    """shard.rs:85-94."""
    n = bias.shape[0]
    if n % world_size != 0:
        raise ValueError(f"bias_shard: out_features ({n}) is not divisible by world_size ({world_size})")
    chunk = n // world_size
    return bias[rank * chunk:(rank + 1) * chunk]


def column_chunk_size(out_features: int, world_size: int) -> int:
    return out_features // world_size


def row_chunk_size(in_features: int, world_size: int) -> int:
    return in_features // world_size


def all_reduce(shards, dtype: str = "f32") -> np.ndarray:
    """acc = shards[0]; acc = acc + s for the rest, in rank order, each sum materialised
    in the tensor dtype (comm.rs:47-62)."""
    if len(shards) == 0:
        raise ValueError("all_reduce: shard list is empty")
    acc = np.asarray(shards[0], dtype=np.float32)
    for s in shards[1:]:
        acc = rnd(acc + np.asarray(s, dtype=np.float32), dtype)
    return acc


def all_reduce_f32(shards, dtype: str = "f32") -> np.ndarray:
    """The CUDA library's order of operations: fp32 accumulation in rank order, one
    rounding at the end."""
    if len(shards) == 0:
        raise ValueError("all_reduce: shard list is empty")
    acc = np.zeros_like(np.asarray(shards[0], dtype=np.float32))
    for s in shards:
        acc = acc + np.asarray(s, dtype=np.float32)
    return rnd(acc, dtype)


def all_gather(shards, dim: int) -> np.ndarray:
    """comm.rs:178-193."""
    if len(shards) == 0:
        raise ValueError("all_gather: shard list is empty")
    if len(shards) == 1:
        return np.asarray(shards[0])
    return np.concatenate([np.asarray(s) for s in shards], axis=dim)


def world_size_check(world_size: int, available: int) -> None:
    """TpWorld::new (world.rs:95-115)."""
    assert world_size >= 1, "world_size must be >= 1"
    if world_size > 1 and available < world_size:
        raise ValueError(
            f"tensor_parallel_size={world_size} requested but only {available} CUDA device(s) detected. "
            "Use --tensor-parallel-size 1 for single-GPU.")
