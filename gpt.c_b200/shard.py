"""Host-side sharding of the attention workload over the GPUs of one box.

Every (batch, head) pair is independent in forward and backward, so the batch axis is cut into
contiguous slices, one per rank, and no collective is needed on the data path: a rank's slice of
qkv / dout / out / dqkv is one contiguous block of the full tensors (the reference stores them
row-major with batch outermost, src/attention.c:95-115 of gpt.c).
"""
from __future__ import annotations


def batch_slices(batch: int, world: int) -> list[tuple[int, int]]:
    """(start, stop) of each rank's batch slice; the first `batch % world` ranks get one more."""
    if batch < 0 or world <= 0:
        raise ValueError("batch must be >= 0 and world > 0")
    base, extra = divmod(batch, world)
    out, start = [], 0
    for r in range(world):
        n = base + (1 if r < extra else 0)
        out.append((start, start + n))
        start += n
    return out


def shard(array, rank: int, world: int):
    """The contiguous batch slice of `array` (anything sliceable on axis 0) that `rank` owns."""
    a, b = batch_slices(array.shape[0], world)[rank]
    return array[a:b]


def flops(batch: int, seq: int, heads: int, head_dim: int, backward: bool = True) -> float:
    """Algorithmic FLOPs of causal attention (T^2/2 convention, recomputation not counted)."""
    f = 2.0 * batch * heads * seq * seq * head_dim
    return f * 3.0 if backward else f
