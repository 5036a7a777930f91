"""Data-parallel sharding of independent sequences (one process per GPU).

The Heron forward has no cross-sequence dependency: suffix-automaton state is
per (sequence, channel) and a CE row only reads labels[row+1] of its own
sequence (reference src/model.rs:27-39).  Ranks therefore take contiguous
blocks of sequences, run the whole forward locally, and exchange only
{loss_sum, n_valid}; the global mean is sum(loss_sum) / sum(n_valid), which is
the reference's single-process mean over all valid positions
(src/model.rs:3253-3257) - not a mean of per-rank means.
"""
from __future__ import annotations

import numpy as np


def shard_range(n_sequences: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous block [lo, hi) of sequences owned by `rank`; blocks differ in
    size by at most one and cover 0..n_sequences exactly once."""
    if world < 1 or not (0 <= rank < world) or n_sequences < 0:
        raise ValueError("bad rank / world / sequence count")
    base, extra = divmod(n_sequences, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_tokens(tokens: np.ndarray, labels: np.ndarray, time: int, rank: int, world: int):
    """Rows of this rank from [B*T] token / label arrays."""
    tokens = np.asarray(tokens).reshape(-1, time)
    labels = np.asarray(labels).reshape(-1, time)
    lo, hi = shard_range(tokens.shape[0], rank, world)
    return tokens[lo:hi].reshape(-1), labels[lo:hi].reshape(-1), hi - lo


def reduce_loss_torch(loss_sum: float, n_valid: int, group=None, device=None):
    """All-reduce (sum) of {loss_sum, n_valid} through torch.distributed (gloo on
    CPU ranks, NCCL on GPU ranks). Returns (loss_sum, n_valid, mean)."""
    import torch
    import torch.distributed as dist

    t = torch.tensor([float(loss_sum), float(n_valid)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    total, n = float(t[0].item()), int(round(float(t[1].item())))
    return total, n, (total / n if n else 0.0)


def global_mean(parts) -> float:
    """Mean over all valid positions from per-rank (loss_sum, n_valid) pairs."""
    total = sum(p[0] for p in parts)
    n = sum(p[1] for p in parts)
    return total / n if n else 0.0
