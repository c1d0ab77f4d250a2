"""Token -> rank layouts for causal masks.

The masks of this engine (like the reference's, ring_attention/ring.py:394-397) are driven by
per-token `positions`, not by block indices, so any assignment of tokens to ranks is legal as
long as the positions travel with the tokens.  With contiguous shards a causal mask gives
rank r work in r+1 of the N ring steps and the slowest rank sets the pace.  The zig-zag
layout cuts the sequence into 2N chunks and gives rank r chunks r and 2N-1-r: every rank
then sees exactly half of every block pair, at every step.
"""
from __future__ import annotations

import torch


def zigzag_indices(total_len: int, rank: int, nranks: int, device=None) -> torch.Tensor:
    """Global token indices held by `rank`: chunk `rank` followed by chunk `2*nranks-1-rank`."""
    if total_len % (2 * nranks):
        raise ValueError(f"sequence length {total_len} is not a multiple of 2*nranks = {2 * nranks}")
    c = total_len // (2 * nranks)
    a = torch.arange(rank * c, (rank + 1) * c, device=device)
    b = torch.arange((2 * nranks - 1 - rank) * c, (2 * nranks - rank) * c, device=device)
    return torch.cat([a, b])


def zigzag_shard(x: torch.Tensor, rank: int, nranks: int, dim: int = 1) -> torch.Tensor:
    """This rank's shard of a global array under the zig-zag layout."""
    idx = zigzag_indices(x.shape[dim], rank, nranks, device=x.device)
    return x.index_select(dim, idx).contiguous()


def zigzag_unshard(shards, dim: int = 1) -> torch.Tensor:
    """Inverse of zigzag_shard over the list of all ranks' shards (rank order)."""
    n = len(shards)
    total = sum(s.shape[dim] for s in shards)
    out_shape = list(shards[0].shape)
    out_shape[dim] = total
    out = shards[0].new_empty(out_shape)
    for r, s in enumerate(shards):
        out.index_copy_(dim, zigzag_indices(total, r, n, device=s.device), s)
    return out
