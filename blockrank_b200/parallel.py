"""Data parallelism by ranking prompt: static partition, one replica per GPU, one gather of scores.

The reference shards its eval DataLoader with Accelerate and gathers top-k
indices every step (scripts/eval_attn.py:98, :154).  Here prompts are assigned
up front, every rank scores its share with no data-path communication, and the
fp32 score rows are gathered once at the end.  Works with any
torch.distributed backend (NCCL on GPUs, Gloo for CPU tests).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


def partition_prompts(num_prompts: int, world_size: int, rank: int, costs: Optional[Sequence[float]] = None) -> List[int]:
    """Prompt indices owned by ``rank``.

    Without costs: contiguous chunks whose sizes differ by at most one.  With
    per-prompt costs (e.g. token counts of ragged prompts): longest-processing-
    time greedy assignment, deterministic on every rank.
    """
    if not 0 <= rank < world_size:
        raise ValueError("rank out of range")
    if costs is None:
        base, extra = divmod(num_prompts, world_size)
        lo = rank * base + min(rank, extra)
        return list(range(lo, lo + base + (1 if rank < extra else 0)))
    if len(costs) != num_prompts:
        raise ValueError("one cost per prompt expected")
    load = [0.0] * world_size
    owner = [0] * num_prompts
    for p in sorted(range(num_prompts), key=lambda i: (-float(costs[i]), i)):
        r = min(range(world_size), key=lambda j: (load[j], j))
        owner[p] = r
        load[r] += float(costs[p])
    return [p for p in range(num_prompts) if owner[p] == rank]


def gather_scores(local_scores: torch.Tensor, local_ids: Sequence[int], num_prompts: int,
                  group: Optional[dist.ProcessGroup] = None, max_share: Optional[int] = None) -> torch.Tensor:
    """All-gather fp32 score rows and put them back in prompt order.

    local_scores (n_local, num_docs) for prompts ``local_ids``.  Every rank
    receives the full (num_prompts, num_docs) tensor.  One
    ``all_gather_into_tensor`` and no host synchronisation on the regular path:
    rows are padded to ``max_share``, the largest number of prompts any rank
    owns, which every rank must compute the same way -- by default
    ceil(num_prompts / world), the bound of :func:`partition_prompts` without
    costs; pass it for a cost-balanced partition.  A prompt that no rank
    delivered raises RuntimeError on every rank.
    """
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        out = local_scores.new_zeros(num_prompts, local_scores.shape[1])
        out[torch.as_tensor(list(local_ids), dtype=torch.long, device=local_scores.device)] = local_scores
        return out
    world = dist.get_world_size(group)
    nd = local_scores.shape[1]
    cap = int(max_share) if max_share is not None else -(-num_prompts // world)
    n = len(local_ids)
    if n > cap:
        raise ValueError(f"this rank owns {n} prompts but max_share is {cap}: pass the largest share of the partition")
    send = local_scores.new_full((cap, nd + 1), -1.0)
    if n:
        send[:n, :nd] = local_scores
        send[:n, nd] = torch.as_tensor(list(local_ids), dtype=local_scores.dtype, device=local_scores.device)
    recv = local_scores.new_empty(world * cap, nd + 1)
    dist.all_gather_into_tensor(recv, send.contiguous(), group=group)
    ids = recv[:, nd].round().long()
    keep = ids >= 0
    out = local_scores.new_zeros(num_prompts, nd)
    seen = torch.zeros(num_prompts, dtype=torch.bool, device=recv.device)
    out[ids[keep]] = recv[keep][:, :nd]
    seen[ids[keep]] = True
    if not bool(seen.all()):
        missing = (~seen).nonzero().flatten().tolist()
        raise RuntimeError(f"no rank delivered scores for prompts {missing}")
    return out
