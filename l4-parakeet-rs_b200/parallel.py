"""Utterance-level data parallelism over the GPUs of one node.

Utterances are independent end to end (no cross-utterance state, eval-mode BatchNorm,
per-row LayerNorm), so they are dealt to ranks round-robin; there is no collective on the
compute path.  The only exchange is a host-side gather of token ids."""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist


def shard_utterances(total: int, world_size: int, rank: int) -> list[int]:
    """Utterance u goes to rank u mod world_size."""
    return [u for u in range(total) if u % world_size == rank]


def gather_token_lists(local: dict[int, np.ndarray], total: int, group=None, dst: int = 0):
    """Host gather: every rank contributes {utterance id: token ids}; rank `dst` returns the
    list for all `total` utterances (others return None).  Works on any backend that
    supports CPU tensors (gloo); payload is a few KB per utterance."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return [local[u] for u in range(total)]
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    ids = sorted(local)
    lengths = torch.tensor([len(ids)] + [len(local[u]) for u in ids], dtype=torch.int64)
    payload = torch.from_numpy(np.concatenate([np.asarray(ids, dtype=np.int64)] +
                                              [np.asarray(local[u], dtype=np.int64) for u in ids])
                               if ids else np.zeros(0, np.int64))
    sizes = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(sizes, torch.tensor([lengths.numel() + payload.numel()], dtype=torch.int64), group=group)
    cap = int(max(int(s.item()) for s in sizes))
    buf = torch.zeros(cap + 1, dtype=torch.int64)
    buf[0] = lengths.numel()
    packed = torch.cat([lengths, payload])
    buf[1:1 + packed.numel()] = packed
    gathered = [torch.zeros(cap + 1, dtype=torch.int64) for _ in range(world)] if rank == dst else None
    dist.gather(buf, gathered, dst=dst, group=group)
    if rank != dst:
        return None
    out: list = [None] * total
    for b in gathered:
        nlen = int(b[0].item())
        lens = b[1:1 + nlen].tolist()
        n_ids = lens[0]
        body = b[1 + nlen:]
        uids = body[:n_ids].tolist()
        pos = n_ids
        for u, ln in zip(uids, lens[1:]):
            out[u] = body[pos:pos + ln].numpy().astype(np.int32)
            pos += ln
    return out
