"""Host-side multi-rank logic on CPU: utterance sharding and the gloo token gather
(world_size 2, spawned processes, rendezvous on 127.0.0.1)."""
import importlib
import os
import sys
from pathlib import Path

import numpy as np
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def test_shard_is_a_partition(pk):
    for world in (1, 2, 4, 8):
        seen = sorted(u for r in range(world) for u in pk.parallel.shard_utterances(64, world, r))
        assert seen == list(range(64))
        assert all(len(pk.parallel.shard_utterances(64, world, r)) == 64 // world for r in range(world))


def _tokens_for(u):
    rng = np.random.default_rng(u)
    return rng.integers(0, 1024, size=int(rng.integers(0, 40)), dtype=np.int32)


def _worker(rank, world, port, total, q):
    sys.path.insert(0, str(ROOT))
    pk = importlib.import_module("l4-parakeet-rs_b200")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    mine = {u: _tokens_for(u) for u in pk.parallel.shard_utterances(total, world, rank)}
    out = pk.parallel.gather_token_lists(mine, total)
    if rank == 0:
        q.put([o.tolist() for o in out])
    else:
        assert out is None
    dist.barrier()
    dist.destroy_process_group()


def test_gloo_gather_world_size_2():
    total, world = 10, 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, total, q)) for r in range(world)]
    for p in procs:
        p.start()
    result = q.get(timeout=120)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert result == [_tokens_for(u).tolist() for u in range(total)]
