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


def test_chunk_plan_covers_the_utterance_with_aligned_overlapping_chunks(pk):
    P = pk.parallel
    assert P.exact_halo_rows(24, tile_sparse=False) == 24 * 132 == 3168
    assert P.exact_halo_rows(24) == 6144 and P.exact_halo_rows(0) == 0
    for total, world, halo in ((45000, 8, 6144), (45000, 8, 3168), (750, 8, 512), (2000, 3, 0), (1, 2, 128), (0, 4, 128)):
        plan = P.chunk_plan(total, world, halo)
        assert len(plan) == world and [c.rank for c in plan] == list(range(world))
        cores = [c.core for c in plan if c.core[1] > c.core[0]]
        assert (cores[0][0] == 0 and cores[-1][1] == total) if total else not cores
        assert all(a[1] == b[0] for a, b in zip(cores, cores[1:]))
        for c in plan:
            if c.core[1] == c.core[0]:
                continue
            x0, x1 = c.extended
            assert x0 % 128 == 0 and c.core[0] % 128 == 0
            assert x0 <= max(0, c.core[0] - halo) and x1 >= min(total, c.core[1] + halo) and x1 <= total
            assert c.interior == slice(c.core[0] - x0, c.core[1] - x0)
            first, last, lead = P.mel_range(c, 8 * total)
            assert first == 8 * (x0 - lead) and lead == (1 if x0 > 0 else 0) and last <= 8 * total


def _rows_worker(rank, world, port, total, q):
    sys.path.insert(0, str(ROOT))
    pk = importlib.import_module("l4-parakeet-rs_b200")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    full = np.random.default_rng(3).standard_normal((total, 640)).astype(np.float16).astype(np.float32)
    chunk = pk.parallel.chunk_plan(total, world, 256)[rank]
    # stand-in for the encoder: this rank "computes" its extended rows and keeps the interior
    extended = full[chunk.extended[0]:chunk.extended[1]]
    parts = pk.parallel.gather_rows(extended[chunk.interior])
    if rank == 0:
        q.put(bool(np.array_equal(pk.parallel.stitch_rows(parts), full)))
        # the token gather that follows the decode on rank 0 uses the same group
    else:
        assert parts is None
    tokens = pk.parallel.gather_token_lists({0: np.arange(5, dtype=np.int32)} if rank == 0 else {}, 1)
    assert (tokens is None) == (rank != 0)
    dist.barrier()
    dist.destroy_process_group()


def test_gloo_row_gather_and_stitch_world_size_2():
    total, world = 1500, 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + os.getpid() % 2000
    procs = [ctx.Process(target=_rows_worker, args=(r, world, port, total, q)) for r in range(world)]
    for p in procs:
        p.start()
    assert q.get(timeout=120) is True
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0


def test_pipeline_plan_of_encode_and_decode_groups(pk):
    """PipelineEngine._plan: the utterances cut into decode groups, consecutive decode groups joined
    into encode groups; every utterance exactly once, group sizes differ by at most one."""
    from types import SimpleNamespace
    plan_of = pk.pipeline.PipelineEngine._plan
    split = pk.pipeline.PipelineEngine._split
    for utterances in range(1, 9):
        for enc_groups in (1, 2, 3):
            for dec_groups in (1, 2, 4, 7, 8):
                eng = SimpleNamespace(encode_groups=enc_groups, decode_groups=max(enc_groups, dec_groups), _split=split)
                plan = plan_of(eng, utterances)
                decs = [d for _, ds in plan for d in ds]
                assert decs[0][0] == 0 and decs[-1][1] == utterances
                assert all(a[1] == b[0] for a, b in zip(decs, decs[1:]))
                assert len(decs) == min(eng.decode_groups, utterances) and len(plan) == min(enc_groups, len(decs))
                sizes = [b - a for a, b in decs]
                assert max(sizes) - min(sizes) <= 1 and min(sizes) >= 1
                for (e0, e1), ds in plan:
                    assert ds[0][0] == e0 and ds[-1][1] == e1
    eng = SimpleNamespace(encode_groups=1, decode_groups=7, _split=split)
    assert plan_of(eng, 8) == [((0, 8), [(0, 2), (2, 3), (3, 4), (4, 5), (5, 6), (6, 7), (7, 8)])]
    assert plan_of(eng, 8, 4)[0][1] == [(0, 2), (2, 4), (4, 6), (6, 8)]
