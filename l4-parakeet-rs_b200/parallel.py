"""Data parallelism over the GPUs of one node, without a collective on the compute path.

Many utterances: they are independent end to end (no cross-utterance state, eval-mode BatchNorm,
per-row LayerNorm), so they are dealt to ranks round-robin and only token ids are gathered, on
the host.

One long utterance: the encoder rows are cut into one chunk per rank.  A block of the encoder
couples rows over +-132 positions (attention +-128, depthwise convolution +-4) and, through the
128-row tile threshold of the FF hidden activations, over the 128-row tile a row lies in.  A rank
therefore encodes its chunk plus a halo on each side and keeps the interior; with the halo of
`exact_halo_rows` the interior equals the unsplit result bit for bit (chunk starts are multiples
of 128 rows, so every tile is the same tile in both runs), a smaller halo is an approximation
whose error is measured, not assumed.  The projected encoder rows of the interiors are gathered on
the host and decoded by one rank: the decoder is one sequential chain over the utterance.  The
reference handles length by tiling inside one GPU instead (src/cuda/subsampling.rs:528-536, the
row-count thresholds of src/cuda/encoder.rs:24-26)."""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch
import torch.distributed as dist

ATTENTION_REACH = 128        # rows on each side a query attends to
DEPTHWISE_REACH = 4          # (9 - 1) / 2 taps of the depthwise convolution
TILE_ROWS = 128              # rows of one tile of the FF hidden-activation threshold


def _up(value: int, multiple: int) -> int:
    return (value + multiple - 1) // multiple * multiple


def exact_halo_rows(layers: int, tile_sparse: bool = True) -> int:
    """Rows beside a chunk that have to be encoded with it so that the chunk's own rows come out
    exactly as in the unsplit run.  `front` = how far from a cut a row can differ: each block moves
    it by 132 rows, and with the tile threshold on every FF module widens it to whole tiles (a
    tile's keep / drop decision reads all of its 128 rows).  24 blocks: 3168 rows dense, 6144 with
    tile sparsity."""
    front = 0
    for _ in range(layers):
        if tile_sparse:
            front = _up(front, TILE_ROWS)                       # first FF module
        front += ATTENTION_REACH + DEPTHWISE_REACH
        if tile_sparse:
            front = _up(front, TILE_ROWS)                       # second FF module
    return front


@dataclass(frozen=True)
class Chunk:
    rank: int
    core: tuple[int, int]        # rows this rank contributes, [begin, end)
    extended: tuple[int, int]    # rows it encodes, [begin, end); begin is a multiple of 128

    @property
    def interior(self) -> slice:
        """The core inside the extended range."""
        return slice(self.core[0] - self.extended[0], self.core[1] - self.extended[0])


def chunk_plan(total_rows: int, world_size: int, halo: int) -> list[Chunk]:
    """One chunk per rank over encoder rows [0, total_rows).  Core and extended ranges start on
    multiples of 128 rows (the tile grid of the unsplit run); a rank whose core would start beyond
    the utterance gets an empty chunk."""
    if total_rows < 0 or world_size <= 0 or halo < 0:
        raise ValueError("chunk_plan: negative size")
    per = _up(-(-total_rows // world_size), TILE_ROWS) if total_rows else 0
    chunks = []
    for r in range(world_size):
        c0, c1 = min(r * per, total_rows), min((r + 1) * per, total_rows)
        if c0 == c1:
            chunks.append(Chunk(r, (c0, c0), (c0, c0)))
            continue
        x0 = max(0, (c0 - halo) // TILE_ROWS * TILE_ROWS)
        x1 = min(total_rows, _up(c1 + halo, TILE_ROWS))     # whole tiles, or the utterance's true end
        chunks.append(Chunk(r, (c0, c1), (x0, x1)))
    return chunks


def mel_range(chunk: Chunk, mel_frames: int) -> tuple[int, int, int]:
    """Mel frames a rank needs for its extended rows and how many leading output rows to drop:
    8x subsampling (three stride-2 convolutions of kernel 3) makes row r depend on frames
    8r - 7 .. 8r + 7, so a chunk that starts inside the utterance takes one row more on the left
    (frames from 8 (begin - 1)) and drops it: that row saw zero padding instead of its left
    context, every row after it is exact.  Returns (first_frame, last_frame_exclusive, lead_rows)."""
    x0, x1 = chunk.extended
    lead = 1 if x0 > 0 else 0
    first = 8 * (x0 - lead)
    last = min(mel_frames, 8 * x1 + 8)
    return first, last, lead


def stitch_rows(parts: list[np.ndarray]) -> np.ndarray:
    """Interiors in rank order -> the rows of the whole utterance."""
    parts = [p for p in parts if p is not None and len(p)]
    return np.concatenate(parts, axis=0) if parts else np.zeros((0, 0), np.float32)


def gather_rows(local: np.ndarray, group=None, dst: int = 0):
    """Host gather of one 2-D array per rank (its interior rows; row counts may differ), returned
    on rank `dst` as the list in rank order.  gloo, CPU tensors; 1280 bytes per projected row."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return [local]
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    local = np.ascontiguousarray(local)
    shape = torch.tensor(local.shape if local.ndim == 2 else (0, 0), dtype=torch.int64)
    shapes = [torch.zeros(2, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(shapes, shape, group=group)
    cap = max(int(s[0] * s[1]) for s in shapes)
    buf = torch.zeros(cap, dtype=torch.float32)
    buf[:local.size] = torch.from_numpy(local.astype(np.float32).ravel())
    gathered = [torch.zeros(cap, dtype=torch.float32) for _ in range(world)] if rank == dst else None
    dist.gather(buf, gathered, dst=dst, group=group)
    if rank != dst:
        return None
    return [g[:int(s[0] * s[1])].numpy().reshape(int(s[0]), int(s[1])) for g, s in zip(gathered, shapes)]


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
