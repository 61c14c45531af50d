"""One long utterance cut into overlapping chunks (one per GPU): with the exact halo the chunk
interiors reproduce the unsplit encoder rows BIT FOR BIT; a reduced halo is an approximation
whose error is measured here.  The ranks are played one after the other on one GPU (they share
nothing on the device, so this is the same computation)."""
import numpy as np
import pytest
import torch

from tests.util import dev16, host, nrmse

pytestmark = pytest.mark.gpu

LAYERS = 2


@pytest.fixture(scope="module")
def stack(pk, cuda):
    """Two blocks with calibrated tile thresholds and a 2000-row input (one utterance)."""
    rows_valid, rows = 2000, 2048
    g = torch.Generator().manual_seed(5)
    x = torch.randn((rows, 1024), generator=g).half()
    x[rows_valid:] = 0
    enc = pk.encoder.EncoderLayers(cuda)
    for l in range(LAYERS):
        enc.add_layer(pk.synth.layer_weights(8, l, randomize_norms=True))
    arena, ws = enc.make_workspace(rows)
    pk.encoder.calibrate_tile_thresholds(enc, x.to(cuda), ws, 1, rows, rows_valid)
    assert all(l.ff1.tau > 0 and l.ff2.tau > 0 for l in enc.layers)
    a, b = x.to(cuda), torch.zeros((rows, 1024), dtype=torch.float16, device=cuda)
    whole = host(enc.run(a, b, ws, 1, rows, rows_valid)).copy()
    assert enc.status(arena, ws) & 1 == 0
    return enc, arena, ws, x, whole, rows_valid, rows


def _run_chunk(pk, cuda, enc, ws, x, chunk, rows):
    x0, x1 = chunk.extended
    n = x1 - x0
    a = torch.zeros((rows, 1024), dtype=torch.float16, device=cuda)
    a[:n] = x[x0:x1].to(cuda)
    b = torch.zeros_like(a)
    return host(enc.run(a, b, ws, 1, rows, n))[:n]


def test_exact_halo_reproduces_the_unsplit_rows_bit_for_bit(pk, cuda, stack):
    enc, arena, ws, x, whole, valid, rows = stack
    halo = pk.parallel.exact_halo_rows(LAYERS)
    assert halo == 512
    plan = pk.parallel.chunk_plan(valid, 2, halo)
    assert [c.core for c in plan] == [(0, 1024), (1024, 2000)] and plan[1].extended[0] % 128 == 0
    parts = []
    for chunk in plan:
        got = _run_chunk(pk, cuda, enc, ws, x, chunk, rows)
        parts.append(got[chunk.interior])
    assert enc.status(arena, ws) & 1 == 0
    stitched = pk.parallel.stitch_rows(parts)
    assert stitched.shape == (valid, 1024)
    assert np.array_equal(stitched, whole[:valid])
    # three ranks, one of them with a short last chunk
    parts = [_run_chunk(pk, cuda, enc, ws, x, c, rows)[c.interior] for c in pk.parallel.chunk_plan(valid, 3, halo)]
    assert np.array_equal(pk.parallel.stitch_rows(parts), whole[:valid])


def test_reduced_halo_is_an_approximation_with_a_measured_error(pk, cuda, stack):
    enc, arena, ws, x, whole, valid, rows = stack
    errors = {}
    for halo in (0, 128, 256):
        parts = [_run_chunk(pk, cuda, enc, ws, x, c, rows)[c.interior] for c in pk.parallel.chunk_plan(valid, 2, halo)]
        stitched = pk.parallel.stitch_rows(parts)
        errors[halo] = nrmse(stitched, whole[:valid])
        differing = np.flatnonzero(np.any(stitched != whole[:valid], axis=1))
        # only rows near the cut can differ: within the exact halo of it
        assert differing.size == 0 or (differing.min() >= 1024 - 512 and differing.max() < 1024 + 512)
    print("reduced-halo nRMSE over the whole utterance:", {k: f"{v:.2e}" for k, v in errors.items()})
    assert errors[0] > 0 and errors[256] <= errors[0] and errors[256] < 3e-2


def test_long_utterance_from_mel_in_two_chunks(pk, cuda):
    """Through the pipeline: each rank subsamples only the mel frames of its extended rows (one row
    more on the left, dropped), encodes, projects; the stitched interiors equal the unsplit
    projection bit for bit and decode to the same tokens."""
    frames = 8 * 1500
    mel = torch.from_numpy(pk.synth.mel_input(77, frames))
    one = pk.pipeline.PipelineEngine(cuda, layers=LAYERS, decoder_layers=2, seed=6, max_utterances=1,
                                     mel_frames=frames, decode_groups=1)
    one.mel_dev[0].copy_(mel)
    one.calibrate(1)
    whole_tokens = pk.pipeline.transcribe_long(one, mel)          # world of one: the unsplit run
    whole_proj = host(one.enc_proj[:1500]).copy()
    halo = pk.parallel.exact_halo_rows(LAYERS)
    plan = pk.parallel.chunk_plan(1500, 2, halo)
    longest = max(pk.parallel.mel_range(c, frames)[1] - pk.parallel.mel_range(c, frames)[0] for c in plan)
    eng = pk.pipeline.PipelineEngine(cuda, layers=LAYERS, decoder_layers=2, seed=6, max_utterances=1,
                                     mel_frames=longest, decode_groups=1)
    for l, lw in enumerate(one.enc.layers):
        eng.enc.set_tau(l, lw.ff1.tau, lw.ff2.tau)
    parts = []
    for chunk in plan:
        first, last, lead = pk.parallel.mel_range(chunk, frames)
        proj = eng.encode_chunk(mel[first:last], lead, chunk.extended[1] - chunk.extended[0])
        parts.append(host(proj[chunk.interior]).copy())
    assert eng.status() == 0
    stitched = pk.parallel.stitch_rows(parts)
    assert np.array_equal(stitched, whole_proj)
    # the same rows decode to the same tokens (1500 frames: the long-request numerics)
    rows_dev = torch.zeros((1536, 640), dtype=torch.float16, device=cuda)
    rows_dev[:1500] = dev16(stitched)
    fr = torch.tensor([1500], dtype=torch.int32, device=cuda)
    tokens, _, counts = eng.dec.decode(rows_dev, 1, 1536, fr, 15000, lstm_cache="int8")
    torch.cuda.synchronize()
    assert np.array_equal(host(tokens)[0][:int(host(counts)[0])], whole_tokens) and len(whole_tokens) > 100
