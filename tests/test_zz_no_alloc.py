"""The allocation-free decoder entry point (`pk100_tdt_decode_static`).

Written for hosts that hand a plug-in no way to allocate device memory: the scratch the
decoder needs sits in a fixed array inside libpk100.so.  The test drives the entry point
through the C ABI exactly as such a host would -- it passes inputs and outputs only -- and
requires the same tokens, durations and counts as the regular entry point (integer outputs:
bit-exact), on two consecutive calls so that leftovers of the first call in the shared
array cannot leak into the second.  Collected last on purpose (file name)."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import codec, decoder as D

pytestmark = pytest.mark.gpu


def _decode_static(pk, dec, enc, utterances, seg_stride, frames, max_tokens):
    fn = pk.lib.lib.pk100_tdt_decode_static
    vp = C.c_void_p
    fn.argtypes = [vp, C.POINTER(type(dec.c)), vp, C.c_int, C.c_int, vp, vp, vp, vp, C.c_int, vp]
    fn.restype = C.c_int
    dev = enc.device
    tokens = torch.full((utterances, max_tokens), -1, dtype=torch.int32, device=dev)
    durations = torch.full((utterances, max_tokens), -1, dtype=torch.int32, device=dev)
    counts = torch.full((utterances,), -1, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    rc = fn(torch.cuda.current_stream().cuda_stream, C.byref(dec.c), enc.data_ptr(), utterances, seg_stride,
            frames.data_ptr(), tokens.data_ptr(), durations.data_ptr(), counts.data_ptr(), max_tokens,
            status.data_ptr())
    return rc, tokens, durations, counts, status


def test_static_scratch_decoder_matches_regular_entry_point(pk, cuda):
    w = D.make_decoder_weights(41, layers=2)
    dec = pk.decoder.TdtDecoder(w, cuda)
    seg_stride, max_tokens = 64, 640
    rng = np.random.default_rng(12)
    cases = [([64, 40, 17], rng.standard_normal((3 * seg_stride, 640))),
             ([64, 64, 64, 9, 30, 1, 64, 50], rng.standard_normal((8 * seg_stride, 640)))]
    for frames, enc in cases:          # two calls in a row, different batch widths
        utterances = len(frames)
        enc_d = torch.from_numpy(codec.f16_round(enc * 0.5)).half().to(cuda)
        fr = torch.tensor(frames, dtype=torch.int32, device=cuda)
        # the workspace-taking entry point of the same kernel
        want_t, want_d, want_c = dec.decode(enc_d, utterances, seg_stride, fr, max_tokens, kernel="exchange")
        torch.cuda.synchronize()
        want_t, want_d, want_c = want_t.cpu().numpy().copy(), want_d.cpu().numpy().copy(), want_c.cpu().numpy().copy()
        rc, tokens, durations, counts, status = _decode_static(pk, dec, enc_d, utterances, seg_stride, fr, max_tokens)
        torch.cuda.synchronize()
        assert rc == 0 and int(status.item()) == 0
        # the property the entry point exists for: with every buffer already in the caller's hands
        # (here: reused), a further call leaves the device's free memory untouched
        free_before, _ = torch.cuda.mem_get_info()
        fn = pk.lib.lib.pk100_tdt_decode_static
        rc2 = fn(torch.cuda.current_stream().cuda_stream, C.byref(dec.c), enc_d.data_ptr(), utterances, seg_stride,
                 fr.data_ptr(), tokens.data_ptr(), durations.data_ptr(), counts.data_ptr(), max_tokens,
                 status.data_ptr())
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert rc2 == 0 and free_after == free_before
        counts = counts.cpu().numpy()
        assert np.array_equal(counts, want_c) and counts.max() > 10
        for u in range(utterances):
            n = int(counts[u])
            assert np.array_equal(tokens[u, :n].cpu().numpy(), want_t[u, :n])
            assert np.array_equal(durations[u, :n].cpu().numpy(), want_d[u, :n])


def test_static_scratch_decoder_rejects_oversized_batches(pk, cuda):
    w = D.make_decoder_weights(42, layers=1)
    dec = pk.decoder.TdtDecoder(w, cuda)
    enc = torch.zeros((9 * 8, 640), dtype=torch.float16, device=cuda)
    fr = torch.ones(9, dtype=torch.int32, device=cuda)
    rc, *_ = _decode_static(pk, dec, enc, 9, 8, fr, 16)
    assert rc == pk.lib.ERR_LIMIT
