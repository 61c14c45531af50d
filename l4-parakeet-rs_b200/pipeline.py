"""Host-side mirror of the reference's pipeline engine
(src/cuda/pipeline.rs: PipelineEngine::load :121-395, transcribe :397-417,
run_prepared :437-608) for a batch of utterances on one GPU, starting from log-mel
frames (`transcribe_batch`) or from PCM through the log-mel frontend (`transcribe_pcm`).

    mel [U, frames, 128] fp32 (host) --H2D--> subsampling -> 24 encoder blocks
        -> encoder projection -> TDT greedy decode --D2H--> token ids

Everything between the two copies is stream-ordered launches of libpk100 kernels
without host synchronisation.

Decode is a latency-bound chain on 16 SMs (one thread-block cluster); the encoder wants the
other 132.  With `decode_groups` > 1 the batch is cut into that many groups of utterances:
group g is encoded on the caller's stream, then decoded on a high-priority side stream
while group g + 1 is being encoded, the encoder's persistent GEMMs capped at the SMs the
decoders in flight leave free.  Results are identical to the ungrouped run (every kernel
is batch-invariant); only the schedule changes."""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import decoder as dec_mod
from . import lib as L
from . import encoder as enc_mod
from . import subsampling as sub_mod
from . import synth

MAX_SYMBOLS_PER_FRAME = 10


def seg_stride_for(frames_out: int) -> int:
    """Rows reserved per utterance: output frames rounded up to the 128-row tile so that the
    tile-sparsity bitmap and the GEMM tiles never straddle two utterances."""
    return (frames_out + 127) // 128 * 128


class PipelineEngine:
    def __init__(self, device, layers=24, decoder_layers=2, seed=4, max_utterances=8, mel_frames=6000,
                 randomize_norms=False, decode_groups=2, out_proj_resident="f16"):
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.max_utterances = max_utterances
        self.decode_groups = max(1, min(int(decode_groups), max_utterances))
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.mel_frames = mel_frames
        self.frames_out = sub_mod.output_frames(mel_frames)
        self.seg_stride = seg_stride_for(self.frames_out)
        self.rows = max_utterances * self.seg_stride
        self.sub = sub_mod.Subsampling(synth.subsampling_weights(seed), self.device)
        self.enc = enc_mod.EncoderLayers(self.device, out_proj_resident=out_proj_resident)
        for l in range(layers):
            self.enc.add_layer(synth.layer_weights(seed, l, randomize_norms=randomize_norms))
        self.dec = dec_mod.TdtDecoder(synth.decoder_weights(seed, decoder_layers), self.device)
        self.arena, self.ws = self.enc.make_workspace(self.rows)
        dev = self.device
        self.state_a = torch.zeros((self.rows, 1024), dtype=torch.float16, device=dev)
        self.state_b = torch.zeros((self.rows, 1024), dtype=torch.float16, device=dev)
        self.enc_proj = torch.zeros((self.rows, 640), dtype=torch.float16, device=dev)
        self.max_tokens = self.frames_out * MAX_SYMBOLS_PER_FRAME
        self.tokens = torch.zeros((max_utterances, self.max_tokens), dtype=torch.int32, device=dev)
        self.durations = torch.zeros((max_utterances, self.max_tokens), dtype=torch.int32, device=dev)
        self.counts = torch.zeros(max_utterances, dtype=torch.int32, device=dev)
        self.mel_dev = torch.zeros((max_utterances, mel_frames, 128), dtype=torch.float32, device=dev)
        self.mel_frames_dev = torch.full((max_utterances,), mel_frames, dtype=torch.int32, device=dev)
        self.out_frames_dev = torch.full((max_utterances,), self.frames_out, dtype=torch.int32, device=dev)
        self.out_frames_host = torch.full((max_utterances,), self.frames_out, dtype=torch.int32)
        self.longest_out_frames = self.frames_out      # max(out_frames_host)
        # pinned host staging for the two copies of a request
        self.tokens_host = torch.zeros((max_utterances, self.max_tokens), dtype=torch.int32).pin_memory()
        self.counts_host = torch.zeros(max_utterances, dtype=torch.int32).pin_memory()
        self.calibrated = False
        self._events = None
        self._lengths = tuple([mel_frames] * max_utterances)
        # one side stream, scratch and event set per decode group
        self.dec_streams = [torch.cuda.Stream(device=self.device, priority=-1) for _ in range(self.decode_groups)]
        self.dec_scratch = [None] + [self.dec.make_scratch() for _ in range(self.decode_groups - 1)]
        self._stage_events = None
        self.last_groups = []

    # ---- profiling hook: CUDA events around the FF-expand GEMMs
    def enable_gemm_timing(self):
        """CUDA events around every FF-expand GEMM (two per block), one set per decode group."""
        n = 2 * 2 * len(self.enc.layers)
        self._events, self._event_arrays = [], []
        for _ in range(self.decode_groups):
            events = [torch.cuda.Event(enable_timing=True) for _ in range(n)]
            for e in events:
                e.record()                   # creates the underlying cudaEvent_t
            self._events.append(events)
            self._event_arrays.append((C.c_void_p * n)(*[e.cuda_event for e in events]))
        torch.cuda.synchronize()
        self.ws.profile_events_len = n

    def gemm_times_ms(self):
        """[(milliseconds, rows of that launch)] for every FF-expand launch of the last request."""
        out = []
        for g, (u0, u1) in enumerate(self.last_groups):
            ev = self._events[g]
            out += [(ev[2 * i].elapsed_time(ev[2 * i + 1]), (u1 - u0) * self.seg_stride) for i in range(len(ev) // 2)]
        return out

    # ---- stages
    def enable_stage_timing(self):
        """CUDA events around the encode and the decode of every group (recording does not synchronise)."""
        mk = lambda: torch.cuda.Event(enable_timing=True)
        self._stage_events = [dict(enc0=mk(), enc1=mk(), dec0=mk(), dec1=mk()) for _ in range(self.decode_groups)]

    def stage_times(self):
        """After a synchronise: per decode group of the last request, its utterance range, encode
        and decode milliseconds, the decode's lockstep rounds, and when the decode started and
        ended relative to the start of the request."""
        out = []
        first = self._stage_events[0]["enc0"]
        for g, (u0, u1) in enumerate(self.last_groups):
            ev = self._stage_events[g]
            out.append(dict(utterances=[u0, u1], encode_ms=ev["enc0"].elapsed_time(ev["enc1"]),
                            decode_ms=ev["dec0"].elapsed_time(ev["dec1"]),
                            decode_start_ms=first.elapsed_time(ev["dec0"]), decode_end_ms=first.elapsed_time(ev["dec1"]),
                            rounds=self.dec.last_rounds(u1 - u0, self.dec_scratch[g])))
        return out

    def set_lengths(self, mel_frames_per_utt):
        self._lengths = tuple(int(f) for f in mel_frames_per_utt) + self._lengths[len(mel_frames_per_utt):]
        mf = torch.tensor(mel_frames_per_utt, dtype=torch.int32)
        of = torch.tensor([sub_mod.output_frames(int(f)) for f in mel_frames_per_utt], dtype=torch.int32)
        self.mel_frames_dev[:len(mf)].copy_(mf)
        self.out_frames_dev[:len(of)].copy_(of)
        self.out_frames_host[:len(of)].copy_(of)
        self.longest_out_frames = int(self.out_frames_host.max())

    def encode(self, utterances):
        self.sub.run(self.mel_dev[:utterances], self.seg_stride, mel_frames=self.mel_frames_dev,
                     out=self.state_a)
        return self.enc.run(self.state_a, self.state_b, self.ws, utterances, self.seg_stride,
                            self.frames_out, seg_valid=self.out_frames_dev)

    def calibrate(self, utterances):
        """One-time: choose every FF module's tile threshold (70 % zero tiles) on the batch
        currently in `mel_dev`."""
        self.sub.run(self.mel_dev[:utterances], self.seg_stride, mel_frames=self.mel_frames_dev,
                     out=self.state_a)
        enc_mod.calibrate_tile_thresholds(self.enc, self.state_a[:utterances * self.seg_stride], self.ws,
                                          utterances, self.seg_stride, self.frames_out,
                                          seg_valid=self.out_frames_dev)
        self.calibrated = True

    def _group_bounds(self, utterances):
        groups = min(self.decode_groups, utterances)
        base, extra = divmod(utterances, groups)
        bounds, u = [], 0
        for g in range(groups):
            n = base + (1 if g < extra else 0)
            bounds.append((u, u + n))
            u += n
        return bounds

    def run_resident(self, utterances):
        """Hot path with the inputs already in HBM: subsampling -> encoder -> projection -> decode,
        group by group (see the module text); returns with everything queued on the caller's
        stream, which waits for the side streams."""
        # the reference switches decoder kernels (and numerics) at 1024 frames per request
        # (src/cuda/decoder.rs:88); a batch of short utterances needs one launch only
        cache = "auto" if self.longest_out_frames >= dec_mod.LONG_REQUEST_FRAMES else "fp16"
        main = torch.cuda.current_stream()
        bounds = self._group_bounds(utterances)
        self.last_groups = bounds
        seg = self.seg_stride
        for g, (u0, u1) in enumerate(bounds):
            ev = self._stage_events[g] if self._stage_events is not None else None
            r0, r1 = u0 * seg, u1 * seg
            if g > 0:
                # decoders of the earlier groups hold 16 SMs each while this group is encoded
                L.lib.pk100_set_gemm_cta_cap(max(self.sm_count - 16 * g, 16))
            if ev:
                ev["enc0"].record(main)
            if self._events is not None:
                self.ws.profile_events = C.cast(self._event_arrays[g], C.POINTER(C.c_void_p))
            self.sub.run(self.mel_dev[u0:u1], seg, mel_frames=self.mel_frames_dev[u0:u1], out=self.state_a[r0:r1])
            encoded = self.enc.run(self.state_a[r0:r1], self.state_b[r0:r1], self.ws, u1 - u0, seg,
                                   self.frames_out, seg_valid=self.out_frames_dev[u0:u1])
            self.dec.project(encoded, out=self.enc_proj[r0:r1])
            if ev:
                ev["enc1"].record(main)
            side = self.dec_streams[g] if len(bounds) > 1 else main
            if side is not main:
                side.wait_stream(main)
            with torch.cuda.stream(side):
                if ev:
                    ev["dec0"].record(side)
                self.dec.decode(self.enc_proj[r0:r1], u1 - u0, seg, self.out_frames_dev[u0:u1], self.max_tokens,
                                self.tokens[u0:u1], self.durations[u0:u1], self.counts[u0:u1], lstm_cache=cache,
                                scratch=self.dec_scratch[g])
                if ev:
                    ev["dec1"].record(side)
        if len(bounds) > 1:
            L.lib.pk100_set_gemm_cta_cap(0)
            for g in range(len(bounds)):
                main.wait_stream(self.dec_streams[g])

    def transcribe_batch(self, mel_host, mel_frames_per_utt=None):
        """mel_host: pinned fp32 CPU tensor [U, frames, 128]; mel_frames_per_utt: true frame
        count of every utterance (default: all of mel_host's frames).  Returns a list of int32
        numpy token arrays (one per utterance).  Includes the H2D copy of the inputs and the
        D2H read of the result (pipeline.rs:398, :409)."""
        utterances = mel_host.shape[0]
        lengths = tuple([int(mel_host.shape[1])] * utterances if mel_frames_per_utt is None
                        else [int(f) for f in mel_frames_per_utt])
        if max(lengths) > mel_host.shape[1] or mel_host.shape[1] > self.mel_frames:
            raise ValueError("utterance longer than the engine was sized for")
        if lengths != self._lengths[:utterances]:
            self.set_lengths(lengths)          # never reuse the lengths an earlier request left behind
        self.mel_dev[:utterances, :mel_host.shape[1]].copy_(mel_host, non_blocking=True)
        self.run_resident(utterances)
        self.counts_host.copy_(self.counts, non_blocking=True)
        self.tokens_host.copy_(self.tokens, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        status = self.status()
        if status != 0:
            raise RuntimeError(f"libpk100 reported an expired bounded wait (status {status})")
        counts = self.counts_host.numpy()
        return [self.tokens_host[u, :int(counts[u])].numpy().copy() for u in range(utterances)]

    # ---- one long utterance cut into chunks over several GPUs (see parallel.py)
    def encode_chunk(self, mel_chunk_host, lead_rows, rows):
        """Encodes `rows` encoder rows of a long utterance from the mel frames that cover them
        (`parallel.mel_range`): subsampling, the `lead_rows` rows in front dropped, the blocks
        on the rest as ONE sequence of `rows` rows, the encoder projection.  Needs an engine
        built for one utterance of at least mel_chunk_host.shape[0] frames.  Returns the
        projected rows [rows, 640] (fp16, device)."""
        frames = int(mel_chunk_host.shape[0])
        if frames > self.mel_frames or self.max_utterances < 1:
            raise ValueError("chunk longer than the engine was sized for")
        if lead_rows + rows > self.seg_stride or rows > sub_mod.output_frames(frames) - lead_rows:
            raise ValueError("the mel frames do not cover the requested rows")
        self.mel_dev[0, :frames].copy_(mel_chunk_host, non_blocking=True)
        self.set_lengths([frames])
        if not hasattr(self, "_chunk_rows"):
            # subsampling output with room for the dropped rows in front of a 128-aligned block
            self._chunk_rows = torch.zeros((self.seg_stride + 128, 1024), dtype=torch.float16, device=self.device)
            self._chunk_valid = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.sub.run(self.mel_dev[:1], self.seg_stride + 128, mel_frames=self.mel_frames_dev[:1], out=self._chunk_rows)
        x = self._chunk_rows[lead_rows:lead_rows + self.seg_stride]
        self._chunk_valid.fill_(rows)
        encoded = self.enc.run(x, self.state_b[:self.seg_stride], self.ws, 1, self.seg_stride, rows,
                               seg_valid=self._chunk_valid)
        self.dec.project(encoded, out=self.enc_proj[:self.seg_stride])
        return self.enc_proj[:rows]

    # ---- optional stage in front: PCM -> log-mel (src/cuda/pipeline.rs:437-470 runs it first)
    def attach_frontend(self, window, mel_filters):
        """window [400] and mel_filters [128, 257]: the artifact's frontend.* tensors."""
        from . import frontend as fe_mod
        self.frontend = fe_mod.MelFrontend(window, mel_filters, self.device)
        self.pcm_capacity = (self.mel_frames - 1) * fe_mod.HOP          # mel_frames rows hold that many samples
        self.pcm_dev = torch.zeros((self.max_utterances, self.pcm_capacity), dtype=torch.float32, device=self.device)
        self.pcm_counts_dev = torch.zeros(self.max_utterances, dtype=torch.int32, device=self.device)

    def transcribe_pcm(self, pcm_host, sample_counts):
        """pcm_host: fp32 CPU tensor [U, samples] (zero padded), sample_counts: list of ints.
        Frontend -> subsampling -> encoder -> decode; returns token arrays like transcribe_batch."""
        from . import frontend as fe_mod
        utterances, samples = pcm_host.shape
        if samples > self.pcm_capacity or max(sample_counts) > samples:
            raise ValueError("utterance longer than the engine was sized for")
        self.pcm_dev[:utterances, :samples].copy_(pcm_host, non_blocking=True)
        if samples < self.pcm_capacity:
            self.pcm_dev[:utterances, samples:].zero_()
        self.pcm_counts_dev[:utterances].copy_(torch.tensor(sample_counts, dtype=torch.int32), non_blocking=True)
        self.frontend.compute(self.pcm_dev[:utterances], self.pcm_counts_dev[:utterances], frame_cap=self.mel_frames,
                              out=self.mel_dev[:utterances])
        self.set_lengths([n // fe_mod.HOP for n in sample_counts])       # valid frames are known on the host
        self.run_resident(utterances)
        self.counts_host.copy_(self.counts, non_blocking=True)
        self.tokens_host.copy_(self.tokens, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        status = self.status()
        if status != 0:
            raise RuntimeError(f"libpk100 reported an expired bounded wait (status {status})")
        counts = self.counts_host.numpy()
        return [self.tokens_host[u, :int(counts[u])].numpy().copy() for u in range(utterances)]

    HIDDEN_SATURATED = 8      # status bit of the encoder: an FF hidden activation was clamped at INT8 +127

    def hidden_saturated(self):
        """True when an FF hidden activation exceeded the INT8 range (x 1/32) since the engine was
        built: harmless for N(0, 0.02) weights, a sign of a wrong hidden scale on a real checkpoint."""
        return bool(self.enc.status(self.arena, self.ws) & self.HIDDEN_SATURATED)

    def status(self):
        """Non-zero when a bounded wait expired inside a kernel (saturation is reported separately)."""
        dec = int(self.dec.status.item()) & ~4          # bit 4: a decode round had only NaN scores
        for scratch in self.dec_scratch[1:]:
            dec |= int(scratch[1].item())
        return (self.enc.status(self.arena, self.ws) & ~self.HIDDEN_SATURATED) | dec | int(self.sub.status.item())


def transcribe_long(eng, mel_host, rank=0, world_size=1, group=None, halo=None, decoder=None):
    """One long utterance over `world_size` GPUs, no collective on the compute path: every rank
    encodes its chunk of encoder rows with a halo (`parallel.chunk_plan`), the projected rows
    of the chunk interiors are gathered on the host, rank 0 decodes them as one sequence and
    returns the token ids (the other ranks return None).
    eng: this rank's PipelineEngine for ONE utterance, sized for the longest extended chunk;
    mel_host: fp32 CPU tensor [frames, 128], the same on every rank; halo: rows beside a chunk
    (default: the exact halo of the engine's depth); decoder: (TdtDecoder, its device) on rank 0
    when the decode should not use eng.dec."""
    from . import parallel
    frames = int(mel_host.shape[0])
    total_rows = sub_mod.output_frames(frames)
    if halo is None:
        halo = parallel.exact_halo_rows(len(eng.enc.layers), tile_sparse=any(l.ff1.tau > 0 or l.ff2.tau > 0
                                                                              for l in eng.enc.layers))
    chunk = parallel.chunk_plan(total_rows, world_size, halo)[rank]
    rows = chunk.extended[1] - chunk.extended[0]
    if rows > 0:
        first, last, lead = parallel.mel_range(chunk, frames)
        proj = eng.encode_chunk(mel_host[first:last], lead, rows)
        mine = proj[chunk.interior].float().cpu().numpy()
    else:
        mine = np.zeros((0, dec_mod.HIDDEN), np.float32)
    if eng.status() != 0:
        raise RuntimeError("libpk100 reported an expired bounded wait")
    parts = parallel.gather_rows(mine, group=group)
    if parts is None:
        return None
    whole = parallel.stitch_rows(parts)
    dec = eng.dec if decoder is None else decoder
    stride = seg_stride_for(total_rows)
    rows_dev = torch.zeros((stride, dec_mod.HIDDEN), dtype=torch.float16, device=eng.device)
    rows_dev[:total_rows].copy_(torch.from_numpy(whole).to(torch.float16))
    fr = torch.tensor([total_rows], dtype=torch.int32, device=eng.device)
    cache = "int8" if total_rows >= dec_mod.LONG_REQUEST_FRAMES else "fp16"
    tokens, _, counts = dec.decode(rows_dev, 1, stride, fr, total_rows * MAX_SYMBOLS_PER_FRAME, lstm_cache=cache)
    torch.cuda.synchronize()
    return tokens[0, :int(counts[0].item())].cpu().numpy()
