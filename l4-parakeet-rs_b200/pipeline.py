"""Host-side mirror of the reference's pipeline engine
(src/cuda/pipeline.rs: PipelineEngine::load :121-395, transcribe :397-417,
run_prepared :437-608) for a batch of utterances on one GPU, starting from log-mel
frames (`transcribe_batch`) or from PCM through the log-mel frontend (`transcribe_pcm`).

    mel [U, frames, 128] fp32 (host) --H2D--> subsampling -> 24 encoder blocks
        -> encoder projection -> TDT greedy decode --D2H--> token ids

Everything between the two copies is stream-ordered launches of libpk100 kernels
without host synchronisation.

Decode is a latency-bound chain on 16 SMs (one thread-block cluster) whose length is the
longest utterance's rounds and whose cost per round grows with the utterances that step in
it; the encoder is throughput-bound and most efficient on the whole batch.  So the batch is
cut twice: into `encode_groups` groups that go through subsampling and the encoder blocks
one after the other on the caller's stream (default 1: the whole batch in one pass), and
into `decode_groups` groups (default: as many 16-CTA clusters as the device holds at once,
7 on a B200) that are decoded side by side, each on its own high-priority stream with its
own workspace, as soon as the encode group they belong to is done.  With more than one encode
group the decoders of the earlier groups run under the encoder of the next, whose persistent
GEMMs are capped at the SMs those decoders leave free.  Results are identical whatever the
grouping (every kernel is batch-invariant); only the schedule changes."""
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


class _Slot:
    """Per-request device and host buffers of one batch in flight (the engine itself is slot 0;
    `transcribe_stream` adds a second one so that a batch can be encoded while the one before
    it is still being decoded)."""

    def __init__(self, eng):
        dev, n = eng.device, eng.max_utterances
        self.mel_dev = torch.zeros_like(eng.mel_dev)
        self.mel_frames_dev = torch.full((n,), eng.mel_frames, dtype=torch.int32, device=dev)
        self.out_frames_dev = torch.full((n,), eng.frames_out, dtype=torch.int32, device=dev)
        self.out_frames_host = torch.full((n,), eng.frames_out, dtype=torch.int32)
        self.longest_out_frames = eng.frames_out
        self._lengths = tuple([eng.mel_frames] * n)
        self.enc_proj = torch.zeros_like(eng.enc_proj)
        self.tokens, self.durations, self.counts = (torch.zeros_like(t) for t in (eng.tokens, eng.durations, eng.counts))
        self.tokens_host = torch.zeros_like(eng.tokens_host).pin_memory()
        self.counts_host = torch.zeros_like(eng.counts_host).pin_memory()
        self.dec_streams = [torch.cuda.Stream(device=dev, priority=-1) for _ in range(eng.decode_groups)]
        self.dec_scratch = [eng.dec.make_scratch() for _ in range(eng.decode_groups)]


class PipelineEngine:
    def __init__(self, device, layers=24, decoder_layers=2, seed=4, max_utterances=8, mel_frames=6000,
                 randomize_norms=False, decode_groups=None, out_proj_resident="f16", encode_groups=1,
                 subsampling_precision="fp16"):
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.max_utterances = max_utterances
        self.encode_groups = max(1, min(int(encode_groups), max_utterances))
        if decode_groups is None:
            decode_groups = max(1, int(L.lib.pk100_tdt_cluster_capacity(decoder_layers)))
        self.decode_groups = max(self.encode_groups, min(int(decode_groups), max_utterances))
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.mel_frames = mel_frames
        self.frames_out = sub_mod.output_frames(mel_frames)
        self.seg_stride = seg_stride_for(self.frames_out)
        self.rows = max_utterances * self.seg_stride
        self.sub = sub_mod.Subsampling(synth.subsampling_weights(seed), self.device, precision=subsampling_precision)
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
        """CUDA events around every FF-expand GEMM (two per block), one set per encode group."""
        n = 2 * 2 * len(self.enc.layers)
        self._events, self._event_arrays = [], []
        for _ in range(self.encode_groups):
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
        for e, (u0, u1) in enumerate(self.last_encode_groups):
            ev = self._events[e]
            out += [(ev[2 * i].elapsed_time(ev[2 * i + 1]), (u1 - u0) * self.seg_stride) for i in range(len(ev) // 2)]
        return out

    # ---- stages
    def enable_stage_timing(self):
        """CUDA events around the encode and the decode of every group (recording does not synchronise)."""
        mk = lambda: torch.cuda.Event(enable_timing=True)
        self._stage_events = dict(enc=[(mk(), mk()) for _ in range(self.encode_groups)],
                                  dec=[(mk(), mk()) for _ in range(self.decode_groups)])

    def stage_times(self):
        """After a synchronise: per decode group of the last request, its utterance range, encode
        and decode milliseconds, the decode's lockstep rounds, and when the decode started and
        ended relative to the start of the request."""
        out = []
        first = self._stage_events["enc"][0][0]
        for g, (u0, u1) in enumerate(self.last_groups):
            enc0, enc1 = self._stage_events["enc"][self.last_encode_of[g]]
            dec0, dec1 = self._stage_events["dec"][g]
            out.append(dict(utterances=[u0, u1], encode_group=self.last_encode_of[g],
                            encode_ms=enc0.elapsed_time(enc1), encode_end_ms=first.elapsed_time(enc1),
                            decode_ms=dec0.elapsed_time(dec1),
                            decode_start_ms=first.elapsed_time(dec0), decode_end_ms=first.elapsed_time(dec1),
                            rounds=self.dec.last_rounds(u1 - u0, self.dec_scratch[g])))
        return out

    def set_lengths(self, mel_frames_per_utt, slot=None):
        b = self if slot is None else slot
        b._lengths = tuple(int(f) for f in mel_frames_per_utt) + b._lengths[len(mel_frames_per_utt):]
        mf = torch.tensor(mel_frames_per_utt, dtype=torch.int32)
        of = torch.tensor([sub_mod.output_frames(int(f)) for f in mel_frames_per_utt], dtype=torch.int32)
        b.mel_frames_dev[:len(mf)].copy_(mf)
        b.out_frames_dev[:len(of)].copy_(of)
        b.out_frames_host[:len(of)].copy_(of)
        b.longest_out_frames = int(b.out_frames_host.max())

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

    @staticmethod
    def _split(first, last, parts):
        """[first, last) cut into `parts` contiguous ranges whose sizes differ by at most one."""
        base, extra = divmod(last - first, parts)
        bounds, u = [], first
        for g in range(parts):
            n = base + (1 if g < extra else 0)
            bounds.append((u, u + n))
            u += n
        return bounds

    def _plan(self, utterances, decode_groups=None):
        """[((first, last) of an encode group, [(first, last) of each of its decode groups])]:
        the utterances cut into decode groups, consecutive decode groups joined into encode groups."""
        dg = min(self.decode_groups if decode_groups is None else max(1, min(decode_groups, self.decode_groups)),
                 utterances)
        eg = min(self.encode_groups, dg)
        decs = self._split(0, utterances, dg)
        plan = []
        for (g0, g1) in self._split(0, dg, eg):
            plan.append(((decs[g0][0], decs[g1 - 1][1]), decs[g0:g1]))
        return plan

    def run_resident(self, utterances, slot=None, join=True, clusters_in_flight=0, decode_groups=None):
        """Hot path with the inputs already in HBM: subsampling -> encoder -> projection -> decode,
        group by group (see the module text); returns with everything queued on the caller's
        stream, which waits for the side streams (join=False: it does not, and the decode groups'
        streams are returned).  slot: the buffers of the batch (default: the engine's own);
        clusters_in_flight: decoder clusters of an earlier batch still running beside this one."""
        b = self if slot is None else slot
        # the reference switches decoder kernels (and numerics) at 1024 frames per request
        # (src/cuda/decoder.rs:88); a batch of short utterances needs one launch only
        cache = "auto" if b.longest_out_frames >= dec_mod.LONG_REQUEST_FRAMES else "fp16"
        main = torch.cuda.current_stream()
        plan = self._plan(utterances, decode_groups)
        self.last_encode_groups = [enc for enc, _ in plan]
        self.last_groups = [d for _, decs in plan for d in decs]
        self.last_encode_of = [e for e, (_, decs) in enumerate(plan) for _ in decs]
        single = len(self.last_groups) == 1 and join
        seg = self.seg_stride
        g = 0
        for e, ((a0, a1), decs) in enumerate(plan):
            ev = self._stage_events if slot is None else None
            r0, r1 = a0 * seg, a1 * seg
            if g + clusters_in_flight > 0:
                # decoders already running hold 16 SMs each while this group is encoded
                L.lib.pk100_set_gemm_cta_cap(max(self.sm_count - 16 * (g + clusters_in_flight), 16))
            if ev:
                ev["enc"][e][0].record(main)
            if self._events is not None and slot is None:
                self.ws.profile_events = C.cast(self._event_arrays[e], C.POINTER(C.c_void_p))
            self.sub.run(b.mel_dev[a0:a1], seg, mel_frames=b.mel_frames_dev[a0:a1], out=self.state_a[r0:r1])
            encoded = self.enc.run(self.state_a[r0:r1], self.state_b[r0:r1], self.ws, a1 - a0, seg,
                                   self.frames_out, seg_valid=b.out_frames_dev[a0:a1])
            self.dec.project(encoded, out=b.enc_proj[r0:r1])
            if ev:
                ev["enc"][e][1].record(main)
            for (u0, u1) in decs:
                side = main if single else b.dec_streams[g]
                if side is not main:
                    side.wait_stream(main)
                with torch.cuda.stream(side):
                    if ev:
                        ev["dec"][g][0].record(side)
                    self.dec.decode(b.enc_proj[u0 * seg:u1 * seg], u1 - u0, seg, b.out_frames_dev[u0:u1],
                                    self.max_tokens, b.tokens[u0:u1], b.durations[u0:u1], b.counts[u0:u1],
                                    lstm_cache=cache, scratch=b.dec_scratch[g])
                    if ev:
                        ev["dec"][g][1].record(side)
                g += 1
        L.lib.pk100_set_gemm_cta_cap(0)
        if single:
            return []
        if join:
            for k in range(g):
                main.wait_stream(b.dec_streams[k])
        return b.dec_streams[:g]

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
        self._queue_status()
        torch.cuda.current_stream().synchronize()
        status = self._queued_status()
        if status != 0:
            raise RuntimeError(f"libpk100 reported an expired bounded wait (status {status})")
        counts = self.counts_host.numpy()
        return [self.tokens_host[u, :int(counts[u])].numpy().copy() for u in range(utterances)]

    def transcribe_stream(self, batches, decode_groups=1, depth=4):
        """Throughput mode: a generator over `batches` (each a pinned fp32 CPU tensor [U, frames, 128]
        or a pair (tensor, true frame counts)) that yields, in order, what `transcribe_batch` returns
        for each.  `depth` sets of request buffers rotate: a batch is copied in and encoded while the
        decoder clusters of up to depth - 1 earlier batches are still running, the encoder's persistent
        GEMMs capped at the SMs those clusters leave free (`decode_groups` clusters per batch: fewer
        than in `transcribe_batch`, where nothing runs beside them), and the host waits for a batch's
        tokens only when its buffers are needed again or the newest batch has been queued.  Steady
        state per batch: the larger of the (slowed) encode and the decoder-cluster time of a batch
        divided by the clusters in flight, instead of encode + longest chain.  Measured for batches of
        8 x 60 s: one lockstep cluster per batch and four batches in flight (the defaults) give 11.5 ms
        per batch; four clusters per batch and two batches in flight 19.9 ms; a batch on its own 34.4 ms."""
        depth = max(2, int(depth))
        if not hasattr(self, "_extra_slots"):
            self._extra_slots, self._collect_streams, self._slot_status = [], [], []
        while len(self._extra_slots) < depth - 1:
            self._extra_slots.append(_Slot(self))
        while len(self._collect_streams) < depth:
            self._collect_streams.append(torch.cuda.Stream(device=self.device))
        slots = [self] + self._extra_slots[:depth - 1]
        words = self._status_words()
        while len(self._slot_status) < depth or any(t.numel() != len(words) for t in self._slot_status):
            self._slot_status = [torch.zeros(len(words), dtype=torch.int32).pin_memory() for _ in range(depth)]
        main = torch.cuda.current_stream()

        def finish(entry):
            k, utterances, done, _ = entry
            b = slots[k]
            done.synchronize()
            status = self._combine_status(self._slot_status[k].tolist())
            if status != 0:
                raise RuntimeError(f"libpk100 reported an expired bounded wait (status {status})")
            counts = b.counts_host.numpy()
            return [b.tokens_host[u, :int(counts[u])].numpy().copy() for u in range(utterances)]

        pending = []                              # oldest first: (slot index, utterances, event, clusters)
        for i, item in enumerate(batches):
            mel_host, lengths = item if isinstance(item, (tuple, list)) else (item, None)
            k = i % depth
            if len(pending) == depth:             # the slot's previous batch has to be out first
                yield finish(pending.pop(0))
            b = slots[k]
            utterances = mel_host.shape[0]
            lengths = tuple([int(mel_host.shape[1])] * utterances if lengths is None else [int(f) for f in lengths])
            if max(lengths) > mel_host.shape[1] or mel_host.shape[1] > self.mel_frames or utterances > self.max_utterances:
                raise ValueError("batch larger than the engine was sized for")
            if lengths != b._lengths[:utterances]:
                self.set_lengths(lengths, slot=b)
            b.mel_dev[:utterances, :mel_host.shape[1]].copy_(mel_host, non_blocking=True)
            streams = self.run_resident(utterances, slot=b, join=False,
                                        clusters_in_flight=sum(e[3] for e in pending), decode_groups=decode_groups)
            collect = self._collect_streams[k]
            for st in streams:
                collect.wait_stream(st)
            with torch.cuda.stream(collect):
                b.counts_host.copy_(b.counts, non_blocking=True)
                b.tokens_host.copy_(b.tokens, non_blocking=True)
                for n, w in enumerate(words):
                    self._slot_status[k][n:n + 1].copy_(w, non_blocking=True)
                done = torch.cuda.Event()
                done.record(collect)
            pending.append((k, utterances, done, len(streams)))
            if len(pending) == depth:
                yield finish(pending.pop(0))
        while pending:
            yield finish(pending.pop(0))
        main.synchronize()

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
        self._queue_status()
        torch.cuda.current_stream().synchronize()
        status = self._queued_status()
        if status != 0:
            raise RuntimeError(f"libpk100 reported an expired bounded wait (status {status})")
        counts = self.counts_host.numpy()
        return [self.tokens_host[u, :int(counts[u])].numpy().copy() for u in range(utterances)]

    HIDDEN_SATURATED = 8      # status bit of the encoder: an FF hidden activation was clamped at INT8 +127

    def hidden_saturated(self):
        """True when an FF hidden activation exceeded the INT8 range (x 1/32) since the engine was
        built: harmless for N(0, 0.02) weights, a sign of a wrong hidden scale on a real checkpoint."""
        return bool(self.enc.status(self.arena, self.ws) & self.HIDDEN_SATURATED)

    def _status_words(self):
        """Device int32 views of every status word: encoder, subsampling, then the decoders'."""
        off = self.ws.status - self.arena.data_ptr()
        extra = list(self.dec_scratch[1:])
        for slot in getattr(self, "_extra_slots", []):
            extra += slot.dec_scratch
        return [self.arena[off:off + 4].view(torch.int32), self.sub.status, self.dec.status] + [s[1] for s in extra]

    def _queue_status(self):
        """Copies the status words to pinned host memory on the current stream, behind the request
        (one synchronise then serves the tokens and the status: no further device round trips)."""
        words = self._status_words()
        if getattr(self, "_status_host", None) is None or self._status_host.numel() != len(words):
            self._status_host = torch.zeros(len(words), dtype=torch.int32).pin_memory()
        for i, w in enumerate(words):
            self._status_host[i:i + 1].copy_(w, non_blocking=True)

    def _queued_status(self):
        """After a synchronise: what `status()` would return, from the words `_queue_status` copied."""
        return self._combine_status(self._status_host.tolist())

    def _combine_status(self, h):
        dec = 0
        for v in h[2:]:
            dec |= v & ~4                               # bit 4: a decode round had only NaN scores
        return (h[0] & ~self.HIDDEN_SATURATED) | h[1] | dec

    def status(self):
        """Non-zero when a bounded wait expired inside a kernel (saturation is reported separately)."""
        return self._combine_status([int(w.item()) for w in self._status_words()])


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
