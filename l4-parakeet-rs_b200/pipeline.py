"""Host-side mirror of the reference's pipeline engine
(src/cuda/pipeline.rs: PipelineEngine::load :121-395, transcribe :397-417,
run_prepared :437-608) for a batch of utterances on one GPU, starting from log-mel
frames (the audio frontend is outside this build's scope).

    mel [U, frames, 128] fp32 (host) --H2D--> subsampling -> 24 encoder blocks
        -> encoder projection -> TDT greedy decode --D2H--> token ids

Everything between the two copies is stream-ordered launches of libpk100 kernels
without host synchronisation."""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import decoder as dec_mod
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
                 randomize_norms=False):
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.max_utterances = max_utterances
        self.mel_frames = mel_frames
        self.frames_out = sub_mod.output_frames(mel_frames)
        self.seg_stride = seg_stride_for(self.frames_out)
        self.rows = max_utterances * self.seg_stride
        self.sub = sub_mod.Subsampling(synth.subsampling_weights(seed), self.device)
        self.enc = enc_mod.EncoderLayers(self.device)
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

    # ---- profiling hook: CUDA events around the FF-expand GEMMs
    def enable_gemm_timing(self):
        n = 2 * 2 * len(self.enc.layers)
        self._events = [torch.cuda.Event(enable_timing=True) for _ in range(n)]
        for e in self._events:
            e.record()                       # creates the underlying cudaEvent_t
        torch.cuda.synchronize()
        arr = (C.c_void_p * n)(*[e.cuda_event for e in self._events])
        self._event_array = arr
        self.ws.profile_events = C.cast(arr, C.POINTER(C.c_void_p))
        self.ws.profile_events_len = n

    def gemm_times_ms(self):
        return [self._events[2 * i].elapsed_time(self._events[2 * i + 1]) for i in range(len(self._events) // 2)]

    # ---- stages
    def set_lengths(self, mel_frames_per_utt):
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

    def run_resident(self, utterances):
        """Hot path with the inputs already in HBM: subsampling -> encoder -> decode."""
        encoded = self.encode(utterances)
        self.dec.project(encoded, out=self.enc_proj)
        # the reference switches decoder kernels (and numerics) at 1024 frames per request
        # (src/cuda/decoder.rs:88); a batch of short utterances needs one launch only
        cache = "auto" if self.longest_out_frames >= dec_mod.LONG_REQUEST_FRAMES else "fp16"
        self.dec.decode(self.enc_proj, utterances, self.seg_stride, self.out_frames_dev, self.max_tokens,
                        self.tokens, self.durations, self.counts, lstm_cache=cache)

    def transcribe_batch(self, mel_host):
        """mel_host: pinned fp32 CPU tensor [U, frames, 128].  Returns a list of int32 numpy
        token arrays (one per utterance).  Includes the H2D copy of the inputs and the D2H
        read of the result (pipeline.rs:398, :409)."""
        utterances = mel_host.shape[0]
        self.mel_dev[:utterances].copy_(mel_host, non_blocking=True)
        self.run_resident(utterances)
        self.counts_host.copy_(self.counts, non_blocking=True)
        self.tokens_host.copy_(self.tokens, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        status = self.status()
        if status != 0:
            raise RuntimeError(f"libpk100 reported an expired bounded wait (status {status})")
        counts = self.counts_host.numpy()
        return [self.tokens_host[u, :int(counts[u])].numpy().copy() for u in range(utterances)]

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

    def status(self):
        return (self.enc.status(self.arena, self.ws) | int(self.dec.status.item()) | int(self.sub.status.item()))
