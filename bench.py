#!/usr/bin/env python
"""Benchmark of the B200 hot path: real-time factor (audio seconds / wall seconds) of
TDT transcription from log-mel frames, data-parallel over the GPUs of one node.

    python bench.py --gpus N --steps K --warmup W          (N > 1: launched by torchrun)
    python bench.py --impl reference ...                    (CPU reference arm)

One step = one batch of 8 synthetic 60 s utterances per GPU through subsampling, the
24-block FastConformer encoder (mixed FP8 / INT8 / INT4 GEMMs, tile-sparse FF hidden
activations, local relative-position attention), the encoder projection and the TDT greedy
decode.  Weak scaling: every GPU gets its own 8 utterances (utterance u -> rank u mod N),
there is no collective on the compute path; token ids are gathered on the host.

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

UTTERANCES_PER_GPU = 8
MEL_FRAMES = 6000           # 60 s at 10 ms hop
AUDIO_SECONDS = 60.0
ENCODER_LAYERS = 24
SEED = 4
METRIC = "RTFx (audio s / wall s)"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--decoder-layers", type=int, default=1,
                    help="LSTM layers of the prediction network (benchmark config: 1; the reference model: 2)")
    ap.add_argument("--layers", type=int, default=ENCODER_LAYERS)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--tau-cache", default=None,
                    help="JSON file with calibrated tile thresholds: loaded if present, written otherwise")
    ap.add_argument("--micro", default=None,
                    choices=["ff_expand", "ff_contract", "qkv", "out_proj", "out_proj_f16", "attention", "layer_norm", "depthwise", "decode"],
                    help="time ONE kernel of the path on synthetic operands (used for ncu captures)")
    ap.add_argument("--rows", type=int, default=6144, help="rows (M) of the --micro case")
    ap.add_argument("--out-proj", default="f16", choices=["f16", "int4"],
                    help="resident form of the INT4-g128 out-proj weights: expanded fp16 (default) or packed codes "
                         "dequantised inside the GEMM; same bits")
    ap.add_argument("--subsampling", default="fp16", choices=["fp16", "fp8"],
                    help="pointwise / projection GEMMs of the subsampling stage: fp16 (default) or the reference's "
                         "long-request variant with E4M3 activations and weights")
    ap.add_argument("--plain-launch", action="store_true",
                    help="launch the kernels of the block chain in plain stream order (no programmatic dependent launch)")
    ap.add_argument("--cta-pairs", action="store_true",
                    help="256-column GEMM tiles on CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles)")
    ap.add_argument("--utterances", type=int, default=UTTERANCES_PER_GPU,
                    help="utterances per GPU and step (8 = benchmark configuration 4; 1 = configuration 3, "
                         "the batch-1 encoder + decode)")
    ap.add_argument("--encode-groups", type=int, default=1,
                    help="groups that pass through subsampling and the encoder one after the other (1 = the whole "
                         "batch in one pass; more = a group's decode runs under the next group's encode)")
    ap.add_argument("--stream-depth", type=int, default=4,
                    help="sets of request buffers in the streamed measurement (batches in flight)")
    ap.add_argument("--stream-decode-groups", type=int, default=1,
                    help="decoder clusters per batch in the streamed (throughput) measurement")
    ap.add_argument("--decode-groups", type=int, default=None,
                    help="groups decoded side by side, one 16-CTA cluster each (default: as many clusters as the "
                         "device holds at once)")
    ap.add_argument("--no-reference-kernels", action="store_true",
                    help="skip the timing of the reference's own kernels (oracle/_ref) beside this build's")
    return ap.parse_args()


# DRAM bytes (read + write) of one FF-expand launch at 32768 rows, from the committed ncu summary.
NCU_DRAM_BYTES_AT_32768_ROWS = 145.5e6


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], bf16=d["bf16_tflops"], bf16_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()            # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # samples taken under load: the top half of the observed clocks excludes idle gaps
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


def load_synth():
    """The seeded synthetic tensors (l4-parakeet-rs_b200/synth.py) loaded by file path: the CPU arms
    need the same weights as the GPU arm without importing the package, which would map libpk100.so
    into a process that must not touch it."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("pk100_synth", ROOT / "l4-parakeet-rs_b200" / "synth.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class CpuReference:
    """The CPU restatement of the path (oracle/) timed on the host cores: torch fp32 matmuls on all
    host threads for the GEMMs and the attention, numpy for the bit-exact quantisers (the oracle's
    timing mode; its parity mode accumulates in float64).  `sample()` times a bounded sample of one
    utterance and extrapolates; `whole()` runs one whole utterance."""

    def __init__(self, synth, layers_total, decoder_layers, sample_layers=1, sample_frames=100):
        import torch
        from oracle import ops as O
        torch.set_num_threads(os.cpu_count() or 1)
        O.set_timing_mode(True)
        self.layers_total, self.sample_layers, self.sample_frames = layers_total, sample_layers, sample_frames
        self.synth, self.decoder_layers = synth, decoder_layers
        self.mel = synth.mel_input(100, MEL_FRAMES)
        self.sub_w = synth.subsampling_weights(SEED)
        self.prepared = [O.prepare_layer(synth.layer_weights(SEED, l)) for l in range(sample_layers)]
        self.dec_w = synth.decoder_weights(SEED, decoder_layers)

    def sample(self):
        from oracle import pipeline as P
        taus = [(0.0, 0.0)] * self.sample_layers
        total_s, parts = P.timed_sample(self.mel, self.sub_w, self.prepared, taus, self.dec_w,
                                        self.sample_layers, self.sample_frames, self.layers_total)
        what = (f"1 of 8 utterances: subsampling of the first 15 s of mel ({parts['subsampling_s']:.2f} s after "
                f"x4), {self.sample_layers} of {self.layers_total} encoder blocks at T={parts['frames']} "
                f"({parts['layers_s']:.2f} s, scaled x{self.layers_total // self.sample_layers}), projection, "
                f"{parts['sample_frames']} of {parts['frames']} decoder frames ({parts['decoder_s']:.2f} s, "
                f"scaled); torch fp32 matmuls on all host threads + numpy quantisers")
        return AUDIO_SECONDS / total_s, what

    def whole(self):
        """One whole 60 s utterance, nothing extrapolated (about 20-30 s of CPU work)."""
        from oracle import ops as O, pipeline as P
        prepared = self.prepared + [O.prepare_layer(self.synth.layer_weights(SEED, l))
                                    for l in range(len(self.prepared), self.layers_total)]
        taus = [(0.0, 0.0)] * self.layers_total
        t0 = time.perf_counter()
        tokens, _, _ = P.transcribe(self.mel, self.sub_w, prepared, taus, self.dec_w)
        total_s = time.perf_counter() - t0
        what = (f"1 whole 60 s utterance of the 8 (subsampling, {self.layers_total} encoder blocks at T=750, projection, "
                f"TDT greedy decode of {len(tokens)} tokens; tile thresholds off) in {total_s:.1f} s; torch fp32 "
                f"matmuls on all host threads + numpy quantisers")
        return AUDIO_SECONDS / total_s, what


def run_reference(args, rank):
    """Reference arm: the reference has no CPU encoder of its own (its CPU code on this path
    is the weight quantiser and sampled dot-product checkers) and its Rust host cannot be
    built here, so this arm times the CPU restatement of the same path (oracle/)."""
    if rank != 0:
        return
    pk_cpu = load_synth()

    values, sample = [], ""
    ref = CpuReference(pk_cpu, args.layers, args.decoder_layers)
    for _ in range(min(args.warmup, 1)):
        ref.sample()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        v, sample = ref.sample()
        values.append(v)
    wall = time.perf_counter() - t0
    value = statistics.median(values)
    cores = os.cpu_count()
    line = dict(impl="reference", metric=METRIC, value=value, unit="x real time", n_gpus=args.gpus,
                steps=args.steps, warmup=args.warmup, ms_per_step=wall / args.steps * 1e3,
                higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32 (CPU restatement)",
                data="synthetic",
                config=workload_config(args),
                cpu_baseline=dict(value=value, unit="x real time", cores=cores, kind="port", sample=sample),
                e2e=dict(value=value, unit="x real time", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                gpu_launches=0)
    print(json.dumps(line), flush=True)


def workload_config(args):
    return dict(
        workload=((f"end-to-end TDT transcription, per-GPU share of 64 x 60 s utterances over 8 GPUs: 8 x 60 s utterances "
                   "(mel [6000,128] ~N(0,1), seeds 100+u) " if args.utterances >= UTTERANCES_PER_GPU else
                   f"24-block encoder + TDT decode, batch {args.utterances} x 60 s (benchmark configuration 3 at batch 1) ") +
                  "-> 8x conv subsampling -> 24-block FastConformer encoder (T=750 per utterance, 768-row "
                  "segments) -> TDT greedy decode"),
        utterances_per_gpu=min(args.utterances, UTTERANCES_PER_GPU), audio_seconds_per_utterance=AUDIO_SECONDS,
        encode_groups=args.encode_groups, decode_groups=args.decode_groups or "one per decoder cluster the device holds",
        encoder_layers=args.layers, decoder_lstm_layers=args.decoder_layers,
        precision_map=("FF: E4M3 x E4M3 expand + SiLU + 70% zero 128x64 tiles -> INT8 x INT8 contract with "
                       "tile skip; QKV INT8; out-proj INT4-g128 values, fp16 MMA (" +
                       ("expanded to fp16 at load" if args.out_proj == "f16" else "dequantised inside the GEMM") +
                       "); conv pointwise E4M3; attention fp16 (tcgen05)"),
        weights="random-init N(0,0.02), seed 4",
        l2=("no flush: each step streams ~0.6 GB of weights and ~0.3 GB of activations, "
            "several times the 126 MB L2"),
        parallelism="utterance data-parallel, no collective on the compute path, host gather of tokens")


def run_micro(args):
    """One kernel of the path in isolation: `--micro NAME --rows M --steps K --warmup W`.
    Prints a JSON line with the average launch time and the achieved rate."""
    import numpy as np
    import torch
    pk = importlib.import_module("l4-parakeet-rs_b200")
    L = pk.lib
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    if args.cta_pairs:
        L.lib.pk100_set_gemm_cta_pairs(1)
    if args.plain_launch:
        L.lib.pk100_set_dependent_launch(0)
    g = torch.Generator(device="cpu").manual_seed(1)
    m = args.rows
    peaks = measured_peaks()

    def rand16(*shape, std=1.0):
        return (torch.randn(shape, generator=g) * std).half().to(dev)

    if args.micro in ("out_proj", "out_proj_f16"):
        # attention output projection: fp16 activations x INT4 group-128 weights dequantised in shared memory
        # (out_proj_f16: the same product with the weights expanded to fp16 beforehand, for comparison)
        x = rand16(m, 1024)
        codes, gs = pk.ops.pack_weight_rows(rand16(1024, 1024, std=0.02), L.PACK_S4_G128)
        res = rand16(m, 1024)
        if args.micro == "out_proj":
            call = lambda: pk.ops.gemm(x, codes, kind=L.KIND_F16_W4G128, out=res, residual=res, b_group_scales=gs, n=1024)
        else:
            w16 = pk.ops.dequant_w4g128(codes, gs)
            call = lambda: pk.ops.gemm(x, w16, kind=L.KIND_F16, out=res, residual=res)
        flops, nbytes = 2.0 * m * 1024 * 1024, m * 1024 * 2 * 3 + 1024 * 512 + 8 * 1024 * 2
        peak, unit, bound = peaks["bf16"], "TFLOP/s", "tensor"
        work = flops / 1e12
    elif args.micro in ("ff_expand", "ff_contract", "qkv"):
        if args.micro == "ff_expand":
            x = rand16(m, 1024)
            w = rand16(4096, 1024, std=0.02)
            xq = pk.ops.quantize_fp8_fixed(x, 56.0)
            wq, ws = pk.ops.pack_weight_rows(w, L.PACK_E4M3)
            out = torch.empty((m, 4096), dtype=torch.int8, device=dev)
            keep = torch.zeros(((m + 127) // 128, 64), dtype=torch.uint8, device=dev)
            stats = torch.zeros(((m + 127) // 128, 64), dtype=torch.float32, device=dev)
            fn = lambda tau=0.0: pk.ops.gemm(xq, wq, kind=L.KIND_E4M3, epilogue=L.EPI_SPARSE_OUT, out=out,
                                             out_type=L.OUT_S8, out_scale=32.0, row_scale=8.0 / 448.0,
                                             col_scales=ws, tau=tau, keep_out=keep, stats_out=stats)
            fn()
            torch.cuda.synchronize()
            tau = pk.encoder.tau_for_zero_fraction(stats.cpu().numpy(), 0.7)
            call = lambda: fn(tau)
            flops, nbytes = 2.0 * m * 4096 * 1024, m * 1024 + 4096 * 1024 + m * 4096
            peak, unit, bound = 2 * peaks["bf16"], "TFLOP/s", "tensor"
        elif args.micro == "ff_contract":
            h = torch.randint(-100, 100, (m, 4096), generator=g, dtype=torch.int8).to(dev)
            keep_h = (torch.rand(((m + 127) // 128, 64), generator=g) < 0.3).to(torch.uint8)
            mask = keep_h.repeat_interleave(128, 0)[:m].repeat_interleave(64, 1).to(dev)
            h = h * mask.to(torch.int8)
            keep = keep_h.to(dev)
            w = rand16(1024, 4096, std=0.02)
            wq, ws = pk.ops.pack_weight_rows(w, L.PACK_S8)
            xres = rand16(m, 1024)
            call = lambda: pk.ops.gemm(h, wq, kind=L.KIND_S8, out=xres, row_scale=1.0 / 32.0, col_scales=ws,
                                       residual=xres, alpha=0.5, keep_in=keep)
            live = float(keep_h.float().mean())
            flops, nbytes = 2.0 * m * 4096 * 1024 * live, m * 4096 * live + 1024 * 4096 + 2 * m * 1024 * 2
            peak, unit, bound = 2 * peaks["bf16"], "TOP/s (executed)", "tensor"
        else:
            x = rand16(m, 1024)
            xq, xs = pk.ops.layer_norm(x, torch.ones(1024, device=dev).half(), torch.zeros(1024, device=dev).half(),
                                       L.LN_S8_ROW)
            wq, ws = pk.ops.pack_weight_rows(rand16(3072, 1024, std=0.02), L.PACK_S8)
            out = torch.empty((m, 3072), dtype=torch.float16, device=dev)
            call = lambda: pk.ops.gemm(xq, wq, kind=L.KIND_S8, out=out, row_scales=xs, col_scales=ws)
            flops, nbytes = 2.0 * m * 3072 * 1024, m * 1024 + 3072 * 1024 + m * 3072 * 2
            peak, unit, bound = 2 * peaks["bf16"], "TOP/s", "tensor"
        work = flops / 1e12
    elif args.micro == "attention":
        seg = 768
        segs = max(1, m // seg)
        m = segs * seg
        qkv = rand16(m, 3072)
        pos, u, v = rand16(8, 272, 128), rand16(8, 128, std=0.02), rand16(8, 128, std=0.02)
        out = torch.empty((m, 1024), dtype=torch.float16, device=dev)
        if os.environ.get("PK100_ATTENTION") == "mma":
            call = lambda: pk.ops.local_attention(qkv[:, :1024], qkv[:, 1024:2048], qkv[:, 2048:], pos, u, v,
                                                  seg_stride=seg, valid_rows=750, out=out)
        else:
            call = lambda: pk.ops.local_attention_tcgen05(qkv[:, :1024], qkv[:, 1024:2048], qkv[:, 2048:], pos, u, v,
                                                          seg_stride=seg, valid_rows=750, out=out)
        nbytes = m * 1024 * 2 * 4
        work, peak, unit, bound = nbytes / 1e9, peaks["hbm_gbs"], "GB/s", "hbm"
    elif args.micro == "depthwise":
        seg = 768
        segs = max(1, m // seg)
        m = segs * seg
        g_in, wdw = rand16(m, 1024), rand16(1024, 9, std=0.3)
        one, zero = torch.ones(1024, device=dev), torch.zeros(1024, device=dev)
        call = lambda: pk.ops.depthwise_bn_silu(g_in, wdw, one, zero, zero, one, quantize=True, seg_stride=seg,
                                                valid_rows=750)
        nbytes = m * 1024 * 3 + m * 4
        work, peak, unit, bound = nbytes / 1e9, peaks["hbm_gbs"], "GB/s", "hbm"
    elif args.micro == "layer_norm":
        x = rand16(m, 1024)
        gam, bet = torch.ones(1024, device=dev).half(), torch.zeros(1024, device=dev).half()
        out = torch.empty((m, 1024), dtype=torch.uint8, device=dev)
        call = lambda: pk.ops.layer_norm(x, gam, bet, L.LN_E4M3_FIXED, inv_scale=56.0, out=out)
        nbytes = m * 1024 * 3
        work, peak, unit, bound = nbytes / 1e9, peaks["hbm_gbs"], "GB/s", "hbm"
    else:
        dec = pk.decoder.TdtDecoder(pk.synth.decoder_weights(SEED, args.decoder_layers), dev)
        enc = rand16(8 * 768, 640, std=0.5)
        fr = torch.full((8,), min(750, max(1, args.rows)), dtype=torch.int32, device=dev)
        call = lambda: dec.decode(enc, 8, 768, fr, 7500)
        work, peak, unit, bound, nbytes = 0.0, 1.0, "rounds/s", "latency", 0
    for _ in range(max(args.warmup, 1)):
        call()
    torch.cuda.synchronize()
    # `steps` back-to-back launches replayed from a CUDA graph, so the host-side cost of a
    # launch (ctypes, tensor-map encoding) stays out of the device timing
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for _ in range(args.steps):
                call()
        graph.replay()
        side.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(side)
        graph.replay()
        e1.record(side)
        side.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    achieved = work / (ms * 1e-3) if work else None
    line = dict(micro=args.micro, rows=m, avg_launch_ms=ms, achieved=achieved, unit=unit, bound=bound,
                peak=peak, frac=(achieved / peak if achieved else None),
                algorithmic_bytes=nbytes, peak_source=peaks["source"])
    if args.micro == "ff_expand":
        # library bar, same run: cuBLASLt E4M3 GEMM of the same shape with a plain fp16 epilogue
        # (no SiLU, no tile statistics, no INT8 encoding) -- context for the fraction above
        try:
            a8 = torch.randn(m, 1024, device=dev).to(torch.float8_e4m3fn)
            b8 = torch.randn(4096, 1024, device=dev).to(torch.float8_e4m3fn)
            one = torch.ones((), device=dev)
            lib = lambda: torch._scaled_mm(a8, b8.t(), scale_a=one, scale_b=one, out_dtype=torch.float16)
            for _ in range(3):
                lib()
            torch.cuda.synchronize()
            l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            l0.record()
            for _ in range(args.steps):
                lib()
            l1.record()
            torch.cuda.synchronize()
            lib_ms = l0.elapsed_time(l1) / args.steps
            line["library_bar"] = dict(what="cuBLASLt E4M3 (torch._scaled_mm), plain fp16 epilogue",
                                       avg_launch_ms=lib_ms, tflops=flops / (lib_ms * 1e-3) / 1e12)
        except Exception as exc:  # noqa: BLE001 - the bar is optional context
            line["library_bar"] = dict(unavailable=str(exc)[:120])
    print(json.dumps(line), flush=True)


def time_device(call, iters, warmup=20, samples=7):
    """Median device time of one `call` in ms (CUDA events; the reference's protocol,
    src/cuda.rs:574-618: >= 20 warm-ups, 7 samples of `iters` back-to-back launches, median).  The
    launches of a sample are replayed from a CUDA graph so that host-side launch cost stays out."""
    import torch
    for _ in range(warmup):
        call()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for _ in range(iters):
                call()
        graph.replay()
        side.synchronize()
        times = []
        for _ in range(samples):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(side)
            graph.replay()
            e1.record(side)
            side.synchronize()
            times.append(e0.elapsed_time(e1) / iters)
    return statistics.median(times)


def measure_tensor_peaks(dev):
    """Same-run library GEMM rates at 8192^3: cuBLASLt E4M3 (torch._scaled_mm) and INT8
    (torch._int_mm), burst (best of 10) and sustained (back to back for about a second)."""
    import torch
    n = 8192
    out = {}
    cases = {}
    try:
        a8 = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
        b8 = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
        one = torch.ones((), device=dev)
        cases["fp8_e4m3"] = lambda: torch._scaled_mm(a8, b8.t(), scale_a=one, scale_b=one, out_dtype=torch.float16)
    except Exception as exc:  # noqa: BLE001
        out["fp8_e4m3"] = dict(unavailable=str(exc)[:120])
    try:
        ai = torch.randint(-100, 100, (n, n), device=dev, dtype=torch.int8)
        bi = torch.randint(-100, 100, (n, n), device=dev, dtype=torch.int8)
        cases["int8"] = lambda: torch._int_mm(ai, bi.t())
    except Exception as exc:  # noqa: BLE001
        out["int8"] = dict(unavailable=str(exc)[:120])
    for name, fn in cases.items():
        try:
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            best = 1e9
            for _ in range(10):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                best = min(best, e0.elapsed_time(e1))
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = max(10, int(1000.0 / best))
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            flop = 2.0 * n ** 3
            out[name] = dict(burst_tops=flop / (best * 1e-3) / 1e12,
                             sustained_tops=flop / (e0.elapsed_time(e1) / reps * 1e-3) / 1e12, shape=f"{n}^3")
        except Exception as exc:  # noqa: BLE001
            out[name] = dict(unavailable=str(exc)[:120])
    return out


def reference_kernel_times(pk, dev):
    """The reference's own kernels (kernels/sm89/*.cu compiled for sm_100a into oracle/_ref/ by
    oracle/build_ref.py), launched the way its Rust host launches them, timed beside this build's
    kernel for the same operator on the same operands: the "kernel to beat" on this GPU.  A checker
    leg like the CPU baseline; nothing here is on the product path."""
    import numpy as np
    import torch
    try:
        from oracle import refkernels as R
    except Exception as exc:  # noqa: BLE001 - cuda-python absent
        return dict(unavailable=f"oracle.refkernels cannot be imported: {str(exc)[:80]}")
    if not R.available():
        return dict(unavailable="oracle/_ref/*.cubin not built (no reference checkout at build time)")
    L = pk.lib
    g = torch.Generator(device="cpu").manual_seed(7)
    r16 = lambda *shape, std=1.0: (torch.randn(shape, generator=g) * std).half().to(dev)
    ones, zeros = torch.ones(1024, device=dev), torch.zeros(1024, device=dev)
    rows_out = {}
    for rows in (752, 6144):
        seg = 768 if rows % 768 == 0 else rows
        valid = 750 if seg == 768 else rows - 2
        x = r16(rows, 1024)
        gam, bet = ones.half(), zeros.half()
        w1 = r16(4096, 1024, std=0.02)
        xq = pk.ops.quantize_fp8_fixed(x, 56.0)
        w1q, w1s = pk.ops.pack_weight_rows(w1, L.PACK_E4M3)
        h16 = torch.empty((rows, 4096), dtype=torch.float16, device=dev)
        wqkv = r16(3072, 1024, std=0.02)
        x8, x8s = pk.ops.layer_norm(x, gam, bet, L.LN_S8_ROW)
        wq8, wq8s = pk.ops.pack_weight_rows(wqkv, L.PACK_S8)
        qkv = torch.empty((rows, 3072), dtype=torch.float16, device=dev)
        bias3 = torch.zeros(3072, device=dev)
        wo = r16(1024, 1024, std=0.02)
        o16 = torch.empty((rows, 1024), dtype=torch.float16, device=dev)
        e = r16(rows, 2048)
        wdw = r16(1024, 9, std=0.3)
        pos, bu, bv = r16(8, 272, 128), r16(8, 128, std=0.02), r16(8, 128, std=0.02)
        att = torch.empty((rows, 1024), dtype=torch.float16, device=dev)
        glu = pk.ops.glu_masked(e, seg_stride=seg, valid_rows=valid)
        ops = {
            "layer_norm": (lambda: R.layer_norm(x, gam, bet, rows, rows),
                           lambda: pk.ops.layer_norm(x, gam, bet, L.LN_F16, out=o16), "pk_sm89_layer_norm"),
            "ff_expand_fp8_silu": (lambda: R.ffn_expand_fp8(xq, w1q, w1s, rows),
                                   lambda: pk.ops.gemm(xq, w1q, kind=L.KIND_E4M3, out=h16, row_scale=8.0 / 448.0,
                                                       col_scales=w1s, act=L.ACT_SILU),
                                   "pk_sm89_ffn_expand_fp8_async"),
            "qkv_int8_linear": (lambda: R.int8_linear(x8, wq8, wq8s, bias3, rows, 3072, 1024, 0.01),
                                lambda: pk.ops.gemm(x8, wq8, kind=L.KIND_S8, out=qkv, row_scales=x8s, col_scales=wq8s),
                                "pk_sm89_int8_linear_epilogue"),
            "fp16_linear_1024": (lambda: R.fp16_linear(x, wo, None, None, rows, 1024, 1024),
                                 lambda: pk.ops.gemm(x, wo, kind=L.KIND_F16, out=o16), "pk_sm89_fp16_linear_epilogue"),
            "glu_masked": (lambda: R.glu_masked(e, rows, rows, valid), lambda: pk.ops.glu_masked(e, seg, valid),
                           "pk_sm89_glu_masked"),
            "depthwise_bn_silu": (lambda: R.depthwise_bn_silu(glu, wdw, ones, zeros, zeros, ones, rows, rows),
                                  lambda: pk.ops.depthwise_bn_silu(glu, wdw, ones, zeros, zeros, ones, seg_stride=seg,
                                                                   valid_rows=valid),
                                  "pk_sm89_depthwise_batchnorm_silu"),
            "local_attention": (lambda: R.local_attention_scalar(qkv[:, :1024].contiguous(), qkv[:, 1024:2048].contiguous(),
                                                                 qkv[:, 2048:].contiguous(), pos, bu, bv, rows, rows, rows),
                                lambda: pk.ops.local_attention(qkv[:, :1024], qkv[:, 1024:2048], qkv[:, 2048:], pos, bu, bv,
                                                               seg_stride=seg, valid_rows=valid, out=att),
                                "pk_sm89_local_relpos_attention (its fp32 scalar kernel; the reference's T=750 kernel "
                                "_tc_scores needs its FP8 V repack and is not launched here)"),
        }
        pk.ops.gemm(x8, wq8, kind=L.KIND_S8, out=qkv, row_scales=x8s, col_scales=wq8s)
        res = {}
        for name, (ref_call, own_call, ref_name) in ops.items():
            try:
                slow = name == "local_attention" or name == "fp16_linear_1024"
                iters = 2 if (slow and rows > 1000) else 10
                ref_ms = time_device(ref_call, iters, warmup=20 if not slow else 3)
                own_ms = time_device(own_call, 10)
                res[name] = dict(reference_us=ref_ms * 1e3, this_build_us=own_ms * 1e3, reference_kernel=ref_name,
                                 speedup=ref_ms / own_ms)
            except Exception as exc:  # noqa: BLE001
                res[name] = dict(unavailable=str(exc)[:120])
        rows_out[f"rows_{rows}"] = res
    # decoder: one 120-frame request through the reference's cooperative kernel and through this build's
    try:
        from oracle import decoder as D
        from oracle import codec
        w = D.make_decoder_weights(7, layers=2)
        rng = np.random.default_rng(8)
        frames = 120
        enc = torch.from_numpy(codec.f16_round(rng.standard_normal((frames, 640)) * 0.5)).half().to(dev)
        dw = {k: (torch.from_numpy(np.ascontiguousarray(v)).to(dev) if k.startswith("b_")
                  else torch.from_numpy(np.ascontiguousarray(v, dtype=np.float32)).half().to(dev))
              for k, v in w.items() if k != "layers"}
        sms = torch.cuda.get_device_properties(dev).multi_processor_count

        def timed(fn, reps=5):
            fn()
            torch.cuda.synchronize()
            ts = []
            for _ in range(reps):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                out = fn()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            return statistics.median(ts), out
        ref_ms, ref_tokens = timed(lambda: R.tdt_decode(enc, dw, frames, sms))
        dec = pk.decoder.TdtDecoder(w, dev)
        fr = torch.tensor([frames], dtype=torch.int32, device=dev)
        own_ms, own = timed(lambda: dec.decode(enc, 1, frames, fr, frames * 10))
        steps = frames + len(ref_tokens)
        rows_out["tdt_decode_120_frames"] = dict(
            reference_kernel="pk_sm89_tdt_persistent_v2 (cooperative, one grid barrier per step)",
            reference_ms=ref_ms, this_build_ms=own_ms, steps=steps, reference_us_per_step=ref_ms * 1e3 / steps,
            this_build_us_per_step=own_ms * 1e3 / steps, speedup=ref_ms / own_ms,
            note="whole call: this build's figure includes its per-call weight packing and input-table GEMM")
    except Exception as exc:  # noqa: BLE001
        rows_out["tdt_decode_120_frames"] = dict(unavailable=str(exc)[:120])
    rows_out["protocol"] = ("CUDA events, warm-up, 7 samples x N graph-replayed launches, median (src/cuda.rs:574-618); "
                            "reference kernels compiled unmodified for sm_100a")
    return rows_out


DATASHEET_FP8_DENSE_TFLOPS = 4500.0      # B200 dense FP8 / INT8 (NVIDIA datasheet, HGX B200 per-GPU figure)


def main():
    args = parse_args()
    if args.micro:
        run_micro(args)
        return
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import numpy as np
    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: libpk100 has no CPU path")
    pk = importlib.import_module("l4-parakeet-rs_b200")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    gloo = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
        gloo = dist.new_group(backend="gloo")

    per_gpu = max(1, min(args.utterances, UTTERANCES_PER_GPU))
    total_utts = per_gpu * world
    my_utts = pk.parallel.shard_utterances(total_utts, world, rank)
    if args.cta_pairs:
        pk.lib.lib.pk100_set_gemm_cta_pairs(1)
    if args.plain_launch:
        pk.lib.lib.pk100_set_dependent_launch(0)
    eng = pk.pipeline.PipelineEngine(device, layers=args.layers, decoder_layers=args.decoder_layers,
                                     seed=SEED, max_utterances=per_gpu, mel_frames=MEL_FRAMES,
                                     decode_groups=args.decode_groups, encode_groups=args.encode_groups,
                                     out_proj_resident=args.out_proj, subsampling_precision=args.subsampling)
    mel_host = torch.from_numpy(np.stack([pk.synth.mel_input(100 + u, MEL_FRAMES) for u in my_utts])).pin_memory()
    eng.mel_dev.copy_(mel_host)
    cache = Path(args.tau_cache) if args.tau_cache else None
    if cache is not None and cache.exists():
        taus = json.loads(cache.read_text())
        for l, (t1, t2) in enumerate(taus):
            eng.enc.set_tau(l, t1, t2)
    else:
        eng.calibrate(per_gpu)      # load-time: tile thresholds for 70 % zero tiles
        if cache is not None and rank == 0:
            cache.write_text(json.dumps([[l.ff1.tau, l.ff2.tau] for l in eng.enc.layers]))
    eng.enable_gemm_timing()
    eng.enable_stage_timing()
    torch.cuda.synchronize()

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- warm-up through the public API
    tokens = None
    for _ in range(args.warmup):
        tokens = eng.transcribe_batch(mel_host)
    if eng.status() != 0:
        raise SystemExit("a bounded wait expired inside a kernel")

    # ---- timed: inputs resident in HBM
    sampler = ClockSampler(local_rank)
    sync_all()
    if rank == 0:
        print(f"[bench] kernel launches before the timed region: {pk.lib.lib.pk100_launch_count()}",
              file=sys.stderr, flush=True)
    sampler.start()
    launches0 = pk.lib.lib.pk100_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        eng.run_resident(per_gpu)
    e1.record()
    sync_all()
    launches = pk.lib.lib.pk100_launch_count() - launches0
    own_ms_resident = e0.elapsed_time(e1) / args.steps
    ms_resident = max_over_ranks(own_ms_resident)
    gemm_ms = eng.gemm_times_ms()                      # (ms, rows) of every FF-expand launch of the last step
    stages = eng.stage_times()                         # per decode group of the last step

    # ---- timed: end to end through the public API (host buffers, copies inside)
    sync_all()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    for _ in range(args.steps):
        tokens = eng.transcribe_batch(mel_host)
        gathered = pk.parallel.gather_token_lists({u: t for u, t in zip(my_utts, tokens)}, total_utts, group=gloo)
    e3.record()
    sync_all()
    ms_e2e = max_over_ranks(e2.elapsed_time(e3)) / args.steps
    if eng.status() != 0:
        raise SystemExit("a bounded wait expired inside a kernel")

    # ---- throughput mode: a stream of batches through the public API, batch i + 1 copied in and
    # encoded while batch i is decoded; host wall clock between the first and the last batch's results
    stream_n = max(args.steps, 4) + args.stream_depth
    marks = []
    for toks in eng.transcribe_stream((mel_host for _ in range(stream_n)), decode_groups=args.stream_decode_groups,
                                      depth=args.stream_depth):
        marks.append(time.perf_counter())
        if any(len(a) != len(b) or (a != b).any() for a, b in zip(toks, tokens)):
            raise SystemExit("the streamed batches returned other tokens than transcribe_batch")
    # steady state: from the results of batch `depth - 1` (the pipeline is full) to the last batch's
    first = args.stream_depth - 1
    ms_stream = max_over_ranks((marks[-1] - marks[first]) * 1e3 / (len(marks) - 1 - first))
    clocks = sampler.stop()

    audio_per_step = AUDIO_SECONDS * total_utts
    value = audio_per_step / (ms_resident / 1e3)
    e2e_value = audio_per_step / (ms_e2e / 1e3)

    # ---- the decoder: the sequential chain that bounds the step.  A round = one joint evaluation
    # per live utterance; an utterance needs (frames + tokens) rounds, the batch as many as its longest.
    dec_rounds = sum(s["rounds"] for s in stages)
    dec_ms = sum(s["decode_ms"] for s in stages)
    longest = max(s["rounds"] for s in stages)
    mine = dict(rank=rank, ms_per_step=own_ms_resident, longest_chain_rounds=longest, groups=stages,
                decode_us_per_round=dec_ms * 1e3 / max(dec_rounds, 1),
                decode_end_ms=max(s["decode_end_ms"] for s in stages),
                encode_ms=sum({s["encode_group"]: s["encode_ms"] for s in stages}.values()))
    per_rank = [mine]
    if world > 1:
        per_rank = [None] * world
        dist.all_gather_object(per_rank, mine, group=gloo)
    decoder = dict(kernel="tdt_cluster_kernel (one 16-CTA cluster per decode group)",
                   decode_groups=len(stages), rounds=dec_rounds, decode_ms=dec_ms,
                   us_per_round=mine["decode_us_per_round"], longest_chain_rounds=longest,
                   share_of_step=max(s["decode_end_ms"] - s["decode_start_ms"] for s in stages) / own_ms_resident,
                   note=("rank 0, last timed step; a round = one joint evaluation per live utterance (a token or a "
                         "blank), the groups decode side by side; the step ends when the slowest group's chain ends: "
                         "ms_per_step ~ that group's decode_start_ms + its rounds x us_per_round"))

    # ---- roofline of the designated kernel: FF expand (E4M3 tcgen05 GEMM + SiLU + tile threshold)
    peaks = measured_peaks()
    # every FF-expand launch of the last timed step (all groups): total flops / total time
    rows = sum(r for _, r in gemm_ms) / len(gemm_ms)
    flops = 2.0 * rows * 4096 * 1024
    gemm_avg_ms = sum(ms for ms, _ in gemm_ms) / len(gemm_ms)
    achieved = flops / (gemm_avg_ms * 1e-3) / 1e12
    fp8_peak = 2.0 * peaks["bf16_sustained"]
    roofline = dict(
        bound="tensor", kernel="gemm_kernel<E4M3, 256, 128B swizzle, SPARSE_OUT> (FF expand 1024->4096)",
        achieved=achieved, peak=fp8_peak, unit="TFLOP/s", frac=achieved / fp8_peak,
        peak_note=(f"2 x {peaks['bf16_sustained']} TFLOP/s: MEASURED_PEAKS.json ({peaks['source']}) holds the "
                   "sustained cuBLAS bf16 figure only; E4M3 runs at twice the bf16 rate on this part"),
        frac_datasheet=achieved / DATASHEET_FP8_DENSE_TFLOPS, datasheet_peak=DATASHEET_FP8_DENSE_TFLOPS,
        launches_timed=len(gemm_ms), avg_launch_ms=gemm_avg_ms, rows_per_launch=rows,
        flops_per_launch=flops,
        # dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this kernel at 32768 rows,
        # scaled to this launch by its rows: operand and output bytes all grow in proportion to the
        # rows except the 4 MB of weights
        traffic=NCU_DRAM_BYTES_AT_32768_ROWS * rows / 32768.0,
        traffic_note="scaled from an ncu capture at 32768 rows; inside the step the bytes of a launch are largely L2 hits")

    line = dict(metric=METRIC, value=value, unit="x real time", n_gpus=world, steps=args.steps,
                warmup=args.warmup, ms_per_step=ms_resident, higher_is_better=True, scaling="weak",
                vs_baseline=None, dtype="e4m3/s8/s4 operands, f32/s32 accumulate, f16 activations",
                data="synthetic", config=workload_config(args), clocks=clocks,
                e2e=dict(value=e2e_value, unit="x real time", ms_per_step=ms_e2e,
                         h2d_bytes_per_step=int(mel_host.numel() * 4),
                         d2h_bytes_per_step=int(eng.tokens_host.numel() * 4 + eng.counts_host.numel() * 4)),
                throughput=dict(value=AUDIO_SECONDS * total_utts / (ms_stream / 1e3), unit="x real time",
                                ms_per_batch=ms_stream, batches=stream_n, decode_groups=args.stream_decode_groups,
                                depth=args.stream_depth,
                                note=("PipelineEngine.transcribe_stream: the same batch from pinned host memory over and "
                                      "over, `depth` batches in flight: one is encoded beside the decoder clusters of the "
                                      "earlier ones; host wall clock per batch in steady state, max over ranks; same "
                                      "tokens as e2e")),
                gpu_launches=int(launches), roofline=roofline, decoder=decoder, per_rank=per_rank,
                tensor_map_cache=dict(zip(("hits", "misses"), pk.lib.tensor_map_cache_stats())),
                tokens_per_utterance=[int(len(t)) for t in tokens])

    if rank == 0:
        # same-run library rates: the measured FP8 / INT8 denominators MEASURED_PEAKS.json lacks
        lib_peaks = measure_tensor_peaks(device)
        line["peaks"] = dict(library_8192=lib_peaks, datasheet_fp8_int8_dense_tops=DATASHEET_FP8_DENSE_TFLOPS,
                             measured_file=dict(bf16_tflops=peaks["bf16"], bf16_tflops_sustained=peaks["bf16_sustained"],
                                                hbm_gbs=peaks["hbm_gbs"], source=peaks["source"]))
        fp8 = lib_peaks.get("fp8_e4m3", {})
        if "sustained_tops" in fp8:
            roofline["frac_measured_fp8"] = achieved / fp8["sustained_tops"]
            roofline["measured_fp8_peak"] = fp8["sustained_tops"]
    if rank == 0 and world == 1 and not args.no_reference_kernels:
        line["reference_kernels"] = reference_kernel_times(pk, device)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        v, sample = CpuReference(load_synth(), args.layers, args.decoder_layers).whole()
        line["cpu_baseline"] = dict(value=v, unit="x real time", cores=os.cpu_count(), kind="port", sample=sample)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
