"""CPU oracle -- whole path for one utterance (TEST INFRASTRUCTURE, not product code):
mel -> subsampling -> encoder blocks -> encoder projection -> TDT greedy decode,
restating the order of `run_prepared` (src/cuda/pipeline.rs:437-608).  Also the timed CPU
baseline of the benchmark."""
from __future__ import annotations

import time

import numpy as np

from . import decoder as D
from . import ops as O
from .codec import f16_round


def encode(mel, sub_w, prepared_layers, taus):
    x = O.subsampling(mel, sub_w)
    valid = x.shape[0]
    for p, (t1, t2) in zip(prepared_layers, taus):
        x = O.encoder_layer(x, p, valid, t1, t2)
    return x


def project(encoded16, dec_w):
    return f16_round(np.asarray(encoded16, np.float64) @ dec_w["w_enc"].astype(np.float64).T + dec_w["b_enc"])


def transcribe(mel, sub_w, prepared_layers, taus, dec_w):
    encoded = encode(mel, sub_w, prepared_layers, taus)
    proj = project(encoded, dec_w)
    tokens, steps, ambiguous = D.tdt_greedy(proj, dec_w, proj.shape[0])
    return tokens, encoded, ambiguous


def timed_sample(mel, sub_w, prepared_layers, taus, dec_w, sample_layers, sample_frames, total_layers,
                 sub_fraction=4):
    """Times a bounded sample of one utterance on the host cores and extrapolates to the full
    utterance: subsampling of the first 1/`sub_fraction` of the mel frames (x sub_fraction),
    `sample_layers` encoder blocks at full length (x total/sample), the projection, and
    `sample_frames` decoder frames (x frames/sample).  Returns
    (estimated seconds per utterance, breakdown dict)."""
    part = mel[: mel.shape[0] // sub_fraction]
    t0 = time.perf_counter()
    xs = O.subsampling(part, sub_w)
    t_sub = (time.perf_counter() - t0) * sub_fraction
    # full-length encoder input for the block sample: the sampled rows tiled to T
    valid = (((mel.shape[0] + 1) // 2 + 1) // 2 + 1) // 2
    x = np.tile(xs, (valid // xs.shape[0] + 1, 1))[:valid]
    t0 = time.perf_counter()
    for p, (t1, t2) in list(zip(prepared_layers, taus))[:sample_layers]:
        x = O.encoder_layer(x, p, valid, t1, t2)
    t_layers = time.perf_counter() - t0
    t0 = time.perf_counter()
    proj = project(x, dec_w)
    t_proj = time.perf_counter() - t0
    frames = min(sample_frames, valid)
    t0 = time.perf_counter()
    D.tdt_greedy(proj, dec_w, frames)
    t_dec = time.perf_counter() - t0
    total = t_sub + t_layers * (total_layers / max(sample_layers, 1)) + t_proj + t_dec * (valid / max(frames, 1))
    return total, dict(subsampling_s=t_sub, layers_s=t_layers, projection_s=t_proj, decoder_s=t_dec,
                       sample_layers=sample_layers, sample_frames=frames, frames=valid)
