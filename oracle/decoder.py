"""CPU oracle -- TDT greedy decode (TEST INFRASTRUCTURE, not product code).

Restates `tdt_persistent_fp16` (kernels/sm89/decoder.cu:165-447): LSTM
prediction network (gate order i, f, g, o; :251-266, :323-331), prediction
projection (:336-353), joint `W . relu(enc + pred) + b` (:366-392), token argmax
with ties to the lower id (:35-46, :393-414), duration argmax = first strict
maximum (:416-422) and the frame-advance rules (:431-445).  fp16 weights, fp32
state; dot products are accumulated in float64 here, so a decision whose top-2
margin is below `tie_eps` is reported as ambiguous instead of trusted.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32
HIDDEN = 640
TOKENS = 1025
BLANK = 1024
DURATIONS = 5
MAX_SYMBOLS = 10


def make_decoder_weights(seed: int, layers: int = 2, scale: float = 0.05):
    """Random-init decoder tensors with the manifest's shapes
    (src/weights.rs:526-550, :633-644), fp16-rounded weights, fp32 biases."""
    rng = np.random.default_rng(seed)
    r16 = lambda *s: (rng.standard_normal(s) * scale).astype(np.float16).astype(F32)
    r32 = lambda *s: (rng.standard_normal(s) * scale).astype(F32)
    w = {"embedding": r16(TOKENS, HIDDEN) * F32(4.0), "layers": layers,
         "w_pred": r16(HIDDEN, HIDDEN), "b_pred": r32(HIDDEN),
         "w_joint": r16(TOKENS + DURATIONS, HIDDEN), "b_joint": r32(TOKENS + DURATIONS),
         "w_enc": r16(HIDDEN, 1024), "b_enc": r32(HIDDEN)}
    w["embedding"] = w["embedding"].astype(np.float16).astype(F32)
    for l in range(layers):
        w[f"w_ih{l}"] = r16(4 * HIDDEN, HIDDEN)
        w[f"w_hh{l}"] = r16(4 * HIDDEN, HIDDEN)
        w[f"b_ih{l}"] = r32(4 * HIDDEN)
        w[f"b_hh{l}"] = r32(4 * HIDDEN)
    return w


def _sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def lstm_step(x, h, c, w_ih, w_hh, b_ih, b_hh):
    gates = (w_ih.astype(np.float64) @ x.astype(np.float64) + w_hh.astype(np.float64) @ h.astype(np.float64)
             + (b_ih + b_hh).astype(np.float64)).astype(F32)
    i, f, g, o = np.split(gates, 4)
    i, f, o = _sigmoid(i).astype(F32), _sigmoid(f).astype(F32), _sigmoid(o).astype(F32)
    g = np.tanh(g).astype(F32)
    c_new = (f * c + i * g).astype(F32)
    h_new = (o * np.tanh(c_new)).astype(F32)
    return h_new, c_new


def tdt_greedy(enc_proj16, w, frames, tie_eps=1e-4):
    """Returns (tokens, steps, first_ambiguous_token_index or None).
    steps: list of (frame, token, duration, margin)."""
    layers = w["layers"]
    enc = np.asarray(enc_proj16, dtype=F32)
    h = np.zeros((layers, HIDDEN), F32)
    c = np.zeros((layers, HIDDEN), F32)
    cand_h, cand_c = h.copy(), c.copy()
    pred = np.zeros(HIDDEN, F32)
    tokens, steps = [], []
    ambiguous = None
    frame = symbols = 0
    last, emitted, valid = BLANK, False, False
    wj = w["w_joint"].astype(np.float64)
    while frame < frames:
        if not valid:
            x = w["embedding"][last] if emitted else np.zeros(HIDDEN, F32)
            for l in range(layers):
                cand_h[l], cand_c[l] = lstm_step(x, h[l], c[l], w[f"w_ih{l}"], w[f"w_hh{l}"],
                                                 w[f"b_ih{l}"], w[f"b_hh{l}"])
                x = cand_h[l]
            pred = (w["w_pred"].astype(np.float64) @ cand_h[layers - 1].astype(np.float64)
                    + w["b_pred"]).astype(F32)
            valid = True
        joint_in = np.maximum(enc[frame] + pred, F32(0.0)).astype(np.float64)
        logits = (wj @ joint_in + w["b_joint"]).astype(F32)
        tok_logits = logits[:TOKENS]
        token = int(np.argmax(tok_logits))                      # first maximum = lowest id
        top2 = np.partition(tok_logits, -2)[-2:]
        margin = float(top2[1] - top2[0])
        dur_logits = logits[TOKENS:]
        duration = int(np.argmax(dur_logits))                   # first strict maximum
        d2 = np.partition(dur_logits, -2)[-2:]
        margin = min(margin, float(d2[1] - d2[0]))
        if margin < tie_eps and ambiguous is None:
            ambiguous = len(tokens)
        steps.append((frame, token, duration, margin))
        if token != BLANK:
            tokens.append(token)
            last, emitted, valid = token, True, False
            h, c = cand_h.copy(), cand_c.copy()
        symbols += 1
        frame += duration
        if duration != 0 or symbols == MAX_SYMBOLS:
            if duration == 0:
                frame += 1
            symbols = 0
    return np.array(tokens, dtype=np.int32), steps, ambiguous
