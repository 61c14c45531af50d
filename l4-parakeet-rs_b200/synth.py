"""Seeded synthetic model tensors with the shapes of the reference's manifest
(`expected_model_manifest`, src/weights.rs:510-646).  There is no checkpoint in
this environment: weights are random-init, N(0, 0.02) for linears as the
benchmark configurations specify, generated on the CPU with a torch generator.
All arrays are numpy float32 holding fp16-representable values (fp32 for the
BatchNorm statistics and biases)."""
from __future__ import annotations

import numpy as np
import torch

MODEL_WIDTH = 1024
FF_WIDTH = 4096


def _gen(seed):
    g = torch.Generator(device="cpu")
    g.manual_seed(int(seed))
    return g


def _normal(g, shape, std):
    return (torch.randn(shape, generator=g) * std).to(torch.float16).float().numpy()


def layer_weights(seed: int, layer: int, randomize_norms: bool = False, std: float = 0.02):
    g = _gen(seed * 1000 + layer)
    w = {}
    for ff in ("ff1", "ff2"):
        w[f"{ff}_w1"] = _normal(g, (FF_WIDTH, MODEL_WIDTH), std)
        w[f"{ff}_w2"] = _normal(g, (MODEL_WIDTH, FF_WIDTH), std)
    for name in ("wq", "wk", "wv", "wo", "wpos", "wpw2"):
        w[name] = _normal(g, (MODEL_WIDTH, MODEL_WIDTH), std)
    w["wpw1"] = _normal(g, (2 * MODEL_WIDTH, MODEL_WIDTH), std)
    w["bias_u"] = _normal(g, (8, 128), std)
    w["bias_v"] = _normal(g, (8, 128), std)
    w["dw"] = _normal(g, (MODEL_WIDTH, 9), 0.3)
    for ln in ("ff1", "att", "conv", "ff2", "out"):
        if randomize_norms:
            w[f"ln_{ln}_g"] = (1.0 + _normal(g, (MODEL_WIDTH,), 0.1)).astype(np.float16).astype(np.float32)
            w[f"ln_{ln}_b"] = _normal(g, (MODEL_WIDTH,), 0.1)
        else:
            w[f"ln_{ln}_g"] = np.ones(MODEL_WIDTH, np.float32)
            w[f"ln_{ln}_b"] = np.zeros(MODEL_WIDTH, np.float32)
    if randomize_norms:
        w["bn_g"] = (1.0 + 0.1 * torch.randn(MODEL_WIDTH, generator=g)).numpy().astype(np.float32)
        w["bn_b"] = (0.1 * torch.randn(MODEL_WIDTH, generator=g)).numpy().astype(np.float32)
        w["bn_m"] = (0.1 * torch.randn(MODEL_WIDTH, generator=g)).numpy().astype(np.float32)
        w["bn_v"] = (1.0 + 0.2 * torch.rand(MODEL_WIDTH, generator=g)).numpy().astype(np.float32)
    else:
        w["bn_g"] = np.ones(MODEL_WIDTH, np.float32)
        w["bn_b"] = np.zeros(MODEL_WIDTH, np.float32)
        w["bn_m"] = np.zeros(MODEL_WIDTH, np.float32)
        w["bn_v"] = np.ones(MODEL_WIDTH, np.float32)
    return w


def mel_input(seed: int, frames: int = 6000, bins: int = 128):
    """Seeded Gaussian log-mel stand-in [frames, 128] fp32."""
    return torch.randn((frames, bins), generator=_gen(seed)).numpy().astype(np.float32)


def subsampling_weights(seed: int, std: float = 0.02):
    """Shapes of `pre_encode` in the manifest (src/weights.rs:552-568).  The 3x3 taps are
    drawn wider than the linears so that activations keep a usable dynamic range."""
    g = _gen(seed * 1000 + 900)
    w = {"conv0_w": _normal(g, (256, 9), 0.3), "conv0_b": _normal(g, (256,), 0.1)}
    for stage in (1, 2):
        w[f"dw{stage}_w"] = _normal(g, (256, 9), 0.3)
        w[f"dw{stage}_b"] = _normal(g, (256,), 0.1)
        w[f"pw{stage}_w"] = _normal(g, (256, 256), 0.06)
        w[f"pw{stage}_b"] = (torch.randn(256, generator=g) * 0.05).numpy().astype(np.float32)
    w["proj_w"] = _normal(g, (1024, 4096), std)
    w["proj_b"] = (torch.randn(1024, generator=g) * 0.05).numpy().astype(np.float32)
    return w


def decoder_weights(seed: int, layers: int = 2, std: float = 0.05):
    """Decoder / joint tensors (src/weights.rs:526-550, :633-644)."""
    g = _gen(seed * 1000 + 950)
    w = {"layers": layers, "embedding": _normal(g, (1025, 640), 0.2),
         "w_pred": _normal(g, (640, 640), std), "b_pred": (torch.randn(640, generator=g) * std).numpy(),
         "w_joint": _normal(g, (1030, 640), std), "b_joint": (torch.randn(1030, generator=g) * std).numpy(),
         "w_enc": _normal(g, (640, 1024), std), "b_enc": (torch.randn(640, generator=g) * std).numpy()}
    for l in range(layers):
        w[f"w_ih{l}"] = _normal(g, (2560, 640), std)
        w[f"w_hh{l}"] = _normal(g, (2560, 640), std)
        w[f"b_ih{l}"] = (torch.randn(2560, generator=g) * std).numpy()
        w[f"b_hh{l}"] = (torch.randn(2560, generator=g) * std).numpy()
    return {k: (v.astype(np.float32) if isinstance(v, np.ndarray) else v) for k, v in w.items()}
