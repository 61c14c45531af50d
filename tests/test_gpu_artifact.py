"""A model loaded from a ".pkl4" artifact through the C reader runs exactly like the same
tensors handed over directly (encoder block, subsampling, decoder)."""
import numpy as np
import pytest
import torch

from oracle import artifact as A
from oracle import codec
from tests.util import dev16, host

pytestmark = pytest.mark.gpu

VOCAB = [f"p{i}" for i in range(1024)]


def _checkpoint(rng):
    m = A.manifest("v2_english", encoder_layers=1)
    t = {}
    for name, (_, shape) in m.items():
        if name.endswith("running_var"):
            t[name] = (1.0 + 0.2 * rng.random(shape)).astype(np.float32)
        elif ".norm" in name and name.endswith(".weight"):
            t[name] = (1.0 + 0.1 * rng.standard_normal(shape)).astype(np.float32)
        elif "depthwise" in name or name.startswith("encoder.subsampling.layers.") and "weight" in name and shape[1:2] == (1,):
            t[name] = (rng.standard_normal(shape) * 0.3).astype(np.float32)
        elif name == "decoder.embedding.weight":
            t[name] = (rng.standard_normal(shape) * 0.2).astype(np.float32)
        else:
            t[name] = (rng.standard_normal(shape) * (0.05 if name.startswith(("decoder", "joint", "encoder_projector")) else 0.02)
                       ).astype(np.float32)
    return t


def test_model_from_artifact_runs_like_direct_weights(pk, cuda, tmp_path):
    rng = np.random.default_rng(7)
    tensors = _checkpoint(rng)
    path = tmp_path / "one_block.pkl4"
    A.write(path, tensors, "v2_english", VOCAB)
    art = pk.artifact.Artifact(path)
    _, views = A.read(path)                                   # the oracle's view of the same file
    f32 = lambda name, shape=None: np.asarray(views[name], np.float32).reshape(shape or views[name].shape)

    # ---- encoder block
    p = "encoder.layers.0"
    direct = {"ff1_w1": f32(f"{p}.feed_forward1.linear1.weight"), "ff1_w2": f32(f"{p}.feed_forward1.linear2.weight"),
              "ff2_w1": f32(f"{p}.feed_forward2.linear1.weight"), "ff2_w2": f32(f"{p}.feed_forward2.linear2.weight"),
              "wq": f32(f"{p}.self_attn.q_proj.weight"), "wk": f32(f"{p}.self_attn.k_proj.weight"),
              "wv": f32(f"{p}.self_attn.v_proj.weight"), "wo": f32(f"{p}.self_attn.o_proj.weight"),
              "wpos": f32(f"{p}.self_attn.relative_k_proj.weight"),
              "wpw1": f32(f"{p}.conv.pointwise_conv1.weight", (2048, 1024)),
              "wpw2": f32(f"{p}.conv.pointwise_conv2.weight", (1024, 1024)),
              "bias_u": f32(f"{p}.self_attn.bias_u"), "bias_v": f32(f"{p}.self_attn.bias_v"),
              "dw": f32(f"{p}.conv.depthwise_conv.weight", (1024, 9)),
              "bn_g": f32(f"{p}.conv.norm.weight"), "bn_b": f32(f"{p}.conv.norm.bias"),
              "bn_m": f32(f"{p}.conv.norm.running_mean"), "bn_v": f32(f"{p}.conv.norm.running_var")}
    for ours, norm in (("ff1", "norm_feed_forward1"), ("att", "norm_self_att"), ("conv", "norm_conv"),
                       ("ff2", "norm_feed_forward2"), ("out", "norm_out")):
        direct[f"ln_{ours}_g"], direct[f"ln_{ours}_b"] = f32(f"{p}.{norm}.weight"), f32(f"{p}.{norm}.bias")
    rows, valid = 256, 250
    x = codec.f16_round(rng.standard_normal((rows, 1024)))
    x[valid:] = 0
    outs = []
    for w in (art.layer_weights(0), direct):
        enc = pk.encoder.EncoderLayers(cuda)
        enc.add_layer(w, 0.5, 0.5)
        arena, ws = enc.make_workspace(rows)
        a, b = dev16(x), torch.zeros((rows, 1024), dtype=torch.float16, device=cuda)
        out = enc.run(a, b, ws, 1, rows, valid)
        torch.cuda.synchronize()
        assert enc.status(arena, ws) == 0
        outs.append(host(out).copy())
    assert np.array_equal(outs[0], outs[1]) and np.abs(outs[0]).max() > 0.1

    # ---- subsampling
    s = "encoder.subsampling"
    direct_sub = {"conv0_w": f32(f"{s}.layers.0.weight", (256, 9)), "conv0_b": f32(f"{s}.layers.0.bias"),
                  "dw1_w": f32(f"{s}.layers.2.weight", (256, 9)), "dw1_b": f32(f"{s}.layers.2.bias"),
                  "pw1_w": f32(f"{s}.layers.3.weight", (256, 256)), "pw1_b": f32(f"{s}.layers.3.bias"),
                  "dw2_w": f32(f"{s}.layers.5.weight", (256, 9)), "dw2_b": f32(f"{s}.layers.5.bias"),
                  "pw2_w": f32(f"{s}.layers.6.weight", (256, 256)), "pw2_b": f32(f"{s}.layers.6.bias"),
                  "proj_w": f32(f"{s}.linear.weight"), "proj_b": f32(f"{s}.linear.bias")}
    mel = torch.from_numpy(rng.standard_normal((1, 400, 128)).astype(np.float32)).to(cuda)
    subs = [host(pk.subsampling.Subsampling(w, cuda).run(mel, 128)).copy() for w in (art.subsampling_weights(), direct_sub)]
    torch.cuda.synchronize()
    assert np.array_equal(subs[0][:50], subs[1][:50]) and np.abs(subs[0][:50]).max() > 0

    # ---- decoder (one and two LSTM layers)
    enc_proj = dev16(codec.f16_round(rng.standard_normal((64, 640)) * 0.5))
    fr = torch.tensor([64], dtype=torch.int32, device=cuda)
    for layers in (1, 2):
        direct_dec = {"layers": layers, "embedding": f32("decoder.embedding.weight"),
                      "w_pred": f32("decoder.decoder_projector.weight"), "b_pred": f32("decoder.decoder_projector.bias"),
                      "w_joint": f32("joint.head.weight"), "b_joint": f32("joint.head.bias"),
                      "w_enc": f32("encoder_projector.weight"), "b_enc": f32("encoder_projector.bias")}
        for l in range(layers):
            for kind in ("ih", "hh"):
                direct_dec[f"w_{kind}{l}"] = f32(f"decoder.lstm.weight_{kind}_l{l}")
                direct_dec[f"b_{kind}{l}"] = f32(f"decoder.lstm.bias_{kind}_l{l}")
        got = []
        for w in (art.decoder_weights(layers), direct_dec):
            dec = pk.decoder.TdtDecoder(w, cuda)
            t, d, c = dec.decode(enc_proj, 1, 64, fr, 640)
            torch.cuda.synchronize()
            assert int(dec.status.item()) == 0
            got.append((host(t)[0, :int(host(c)[0])].copy(), int(host(c)[0])))
        assert got[0][1] == got[1][1] and got[0][1] > 5 and np.array_equal(got[0][0], got[1][0])
    art.close()
