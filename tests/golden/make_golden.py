"""Generates tests/golden/reference_kernels.npz: outputs of the REFERENCE'S OWN KERNELS
(oracle/_ref/*.cubin, compiled from the reference checkout by oracle/build_ref.py) on small
seeded inputs, run on a B200.  The inputs are not stored: tests/test_golden.py regenerates them
from the same seeds through `cases()` below.  Usage, on a machine with a GPU and the cubins:

    python tests/golden/make_golden.py <output.npz>
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from oracle import codec, decoder as D, frontend as F, ops as O   # noqa: E402


def cases():
    """Seeded inputs of every golden case (shared by the generator and the test)."""
    c = {}
    rng = np.random.default_rng(100)
    rows, padded = 15, 16
    c["ln"] = dict(x=codec.f16_round(rng.standard_normal((padded, 1024)) * 2),
                   g=codec.f16_round(1 + 0.1 * rng.standard_normal(1024)),
                   b=codec.f16_round(0.1 * rng.standard_normal(1024)), rows=rows, padded=padded)
    rng = np.random.default_rng(101)
    x = codec.f16_round(rng.standard_normal((128, 1024)))
    w = codec.f16_round(rng.standard_normal((4096, 1024)) * 0.02)
    wq, ws = codec.quantize_rows_fp8(w)
    c["ffn"] = dict(xq=codec.quantize_fp8_fixed(x, 56.0), wq=wq, ws=ws, rows=128)
    rng = np.random.default_rng(102)
    c["glu"] = dict(e=codec.f16_round(rng.standard_normal((24, 2048)) * 2), rows=22, padded=24, valid=21)
    c["dw"] = dict(wdw=codec.f16_round(rng.standard_normal((1024, 9)) * 0.3),
                   bn=[(1 + 0.1 * rng.standard_normal(1024)).astype(np.float32),
                       (0.1 * rng.standard_normal(1024)).astype(np.float32),
                       (0.1 * rng.standard_normal(1024)).astype(np.float32),
                       (1 + 0.2 * rng.random(1024)).astype(np.float32)])
    rng = np.random.default_rng(103)
    rows, padded, valid = 40, 40, 37
    q, k, v = [codec.f16_round(rng.standard_normal((padded, 1024))) for _ in range(3)]
    wpos = codec.f16_round(rng.standard_normal((1024, 1024)) * 0.02)
    c["att"] = dict(q=q, k=k, v=v, pos=O.position_table(wpos), u=codec.f16_round(rng.standard_normal((8, 128)) * 0.02),
                    bv=codec.f16_round(rng.standard_normal((8, 128)) * 0.02), rows=rows, padded=padded, valid=valid)
    rng = np.random.default_rng(104)
    c["dec"] = dict(w=D.make_decoder_weights(17, layers=2), enc=codec.f16_round(rng.standard_normal((60, 640)) * 0.5),
                    frames=60)
    rng = np.random.default_rng(106)
    # a request long enough (>= 1024 frames) for the reference to pick its INT8-cache kernel
    c["dec_long"] = dict(w=c["dec"]["w"], enc=codec.f16_round(rng.standard_normal((1024, 640)) * 0.5), frames=1024)
    # the same kernel on 16 short independent requests (the kernel itself has no length limit; only
    # the host's choice depends on the frame count): many decisions before the first near-tie of each
    rng = np.random.default_rng(107)
    c["dec_long_short"] = dict(w=c["dec"]["w"], frames=48,
                               enc=[codec.f16_round(rng.standard_normal((48, 640)) * 0.5) for _ in range(16)])
    # three more requests through the long-request kernel, other weights and lengths (the arithmetic
    # of this kernel feeds every rounding back through 8-bit codes: each extra request pins it further)
    c["dec_long_more"] = []
    for seed, wseed, nframes in ((8, 33, 128), (21, 33, 200), (23, 45, 256)):
        rng = np.random.default_rng(seed)
        c["dec_long_more"].append(dict(w=D.make_decoder_weights(wseed, layers=2), frames=nframes,
                                       enc=codec.f16_round(rng.standard_normal((nframes, 640)) * 0.5)))
    rng = np.random.default_rng(105)
    c["fe"] = dict(x=(rng.standard_normal(1700) * 0.3).astype(np.float32))
    # per-tensor activation x per-row weight scaled linears and their quantisers (linear.cu:325-429, :537-560)
    rng = np.random.default_rng(108)
    m, n, k = 16, 64, 256
    x = codec.f16_round(rng.standard_normal((m, k)))
    w = codec.f16_round(rng.standard_normal((n, k)) * 0.02)
    c["lin"] = dict(x=x, w=w, bias=(0.1 * rng.standard_normal(n)).astype(np.float32), m=m, n=n, k=k,
                    inv8=float(np.float32(127.0) / np.float32(np.max(np.abs(x)))))
    # LayerNorm pair / LayerNorm + per-row dynamic E4M3 (encoder.cu:128-306)
    rng = np.random.default_rng(109)
    c["lnpair"] = dict(x=codec.f16_round(rng.standard_normal((16, 1024)) * 2),
                       g=[codec.f16_round(1 + 0.1 * rng.standard_normal(1024)) for _ in range(2)],
                       b=[codec.f16_round(0.1 * rng.standard_normal(1024)) for _ in range(2)], rows=15, padded=16)
    # convolution subsampling of a 40-frame request (subsampling.cu, one tile); weights: seeded like
    # the product's synthetic pre-encode tensors, restated here so the case stands alone
    rng = np.random.default_rng(110)
    sw = {"conv0_w": codec.f16_round(rng.standard_normal((256, 9)) * 0.3),
          "conv0_b": codec.f16_round(rng.standard_normal(256) * 0.1)}
    for stage in (1, 2):
        sw[f"dw{stage}_w"] = codec.f16_round(rng.standard_normal((256, 9)) * 0.3)
        sw[f"dw{stage}_b"] = codec.f16_round(rng.standard_normal(256) * 0.1)
        sw[f"pw{stage}_w"] = codec.f16_round(rng.standard_normal((256, 256)) * 0.06)
        sw[f"pw{stage}_b"] = (rng.standard_normal(256) * 0.05).astype(np.float32)
    sw["proj_w"] = codec.f16_round(rng.standard_normal((1024, 4096)) * 0.02)
    sw["proj_b"] = (rng.standard_normal(1024) * 0.05).astype(np.float32)
    c["sub"] = dict(w=sw, mel=rng.standard_normal((40, 128)).astype(np.float32), frames=40)
    rng = np.random.default_rng(124)
    h = codec.quantize_fp8_fixed(codec.f16_round(np.maximum(rng.standard_normal((40, 4096)), -0.2)), 16.0)
    h[3, 8:12] = 0x30                                  # equal magnitudes: ties go to the lower index
    c["sparse24"] = dict(h=h, w=codec.f16_round(rng.standard_normal((1024, 4096)) * 0.02),
                         x=codec.f16_round(rng.standard_normal((40, 1024))), rows=40)
    return c


def main(out_path):
    import torch
    from oracle import refkernels as R
    from tests.util import dev, dev16, host
    c = cases()
    g = {}
    ln = c["ln"]
    ref = R.layer_norm(dev16(ln["x"]), dev16(ln["g"]), dev16(ln["b"]), ln["rows"], ln["padded"])
    g["ln"] = host(ref).astype(np.float16)
    g["ln_q"] = host(R.quantize_fp8_fixed(ref, 56.0))
    f = c["ffn"]
    g["ffn"] = host(R.ffn_expand_fp8(dev(f["xq"]), dev(f["wq"]), dev(f["ws"]), f["rows"]))[:, ::16].astype(np.float16)
    gl = c["glu"]
    glu = R.glu_masked(dev16(gl["e"]), gl["rows"], gl["padded"], gl["valid"])
    g["glu"] = host(glu).astype(np.float16)
    dw = c["dw"]
    g["dw"] = host(R.depthwise_bn_silu(glu, dev16(dw["wdw"]), *[dev(t) for t in dw["bn"]], gl["rows"],
                                       gl["padded"])).astype(np.float16)
    a = c["att"]
    g["att"] = host(R.local_attention_scalar(dev16(a["q"]), dev16(a["k"]), dev16(a["v"]), dev16(a["pos"]), dev16(a["u"]),
                                             dev16(a["bv"]), a["rows"], a["padded"], a["valid"])).astype(np.float16)
    d = c["dec"]
    dwts = {k: (dev(v) if k.startswith("b_") else dev16(v)) for k, v in d["w"].items() if k != "layers"}
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    g["dec_tokens"] = R.tdt_decode(dev16(d["enc"]), dwts, d["frames"], sms).astype(np.int32)
    dl = c["dec_long"]
    g["dec_long_tokens"] = R.tdt_decode_long(dev16(dl["enc"]), dwts, dl["frames"]).astype(np.int32)
    dls = c["dec_long_short"]
    for i, enc in enumerate(dls["enc"]):
        g[f"dec_long_short_{i}"] = R.tdt_decode_long(dev16(enc), dwts, dls["frames"]).astype(np.int32)
    for i, m in enumerate(c["dec_long_more"]):
        mw = {k: (dev(v) if k.startswith("b_") else dev16(v)) for k, v in m["w"].items() if k != "layers"}
        g[f"dec_long_more_{i}"] = R.tdt_decode_long(dev16(m["enc"]), mw, m["frames"]).astype(np.int32)
    # the same request through the short-request kernel, to show that the two kernels differ
    g["dec_long_tokens_fp16"] = R.tdt_decode(dev16(dl["enc"]), dwts, dl["frames"], sms).astype(np.int32)
    x = c["fe"]["x"]
    frames, valid = F.frame_counts(x.size)
    w512 = F.center_window(F.hann_window())
    fr = R.frame_window(dev(x), dev(w512), frames)
    g["fe_frames"] = host(fr)
    offsets, bins, values = F.sparse_filters(F.triangular_filters())
    spec = np.fft.rfft(host(fr).astype(np.float64), axis=1)
    spec2 = np.stack([spec.real, spec.imag], axis=-1).astype(np.float32)
    mel = R.mel_log_sparse(dev(spec2), dev(offsets), dev(bins), dev(values), frames, float(F.LOG_ZERO_GUARD))
    g["fe_mel"] = host(mel)
    g["fe_norm"] = host(R.normalize_mel(mel, frames, valid, float(F.NORMALIZE_EPSILON)))
    li = c["lin"]
    q8 = R.quantize_int8(dev16(li["x"]), li["inv8"])
    qf = R.quantize_fp8(dev16(li["x"]), 56.0)
    g["lin_q8"], g["lin_qf"] = host(q8), host(qf)
    w8, w8s = codec.quantize_rows_int8(li["w"])
    wf, wfs = codec.quantize_rows_fp8(li["w"])
    for act in (0, 1, 2):
        g[f"lin_int8_act{act}"] = host(R.int8_linear(q8, dev(w8), dev(w8s), dev(li["bias"]), li["m"], li["n"], li["k"],
                                                     1.0 / li["inv8"], act)).astype(np.float16)
    g["lin_fp8"] = host(R.fp8_linear(qf, dev(wf), dev(wfs), dev(li["bias"]), li["m"], li["n"], li["k"],
                                     8.0 / 448.0, 0)).astype(np.float16)
    lp = c["lnpair"]
    args = [dev16(lp["x"]), dev16(lp["g"][0]), dev16(lp["b"][0]), dev16(lp["g"][1]), dev16(lp["b"][1]),
            lp["rows"], lp["padded"]]
    first, second = R.layer_norm_pair(*args, 0.0)
    g["lnpair_first"], g["lnpair_second"] = host(first).astype(np.float16), host(second).astype(np.float16)
    g["lnpair_second_q"] = host(R.layer_norm_pair(*args, 56.0)[1])
    dq, ds = R.layer_norm_quantize_fp8_dynamic(dev16(lp["x"]), dev16(lp["g"][0]), dev16(lp["b"][0]), lp["rows"], lp["padded"])
    g["lndyn_q"], g["lndyn_s"] = host(dq), host(ds)
    sb = c["sub"]
    sdev = {k: (dev(v) if k in ("pw1_b", "pw2_b", "proj_b") else dev16(v)) for k, v in sb["w"].items()}
    stages, out = R.subsampling(dev(sb["mel"]), sdev, sb["frames"])
    g["sub_conv0"] = host(stages["conv0"]).astype(np.float16)[::7]        # every 7th (frame, feature) row
    g["sub_out"] = host(out).astype(np.float16)
    np.savez_compressed(out_path, **g)
    print("wrote", out_path, {k: v.shape for k, v in g.items()})


def main_sparse24(out_path):
    """Second fixture file (reference_sparse24.npz): pk_sm89_ffn_contract_fp8_sparse (`mma.sp` on the 2:4
    arena written by the oracle's compressor) and pk_sm89_ffn_contract_fp8 on the pruned dense bytes."""
    from oracle import refkernels as R
    from tests.util import dev, dev16, host
    c = cases()["sparse24"]
    wq, ws = codec.quantize_rows_fp8(c["w"])
    flat, pruned = codec.compress_2of4_e4m3(c["h"]), codec.prune_2of4_e4m3(c["h"])
    g = {"sparse": host(R.ffn_contract_fp8(dev(flat), dev(wq), dev(ws), dev16(c["x"]), c["rows"], sparse=True)).astype(np.float16),
         "dense_pruned": host(R.ffn_contract_fp8(dev(pruned), dev(wq), dev(ws), dev16(c["x"]), c["rows"])).astype(np.float16),
         "dense_full": host(R.ffn_contract_fp8(dev(c["h"]), dev(wq), dev(ws), dev16(c["x"]), c["rows"])).astype(np.float16)}
    np.savez_compressed(out_path, **g)
    print("wrote", out_path, {k: v.shape for k, v in g.items()})


if __name__ == "__main__":
    if sys.argv[1] == "sparse24":
        main_sparse24(sys.argv[2])
    else:
        main(sys.argv[1])
