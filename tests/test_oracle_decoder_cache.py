"""CPU checks of the oracle's restatement of the reference's long-request decoder numerics
(kernels/sm89/decoder.cu:86-120, :452-784): INT8 cache codes, lane partition, reduction order."""
import numpy as np

from oracle import decoder as D

F32 = np.float32


def test_quantize_i8_known_answers():
    # round to nearest even, clamp to +-127 (the rule of src/bin/quant_benchmark.rs:968-974)
    assert list(D.quantize_i8(np.array([0.5, 1.5, 2.5, -0.5, -1.5, 200.0, -200.0, 126.5, 127.4]))) == \
        [0, 2, 2, 0, -2, 127, -127, 126, 127]


def test_cache_scale_and_codes():
    w = np.array([[0.5, -1.0, 0.25], [0.0, 0.124, -0.126]], dtype=F32)
    s = D.cache_scale(w)
    assert s == F32(F32(1.0) / F32(127.0))
    codes = D.cache_codes(w, s)
    assert codes.tolist() == [[64, -127, 32], [0, 16, -16]]       # 63.5 -> 64 (even), 31.75 -> 32
    assert D.cache_scale(np.zeros((2, 2), F32)) == F32(1.0)       # all-zero tensor: scale 1


def test_lane_partition_matches_a_scalar_walk():
    """Lane l owns elements 4*l + 128*step .. +3 (decoder.cu:86-89, :107-113)."""
    rng = np.random.default_rng(3)
    codes = rng.integers(-127, 128, size=(3, 640))
    hq = rng.integers(-127, 128, size=640)
    scale = F32(0.004)
    got = D._lane_partials(codes, hq, scale)
    for row in range(3):
        for lane in (0, 7, 31):
            dot = 0
            for step in range(5):
                for k in range(4):
                    i = 4 * lane + 128 * step + k
                    dot += int(codes[row, i]) * int(hq[i])
            assert got[row, lane] == F32(F32(dot) * F32(scale / F32(127.0)))
    assert got.shape == (3, 32)


def test_warp_sum_is_the_shfl_down_tree():
    v = (np.arange(32, dtype=F32) * F32(0.1) + F32(1e-3)).reshape(1, 32)
    want = v[0].copy()
    for width in (16, 8, 4, 2, 1):
        for lane in range(width):
            want[lane] = F32(want[lane] + want[lane + width])
    assert D._warp_sum(v)[0] == want[0]


def test_input_table_is_an_fp16_linear_without_bias():
    w = D.make_decoder_weights(3, layers=1)
    t = D.input_table(w)
    assert t.shape == (1024, 2560)
    ref = (w["embedding"][5].astype(np.float64) @ w["w_ih0"].astype(np.float64).T)
    assert np.array_equal(t[5], ref.astype(F32).astype(np.float16).astype(F32))


def test_long_request_rule_and_divergence():
    """"auto" follows the frame rule (src/cuda/decoder.rs:15, :88) and the two kernels are different
    functions of the same input."""
    w = D.make_decoder_weights(17, layers=2)
    rng = np.random.default_rng(2)
    enc = (rng.standard_normal((40, 640)) * 0.5).astype(np.float16).astype(F32)
    short = D.tdt_greedy(enc, w, 40, lstm_cache="auto")
    assert np.array_equal(short[0], D.tdt_greedy(enc, w, 40, lstm_cache="fp16")[0])
    assert D.LONG_REQUEST_FRAMES == 1024
    cache = D.Int8LstmCache(w)
    h = (rng.standard_normal((2, 640)) * 0.3).astype(F32)
    c = (rng.standard_normal((2, 640)) * 0.3).astype(F32)
    ch, cc = cache.step(7, True, h, c)
    x = w["embedding"][7]
    fh0, _ = D.lstm_step(x, h[0], c[0], w["w_ih0"], w["w_hh0"], w["b_ih0"], w["b_hh0"])
    err = np.max(np.abs(ch[0] - fh0))
    assert 1e-6 < err < 5e-2          # quantisation noise: different, but close
