"""Pins the CPU oracle's codecs to the reference's own known-answer tests."""
import numpy as np
import pytest

from oracle import codec


def test_e4m3_reference_examples():
    # src/cuda/quant_benchmark.rs:961-966
    assert codec.e4m3_encode(np.float32(1.0)) == 0x38
    assert codec.e4m3_encode(np.float32(-1.0)) == 0xB8
    assert codec.e4m3_encode(np.float32(448.0)) == 0x7E


def test_e4m3_saturates_and_rounds_to_even():
    enc = codec.e4m3_encode
    assert enc(np.float32(1e9)) == 0x7E and enc(np.float32(-1e9)) == 0xFE
    assert enc(np.float32(464.0)) == 0x7E and enc(np.float32(480.0)) == 0x7E
    assert enc(np.float32(0.0)) == 0x00 and enc(np.float32(-0.0)) == 0x80
    # 1.0 = 0x38, 1.125 = 0x39: the midpoint 1.0625 ties to the even code 0x38,
    # 1.1875 (between 0x39 and 0x3a) ties to 0x3a
    assert enc(np.float32(1.0625)) == 0x38
    assert enc(np.float32(1.1875)) == 0x3A
    # smallest subnormal 2^-9; half of it ties to zero (even)
    assert enc(np.float32(2.0 ** -9)) == 0x01
    assert enc(np.float32(2.0 ** -10)) == 0x00
    assert enc(np.float32(2.0 ** -10 * 1.01)) == 0x01


def test_e4m3_roundtrip_all_codes():
    codes = np.array([c for c in range(256) if (c & 0x7F) != 0x7F], dtype=np.uint8)
    assert np.array_equal(codec.e4m3_encode(codec.e4m3_decode(codes)), codes)


def test_e4m3_matches_torch_cast_below_saturation():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(0)
    x = (rng.standard_normal(200000) * rng.choice([1e-3, 0.1, 1, 30, 200], 200000)).astype(np.float32)
    x = np.clip(x, -448, 448)
    ref = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(codec.e4m3_encode(x), ref)


def test_int8_quantizer_is_symmetric_and_saturating():
    # src/cuda/quant_benchmark.rs:968-974
    q = lambda v: int(codec.quantize_int8(np.float32(v), 1.0))
    assert q(0.5) == 0 and q(1.5) == 2 and q(200.0) == 127 and q(-200.0) == -127


def test_generated_values_span_both_signs():
    # src/cuda/quant_benchmark.rs:976-984
    vals = [codec.pattern(i, 17, 1.0) for i in range(100)]
    assert any(v < 0 for v in vals) and any(v > 0 for v in vals)
    arr = codec.pattern_array(100, 17, 1.0)
    assert np.allclose(arr, np.array(vals, dtype=np.float32), rtol=0, atol=0)


def test_packing_known_answers():
    # src/packing.rs:168-199
    fp16 = codec.estimate_linear("fp16", 1024, 4096)
    fp8 = codec.estimate_linear("fp8_e4m3", 1024, 4096)
    assert fp16["payload_bytes"] + fp16["metadata_bytes"] == 8 * 1024 * 1024
    assert fp8["payload_bytes"] == 4 * 1024 * 1024 and fp8["metadata_bytes"] == 16 * 1024
    assert codec.estimate_linear("q4_k", 640, 8198) is None
    q4 = codec.estimate_linear("q4_k", 1024, 4096)
    assert q4["payload_bytes"] + q4["metadata_bytes"] == 4096 * 4 * 144
    j = codec.estimate_linear("fp8_e4m3", 640, 8198)
    assert (j["padded_in"], j["padded_out"]) == (640, 8320)
    with pytest.raises(ValueError):
        codec.estimate_linear("fp16", 0, 4)


def test_exl3_known_answers():
    # src/exl3.rs:82-95
    lay = codec.exl3_layout(4096, 1024, 4)
    assert lay["trellis_shape"] == [256, 64, 64]
    assert lay["trellis_bytes"] == 2 * 1024 * 1024 and lay["scale_bytes"] == 10 * 1024
    j = codec.exl3_layout(640, 8198, 4)
    assert j["padded_in"] == 640 and j["padded_out"] == 8320 and j["trellis_shape"] == [40, 520, 64]
    with pytest.raises(ValueError):
        codec.exl3_layout(16, 16, 9)


def test_align_up():
    # src/artifact.rs:766-769
    assert codec.align_up(257, 256) == 512
    with pytest.raises(OverflowError):
        codec.align_up((1 << 64) - 1, 256)


def test_f16_small_integers_exact():
    # src/artifact.rs:726-743 (values 1..6 survive the fp16 round trip)
    v = np.arange(1, 7, dtype=np.float32)
    assert np.array_equal(codec.f16_round(v), v)


def test_int4_row_pack_roundtrip_and_nibble_order():
    rng = np.random.default_rng(1)
    w = rng.standard_normal((8, 64)).astype(np.float32)
    packed, scale = codec.quantize_rows_int4(w)
    q = codec.unpack_nibbles(packed)
    assert q.min() >= -8 and q.max() <= 7
    assert packed[0, 0] == ((int(q[0, 0]) & 15) | ((int(q[0, 1]) & 15) << 4))
    assert np.array_equal(codec.pack_nibbles(q), packed)
    # the row maximum maps to code 7 or the row minimum to -8
    assert np.all((q.max(axis=1) == 7) | (q.min(axis=1) == -8))


def test_int4_g128_dequant_error_bound():
    rng = np.random.default_rng(2)
    w = codec.f16_round(rng.standard_normal((16, 256)) * 0.02)
    packed, scales = codec.quantize_int4_g128(w)
    assert packed.shape == (16, 128) and scales.shape == (2, 16) and scales.dtype == np.float16
    back = codec.dequant_int4_g128(packed, scales)
    step = scales.astype(np.float32).T.repeat(128, axis=1)
    assert np.all(np.abs(back - w) <= 0.5 * step * 1.01 + 1e-6)


def test_two_four_selection():
    # kernels/sm89/encoder.cu:685-704: two largest magnitudes, ties -> lower index
    kept, meta = codec.compress_fp8_quartet([0x38, 0xB8, 0x30, 0x40])
    assert list(kept) == [0x38, 0x40] and meta == (0 | (3 << 2))
    kept, meta = codec.compress_fp8_quartet([0x10, 0x10, 0x10, 0x10])
    assert list(kept) == [0x10, 0x10] and meta == (0 | (1 << 2))


def test_2of4_format_known_answers_and_round_trip():
    """kernels/sm89/encoder.cu:685-704 (selection), :1037-1054 (arena layout): the vectorised format
    functions agree with the scalar quartet rule, the arena has data then metadata, and
    decompress(compress(x)) == prune(x)."""
    rng = np.random.default_rng(3)
    d = rng.integers(0, 256, (7, 64), dtype=np.uint8)
    d[0, :4] = [0x10, 0x90, 0x10, 0x10]          # equal magnitudes (sign ignored): indices 0 and 1 stay
    d[1, :4] = [0x01, 0x7E, 0x00, 0xFE]          # 0x7E and 0xFE (magnitude 126) stay
    keep = codec.keep_2of4(d)
    assert keep[0, :4].tolist() == [True, True, False, False]
    assert keep[1, :4].tolist() == [False, True, False, True]
    assert np.all(keep.reshape(7, 16, 4).sum(axis=2) == 2)
    flat = codec.compress_2of4_e4m3(d)
    assert flat.size == 7 * 32 + 7 * 8
    for r in range(7):
        for q in range(16):
            kept, meta = codec.compress_fp8_quartet(d[r, 4 * q:4 * q + 4])
            assert flat[r * 32 + 2 * q:r * 32 + 2 * q + 2].tolist() == kept.tolist()
            byte = flat[7 * 32 + r * 8 + q // 2]
            assert ((byte >> (4 * (q % 2))) & 15) == meta
    pruned = codec.prune_2of4_e4m3(d)
    assert np.array_equal(codec.decompress_2of4_e4m3(flat, 7, 64), pruned)
    assert np.array_equal(pruned[keep], d[keep]) and not pruned[~keep].any()


def test_int4_row_quantiser_uses_every_code():
    """kernels/sm89/encoder.cu:266-290: scale = max(v/7, -v/8), so +7 and -8 are both reachable."""
    from oracle import ops as O
    y = np.zeros((3, 1024), np.float32)
    y[0, :4] = [7.0, -8.0, 3.5, -0.4]
    y[1, :3] = [-4.0, 1.0, 0.26]                   # scale 0.5: -8, 2, rne(0.52) = 1
    q, s = O.quant_rows_int4_dynamic(y, rows=2)
    assert s.tolist() == [1.0, 0.5, 1.0]
    assert q[0, :4].tolist() == [7, -8, 4, 0] and q[1, :3].tolist() == [-8, 2, 1]
    assert not q[2].any()
    packed = codec.pack_nibbles(q)
    assert packed[0, 0] == (7 | (8 << 4)) and np.array_equal(codec.unpack_nibbles(packed), q)
