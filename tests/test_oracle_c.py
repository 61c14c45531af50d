"""The C restatement of the codecs agrees with the numpy oracle (CPU only)."""
import ctypes as C

import numpy as np
import pytest

from oracle import build_ref, codec


@pytest.fixture(scope="module")
def clib():
    return C.CDLL(str(build_ref.build_c_oracle()))


def test_e4m3_c_matches_numpy(clib):
    rng = np.random.default_rng(0)
    x = np.concatenate([
        (rng.standard_normal(100000) * rng.choice([1e-3, 0.05, 1, 30, 300], 100000)),
        codec.E4M3_DECODE[:127], -codec.E4M3_DECODE[:127],
        (codec.E4M3_DECODE[:126] + codec.E4M3_DECODE[1:127]) / 2,      # every tie point
        [0.0, -0.0, 448.0, 449.0, 1e30, -1e30, 2.0 ** -10, 2.0 ** -11],
    ]).astype(np.float32)
    out = np.zeros(x.size, np.uint8)
    clib.pk_e4m3_encode(x.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p), C.c_long(x.size))
    assert np.array_equal(out, codec.e4m3_encode(x))
    back = np.zeros(256, np.float32)
    codes = np.arange(256, dtype=np.uint8)
    clib.pk_e4m3_decode(codes.ctypes.data_as(C.c_void_p), back.ctypes.data_as(C.c_void_p), C.c_long(256))
    assert np.array_equal(np.nan_to_num(back, nan=-1), np.nan_to_num(codec.e4m3_decode(codes), nan=-1))


def test_int8_c_matches_numpy(clib):
    rng = np.random.default_rng(1)
    x = (rng.standard_normal(50000) * 3).astype(np.float32)
    out = np.zeros(x.size, np.int8)
    clib.pk_quantize_int8(x.ctypes.data_as(C.c_void_p), C.c_float(32.0), out.ctypes.data_as(C.c_void_p),
                          C.c_long(x.size))
    assert np.array_equal(out, codec.quantize_int8(x, 32.0))


def test_decision_key_orders_like_better(clib):
    # kernels/sm89/decoder.cu:35-46: higher score wins, equal scores -> lower id, -0 == +0
    clib.pk_decision_key.restype = C.c_uint64
    key = lambda s, i: clib.pk_decision_key(C.c_float(s), C.c_int(i))
    assert key(1.0, 5) > key(0.5, 1)
    assert key(1.0, 3) > key(1.0, 4)
    assert key(-1.0, 3) < key(-0.5, 900)
    assert key(0.0, 7) == key(-0.0, 7)
    assert key(-3.4e38, 1025) < key(-1e30, 1024)


def test_gemm_s8_c_matches_numpy(clib):
    rng = np.random.default_rng(2)
    a = rng.integers(-127, 128, (9, 256), dtype=np.int8)
    b = rng.integers(-127, 128, (12, 256), dtype=np.int8)
    acc = np.zeros((9, 12), np.int32)
    clib.pk_gemm_s8(a.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p),
                    acc.ctypes.data_as(C.c_void_p), 9, 12, 256)
    assert np.array_equal(acc, a.astype(np.int32) @ b.astype(np.int32).T)
