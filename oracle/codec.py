"""CPU oracle -- number formats and packers (TEST INFRASTRUCTURE, not product code).

Bit-exact numpy restatement of the quantisers and packers the reference uses on
the encoder hot path.  Only tests, the smoke check and the CPU-baseline leg of
the benchmark may import this package; the product path never does.

Every function cites the reference file:line it restates.  The third-party
arithmetic the reference leans on is restated from its published definition:
  * `half` 2.7.1  `f16::from_f32`            -> IEEE binary16 round-to-nearest-even
  * `float8` 0.7.0 `F8E4M3::from_f32` and CUDA `__nv_fp8_e4m3(float)`
                                             -> OCP E4M3 (bias 7, no inf, NaN=0x7f),
                                                RNE, saturate-to-finite at +-448
Pinned by the reference's own known-answer tests (see tests/test_oracle_codec.py):
  src/cuda/quant_benchmark.rs:961-974, src/packing.rs:168-199, src/exl3.rs:82-95.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32

# ----------------------------------------------------------------------------
# FP16
# ----------------------------------------------------------------------------

def f16_round(x):
    """fp32 -> fp16 (RNE) -> fp32.  `__float2half_rn` / `f16::from_f32`
    (kernels/sm89/encoder.cu:123, src/artifact.rs:425)."""
    return np.asarray(x, dtype=F32).astype(np.float16).astype(F32)


# ----------------------------------------------------------------------------
# E4M3
# ----------------------------------------------------------------------------

def _e4m3_table() -> np.ndarray:
    """Decode table for the 256 E4M3 byte codes (OCP FP8: 1-4-3, bias 7)."""
    out = np.zeros(256, dtype=np.float64)
    for code in range(256):
        sign = -1.0 if code & 0x80 else 1.0
        exp = (code >> 3) & 0xF
        man = code & 0x7
        if exp == 0xF and man == 0x7:
            out[code] = np.nan
        elif exp == 0:
            out[code] = sign * (man / 8.0) * 2.0 ** (-6)
        else:
            out[code] = sign * (1.0 + man / 8.0) * 2.0 ** (exp - 7)
    return out


E4M3_DECODE = _e4m3_table()
_E4M3_POS = E4M3_DECODE[:127].copy()                      # 0x00..0x7e, ascending
_E4M3_MID = (_E4M3_POS[:-1] + _E4M3_POS[1:]) * 0.5          # 126 midpoints (exact in f64)
E4M3_MAX = 448.0


def e4m3_encode(x) -> np.ndarray:
    """fp32 -> E4M3 byte, RNE, saturate to +-448, NaN -> 0x7f|sign.

    Restates `__nv_fp8_e4m3(float).__x` (kernels/sm89/encoder.cu:557, :289, :204)
    and `F8E4M3::from_f32(..).to_bits()` (src/cuda/encoder.rs:410).
    """
    x = np.asarray(x, dtype=F32)
    ax = np.abs(x).astype(np.float64)
    idx = np.searchsorted(_E4M3_MID, ax, side="left")        # number of midpoints < |x|
    idx = np.minimum(idx, 126)
    tie = (idx < 126) & (ax == _E4M3_MID[np.minimum(idx, 125)])
    idx = idx + (tie & ((idx & 1) == 1))                     # ties -> even code
    idx = np.where(ax >= E4M3_MAX, 126, idx)                 # satfinite
    idx = np.where(np.isnan(ax), 127, idx)
    sign = np.signbit(x).astype(np.uint8) << 7
    return (idx.astype(np.uint8) | sign).astype(np.uint8)


def e4m3_decode(b) -> np.ndarray:
    return E4M3_DECODE[np.asarray(b, dtype=np.uint8)].astype(F32)


def quantize_fp8_fixed(x16, inverse_scale) -> np.ndarray:
    """`pk_sm89_quantize_fp8_fixed` (kernels/sm89/encoder.cu:549-559):
    byte = E4M3(f32(x) * inverse_scale), product rounded once to fp32."""
    return e4m3_encode(np.asarray(x16, dtype=F32) * F32(inverse_scale))


def quantize_rows_fp8(w) -> tuple[np.ndarray, np.ndarray]:
    """Per-row E4M3 weight packing: scale = absmax/448, byte = E4M3(v/scale).

    Host twin src/cuda/encoder.rs:385-411 (FP8 branch) and
    src/cuda/quant_benchmark.rs:779-801; device twin
    kernels/sm89/encoder.cu:1129-1148.  The device kernel guards absmax == 0
    with scale 1; the host does not (all-zero rows are avoided in tests).
    """
    w = np.asarray(w, dtype=F32)
    absmax = np.max(np.abs(w), axis=1)
    scale = np.where(absmax > 0, absmax / F32(448.0), F32(1.0)).astype(F32)
    q = e4m3_encode((w / scale[:, None]).astype(F32))
    return q, scale


# ----------------------------------------------------------------------------
# INT8
# ----------------------------------------------------------------------------

def rne(x) -> np.ndarray:
    """round-half-to-even, like `__float2int_rn` / `f32::round_ties_even`."""
    return np.rint(np.asarray(x, dtype=F32))


def quantize_int8(x, inverse_scale) -> np.ndarray:
    """`pk_sm89_quantize_int8` (kernels/sm89/linear.cu:549-560) and
    `quantize_i8` (src/cuda/quant_benchmark.rs:827-829):
    clamp(rne(x * inverse_scale), -127, 127)."""
    v = np.asarray(x, dtype=F32) * F32(inverse_scale)
    return np.clip(rne(v), -127, 127).astype(np.int8)


def quantize_rows_int8(w) -> tuple[np.ndarray, np.ndarray]:
    """Per-row INT8 weights: scale = absmax/127, q = clamp(rne(v/scale), +-127)
    (src/cuda/quant_benchmark.rs:803-825)."""
    w = np.asarray(w, dtype=F32)
    absmax = np.max(np.abs(w), axis=1)
    scale = np.where(absmax > 0, absmax / F32(127.0), F32(1.0)).astype(F32)
    q = np.clip(rne((w / scale[:, None]).astype(F32)), -127, 127).astype(np.int8)
    return q, scale


def quantize_rows_int8_dynamic(x) -> tuple[np.ndarray, np.ndarray]:
    """Per-row dynamic INT8 activations (same rule as the per-row weight
    quantiser above, applied to an activation row; zero rows get scale 1 like
    kernels/sm89/encoder.cu:275)."""
    return quantize_rows_int8(x)


# ----------------------------------------------------------------------------
# INT4
# ----------------------------------------------------------------------------

def pack_nibbles(q) -> np.ndarray:
    """Two signed 4-bit codes per byte, low nibble = even index
    (src/cuda/encoder.rs:399-407, kernels/sm89/encoder.cu:283-287)."""
    q = np.asarray(q).astype(np.int16)
    assert q.shape[-1] % 2 == 0
    lo = q[..., 0::2] & 15
    hi = q[..., 1::2] & 15
    return (lo | (hi << 4)).astype(np.uint8)


def unpack_nibbles(b) -> np.ndarray:
    b = np.asarray(b, dtype=np.uint8)
    lo = (b & 15).astype(np.int8)
    hi = (b >> 4).astype(np.int8)
    lo = np.where(lo >= 8, lo - 16, lo)
    hi = np.where(hi >= 8, hi - 16, hi)
    out = np.empty(b.shape[:-1] + (b.shape[-1] * 2,), dtype=np.int8)
    out[..., 0::2] = lo
    out[..., 1::2] = hi
    return out


def quantize_rows_int4(w) -> tuple[np.ndarray, np.ndarray]:
    """Per-row INT4: scale = max_k max(v/7, -v/8); q = clamp(rne(v/scale), -8, 7)
    (src/cuda/encoder.rs:385-407 INT4 branch; device twin
    kernels/sm89/encoder.cu:267-287, which maps scale 0 -> 1)."""
    w = np.asarray(w, dtype=F32)
    s = np.max(np.maximum(w / F32(7.0), -w / F32(8.0)), axis=1)
    s = np.maximum(s, F32(0.0))
    scale = np.where(s > 0, s, F32(1.0)).astype(F32)
    q = np.clip(rne((w / scale[:, None]).astype(F32)), -8, 7).astype(np.int8)
    return pack_nibbles(q), scale


GROUP = 128


def quantize_int4_g128(w) -> tuple[np.ndarray, np.ndarray]:
    """Symmetric INT4 with one fp16 scale per 128 consecutive K per output row.

    No counterpart in the reference (its only INT4 quantiser is per row); defined
    from the benchmark text: codes in [-7, 7], scale = f16(absmax_group / 7)
    (zero group -> scale 1), q = clamp(rne(v / f32(scale)), -7, 7).  Returns
    packed codes [N, K/2] (low nibble = even k) and scales [K/128, N] fp16.
    """
    w = np.asarray(w, dtype=F32)
    n, k = w.shape
    assert k % GROUP == 0
    g = w.reshape(n, k // GROUP, GROUP)
    absmax = np.max(np.abs(g), axis=2)
    scale16 = np.where(absmax > 0, absmax / F32(7.0), F32(1.0)).astype(np.float16)
    scale = scale16.astype(F32)
    scale = np.where(scale > 0, scale, F32(1.0))
    scale16 = scale.astype(np.float16)
    q = np.clip(rne((g / scale[:, :, None]).astype(F32)), -7, 7).astype(np.int8)
    return pack_nibbles(q.reshape(n, k)), np.ascontiguousarray(scale16.T)


def dequant_int4_g128(packed, scales16) -> np.ndarray:
    """W16[n,k] = f16(code[n,k] * f32(scale[k/128, n])) -- the operand the
    tensor core sees after the in-shared-memory dequantisation."""
    q = unpack_nibbles(packed).astype(F32)                    # [N, K]
    n, k = q.shape
    s = np.asarray(scales16, dtype=np.float16).astype(F32).T  # [N, K/128]
    w = q.reshape(n, k // GROUP, GROUP) * s[:, :, None]
    return f16_round(w.reshape(n, k))


# ----------------------------------------------------------------------------
# 2:4 selection (reference FF2 sparsity; kept as a known-answer helper)
# ----------------------------------------------------------------------------

def compress_fp8_quartet(b4) -> tuple[np.ndarray, int]:
    """`compress_fp8_quartet` (kernels/sm89/encoder.cu:685-704): of four E4M3
    bytes keep the two largest 7-bit magnitudes, ties -> lower index; returns
    kept bytes in index order and 4 metadata bits (two 2-bit indices, low first)."""
    b4 = [int(v) for v in b4]
    kept, meta, count = [], 0, 0
    for i in range(4):
        mag = b4[i] & 127
        rank = sum(1 for j in range(4)
                   if (b4[j] & 127) > mag or ((b4[j] & 127) == mag and j < i))
        if rank < 2:
            kept.append(b4[i])
            meta |= i << (2 * count)
            count += 1
    return np.array(kept, dtype=np.uint8), meta


def keep_2of4(dense) -> np.ndarray:
    """Boolean mask [rows, cols] of the bytes the 2:4 rule keeps: per 4 consecutive columns the
    two largest 7-bit magnitudes, ties -> lower index (kernels/sm89/encoder.cu:685-704)."""
    dense = np.asarray(dense, dtype=np.uint8)
    rows, cols = dense.shape
    mag = (dense & 127).astype(np.int32).reshape(rows, cols // 4, 4)
    idx = np.arange(4)
    # rank[i] = #{j : mag[j] > mag[i] or (mag[j] == mag[i] and j < i)}
    greater = mag[:, :, None, :] > mag[:, :, :, None]
    tie_lower = (mag[:, :, None, :] == mag[:, :, :, None]) & (idx[None, None, None, :] < idx[None, None, :, None])
    rank = (greater | tie_lower).sum(axis=3)
    return (rank < 2).reshape(rows, cols)


def prune_2of4_e4m3(dense) -> np.ndarray:
    """E4M3 bytes [rows, cols] with the two smaller magnitudes of every quartet set to +0: the
    values the reference's 2:4-sparse contraction multiplies (`mma.sp`, encoder.cu:706-713)."""
    dense = np.asarray(dense, dtype=np.uint8)
    return np.where(keep_2of4(dense), dense, np.uint8(0)).astype(np.uint8)


def compress_2of4_e4m3(dense) -> np.ndarray:
    """The reference's compressed activation arena (encoder.cu:1037-1054; consumer :740-764) as one
    flat byte array: data `bytes[row * cols/2 + col/2]` (the two kept bytes of a quartet, in index
    order) followed by metadata `bytes[rows * cols/2 + row * cols/8 + col/8]` (4 bits per quartet:
    two 2-bit indices, low first; two quartets per byte, low nibble first)."""
    dense = np.asarray(dense, dtype=np.uint8)
    rows, cols = dense.shape
    keep = keep_2of4(dense).reshape(rows, cols // 4, 4)
    quart = dense.reshape(rows, cols // 4, 4)
    order = np.argsort(~keep, axis=2, kind="stable")[:, :, :2]          # indices of the kept two, ascending
    data = np.take_along_axis(quart, order, axis=2).reshape(rows, cols // 2)
    meta4 = (order[:, :, 0] | (order[:, :, 1] << 2)).astype(np.uint8)   # [rows, cols/4]
    meta = (meta4[:, 0::2] | (meta4[:, 1::2] << 4)).astype(np.uint8)    # [rows, cols/8]
    return np.concatenate([data.reshape(-1), meta.reshape(-1)]).astype(np.uint8)


def decompress_2of4_e4m3(flat, rows, cols) -> np.ndarray:
    """Inverse of `compress_2of4_e4m3`: dense E4M3 bytes [rows, cols] with zeros where nothing was kept."""
    flat = np.asarray(flat, dtype=np.uint8)
    data = flat[:rows * cols // 2].reshape(rows, cols // 4, 2)
    meta = flat[rows * cols // 2:rows * cols // 2 + rows * cols // 8].reshape(rows, cols // 8)
    meta4 = np.empty((rows, cols // 4), dtype=np.uint8)
    meta4[:, 0::2] = meta & 15
    meta4[:, 1::2] = meta >> 4
    out = np.zeros((rows, cols // 4, 4), dtype=np.uint8)
    r, q = np.meshgrid(np.arange(rows), np.arange(cols // 4), indexing="ij")
    out[r, q, meta4 & 3] = data[:, :, 0]
    out[r, q, (meta4 >> 2) & 3] = data[:, :, 1]
    return out.reshape(rows, cols)


# ----------------------------------------------------------------------------
# Deterministic generator of the reference's micro-benchmarks
# ----------------------------------------------------------------------------

_M64 = (1 << 64) - 1


def pattern(index: int, salt: int, amplitude: float) -> float:
    """`pattern()` (src/cuda.rs:809-818): splitmix64-style hash -> uniform in
    +-amplitude on a 16-bit lattice."""
    v = (index + salt * 0x9E3779B97F4A7C15) & _M64
    v ^= v >> 30
    v = (v * 0xBF58476D1CE4E5B9) & _M64
    v ^= v >> 27
    v = (v * 0x94D049BB133111EB) & _M64
    v ^= v >> 31
    unit = F32(v & 0xFFFF) / F32(65535.0)
    return float((unit * F32(2.0) - F32(1.0)) * F32(amplitude))


def pattern_array(count: int, salt: int, amplitude: float) -> np.ndarray:
    idx = np.arange(count, dtype=np.uint64)
    with np.errstate(over="ignore"):
        v = idx + np.uint64((salt * 0x9E3779B97F4A7C15) & _M64)
        v ^= v >> np.uint64(30)
        v *= np.uint64(0xBF58476D1CE4E5B9)
        v ^= v >> np.uint64(27)
        v *= np.uint64(0x94D049BB133111EB)
        v ^= v >> np.uint64(31)
    unit = (v & np.uint64(0xFFFF)).astype(F32) / F32(65535.0)
    return ((unit * F32(2.0) - F32(1.0)) * F32(amplitude)).astype(F32)


# ----------------------------------------------------------------------------
# Packed-layout size contract (pure integers)
# ----------------------------------------------------------------------------

TILE_ALIGNMENT = 128


def _up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def estimate_linear(fmt: str, logical_in: int, logical_out: int, exl3_bits: int = 4):
    """`estimate_linear` (src/packing.rs:71-130).  Returns a dict or None
    (Q4_K with K % 256 != 0).  fmt in {fp16, fp8_e4m3, int8, q4_k, exl3}."""
    if logical_in == 0 or logical_out == 0:
        raise ValueError("linear dimensions must be nonzero")
    pi, po = _up(logical_in, TILE_ALIGNMENT), _up(logical_out, TILE_ALIGNMENT)
    if fmt == "fp16":
        return dict(padded_in=pi, padded_out=po, payload_bytes=pi * po * 2, metadata_bytes=0)
    if fmt in ("fp8_e4m3", "int8"):
        return dict(padded_in=pi, padded_out=po, payload_bytes=pi * po, metadata_bytes=po * 4)
    if fmt == "q4_k":
        if logical_in % 256:
            return None
        return dict(padded_in=logical_in, padded_out=logical_out,
                    payload_bytes=logical_out * (logical_in // 256) * 144, metadata_bytes=0)
    if fmt == "exl3":
        lay = exl3_layout(logical_in, logical_out, exl3_bits)
        return dict(padded_in=lay["padded_in"], padded_out=lay["padded_out"],
                    payload_bytes=lay["trellis_bytes"], metadata_bytes=lay["scale_bytes"])
    raise ValueError(fmt)


def exl3_layout(logical_in: int, logical_out: int, qbits: int):
    """`Exl3Layout` (src/exl3.rs:38-75)."""
    if logical_in == 0 or logical_out == 0:
        raise ValueError("linear dimensions must be nonzero")
    if not 1 <= qbits <= 8:
        raise ValueError(f"EXL3 supports integer rates from 1 through 8 bpw, got {qbits}")
    pi, po = _up(logical_in, 128), _up(logical_out, 128)
    return dict(padded_in=pi, padded_out=po,
                trellis_shape=[pi // 16, po // 16, 16 * qbits],
                trellis_bytes=pi * po * qbits // 8,
                scale_bytes=2 * (pi + po))


def align_up(value: int, alignment: int) -> int:
    """`align_up` (src/artifact.rs, pinned by :766-769): u64 overflow -> error."""
    r = _up(value, alignment)
    if r > _M64:
        raise OverflowError("align_up overflow")
    return r
