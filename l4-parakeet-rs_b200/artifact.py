"""Host-side mirror of the reference's artifact loader (src/artifact.rs: AotArtifactIndex,
src/cuda/encoder.rs:530-601 LayerWeights::load, src/cuda/decoder.rs:227-271 DecoderWeights,
src/cuda/subsampling.rs weight lookup) over the C reader in libpk100.so.

`Artifact(path)` maps the file; `tensor(name)` returns a zero-copy numpy view of the LOGICAL
shape (padding of the linear storages sliced away); `layer_weights(i)`, `subsampling_weights()`
and `decoder_weights()` return the dictionaries that `EncoderLayers.add_layer`, `Subsampling`
and `TdtDecoder` take, keyed by the checkpoint names of src/weights.rs:510-646."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import lib as L

vp = C.c_void_p


class ArtifactTensorC(C.Structure):
    _fields_ = [("name", C.c_char_p), ("storage", C.c_int), ("logical_rank", C.c_int),
                ("physical_rank", C.c_int), ("logical_shape", C.c_longlong * 4),
                ("physical_shape", C.c_longlong * 4), ("offset", C.c_ulonglong), ("bytes", C.c_ulonglong),
                ("data", vp)]


_l = L.lib
_l.pk100_artifact_open.argtypes = [C.c_char_p, C.POINTER(vp), C.c_char_p, C.c_int]
_l.pk100_artifact_open.restype = C.c_int
_l.pk100_artifact_close.argtypes = [vp]
_l.pk100_artifact_close.restype = None
_l.pk100_artifact_tensor_count.argtypes = [vp]
_l.pk100_artifact_tensor_count.restype = C.c_int
_l.pk100_artifact_tensor_at.argtypes = [vp, C.c_int, C.POINTER(ArtifactTensorC)]
_l.pk100_artifact_tensor_at.restype = C.c_int
_l.pk100_artifact_find.argtypes = [vp, C.c_char_p]
_l.pk100_artifact_find.restype = C.c_int
_l.pk100_artifact_vocabulary_size.argtypes = [vp]
_l.pk100_artifact_vocabulary_size.restype = C.c_int
_l.pk100_artifact_vocabulary_at.argtypes = [vp, C.c_int]
_l.pk100_artifact_vocabulary_at.restype = C.c_char_p
_l.pk100_artifact_field.argtypes = [vp, C.c_char_p]
_l.pk100_artifact_field.restype = C.c_char_p
_l.pk100_artifact_read_f32.argtypes = [vp, C.c_char_p, vp, C.c_longlong]
_l.pk100_artifact_read_f32.restype = C.c_int
_l.pk100_encode_fp16.argtypes = [vp, C.c_longlong, vp]
_l.pk100_encode_fp16.restype = C.c_int
_l.pk100_encode_fp16_linear.argtypes = [vp, C.c_longlong, C.c_longlong, C.c_longlong, C.c_longlong, vp]
_l.pk100_encode_fp16_linear.restype = C.c_int
_l.pk100_encode_fp32_bias.argtypes = [vp, C.c_longlong, C.c_longlong, vp]
_l.pk100_encode_fp32_bias.restype = C.c_int
_l.pk100_align_up.argtypes = [C.c_ulonglong, C.c_ulonglong, C.POINTER(C.c_int)]
_l.pk100_align_up.restype = C.c_ulonglong

STORAGE_NAMES = {0: "fp16", 1: "fp32", 2: "sm89_fp16_linear", 3: "sm89_fp32_bias"}
ERR_FORMAT, ERR_IO = -7, -8


class ArtifactError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"invalid L4 artifact: {message}" if code == ERR_FORMAT else message)
        self.code = code
        self.message = message


class Artifact:
    def __init__(self, path):
        self._h = None
        handle = vp()
        error = C.create_string_buffer(512)
        rc = _l.pk100_artifact_open(str(path).encode(), C.byref(handle), error, len(error))
        if rc != 0:
            raise ArtifactError(rc, error.value.decode(errors="replace"))
        self._h = handle
        self.records = {}
        for i in range(_l.pk100_artifact_tensor_count(self._h)):
            rec = ArtifactTensorC()
            L.check(_l.pk100_artifact_tensor_at(self._h, i, C.byref(rec)), "pk100_artifact_tensor_at")
            self.records[rec.name.decode()] = dict(
                storage=STORAGE_NAMES[rec.storage], logical_shape=list(rec.logical_shape[:rec.logical_rank]),
                physical_shape=list(rec.physical_shape[:rec.physical_rank]), offset=rec.offset, bytes=rec.bytes,
                data=rec.data)
        self.vocabulary = [_l.pk100_artifact_vocabulary_at(self._h, i).decode()
                           for i in range(_l.pk100_artifact_vocabulary_size(self._h))]

    def close(self):
        if self._h:
            _l.pk100_artifact_close(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def field(self, key):
        v = _l.pk100_artifact_field(self._h, key.encode())
        return None if v is None else v.decode()

    def find(self, name):
        return _l.pk100_artifact_find(self._h, name.encode())

    def tensor(self, name):
        """Zero-copy view of the logical tensor (valid while the artifact is open)."""
        r = self.records[name]
        dtype = np.float16 if r["storage"] in ("fp16", "sm89_fp16_linear") else np.float32
        count = r["bytes"] // np.dtype(dtype).itemsize
        buf = (C.c_char * r["bytes"]).from_address(r["data"])
        phys = np.frombuffer(buf, dtype=dtype, count=count).reshape(r["physical_shape"])
        return phys[tuple(slice(0, d) for d in r["logical_shape"])]

    def read_f32(self, name):
        r = self.records[name]
        out = np.empty(r["bytes"] // 4, np.float32)
        rc = _l.pk100_artifact_read_f32(self._h, name.encode(), out.ctypes.data, out.size)
        if rc != 0:
            raise ArtifactError(rc, f"{name}: tensor is not plain finite FP32 storage")
        return out.reshape(r["logical_shape"])

    # ------------------------------------------------------------ model views
    def _f32(self, name, shape=None):
        a = np.array(self.tensor(name), dtype=np.float32)     # a writable copy, detached from the mapping
        return a.reshape(shape) if shape is not None else a

    def layer_weights(self, layer):
        """Dictionary for EncoderLayers.add_layer (names of src/weights.rs:575-631)."""
        p = f"encoder.layers.{layer}"
        w = {}
        for ours, ff in (("ff1", "feed_forward1"), ("ff2", "feed_forward2")):
            w[f"{ours}_w1"] = self._f32(f"{p}.{ff}.linear1.weight")
            w[f"{ours}_w2"] = self._f32(f"{p}.{ff}.linear2.weight")
        for ours, proj in (("wq", "q_proj"), ("wk", "k_proj"), ("wv", "v_proj"), ("wo", "o_proj"),
                           ("wpos", "relative_k_proj")):
            w[ours] = self._f32(f"{p}.self_attn.{proj}.weight")
        w["wpw1"] = self._f32(f"{p}.conv.pointwise_conv1.weight")
        w["wpw2"] = self._f32(f"{p}.conv.pointwise_conv2.weight")
        w["bias_u"] = self._f32(f"{p}.self_attn.bias_u")
        w["bias_v"] = self._f32(f"{p}.self_attn.bias_v")
        w["dw"] = self._f32(f"{p}.conv.depthwise_conv.weight", (1024, 9))
        for ours, norm in (("ff1", "norm_feed_forward1"), ("att", "norm_self_att"), ("conv", "norm_conv"),
                           ("ff2", "norm_feed_forward2"), ("out", "norm_out")):
            w[f"ln_{ours}_g"] = self._f32(f"{p}.{norm}.weight")
            w[f"ln_{ours}_b"] = self._f32(f"{p}.{norm}.bias")
        for ours, suffix in (("bn_g", "weight"), ("bn_b", "bias"), ("bn_m", "running_mean"), ("bn_v", "running_var")):
            w[ours] = self._f32(f"{p}.conv.norm.{suffix}")
        return w

    def subsampling_weights(self):
        """Dictionary for Subsampling (names of src/weights.rs:552-568)."""
        s = "encoder.subsampling"
        return {
            "conv0_w": self._f32(f"{s}.layers.0.weight", (256, 9)), "conv0_b": self._f32(f"{s}.layers.0.bias"),
            "dw1_w": self._f32(f"{s}.layers.2.weight", (256, 9)), "dw1_b": self._f32(f"{s}.layers.2.bias"),
            "pw1_w": self._f32(f"{s}.layers.3.weight"), "pw1_b": self._f32(f"{s}.layers.3.bias"),
            "dw2_w": self._f32(f"{s}.layers.5.weight", (256, 9)), "dw2_b": self._f32(f"{s}.layers.5.bias"),
            "pw2_w": self._f32(f"{s}.layers.6.weight"), "pw2_b": self._f32(f"{s}.layers.6.bias"),
            "proj_w": self._f32(f"{s}.linear.weight"), "proj_b": self._f32(f"{s}.linear.bias"),
        }

    def decoder_weights(self, layers=2):
        """Dictionary for TdtDecoder (names of src/weights.rs:526-550, :633-644)."""
        w = {"layers": layers, "embedding": self._f32("decoder.embedding.weight"),
             "w_pred": self._f32("decoder.decoder_projector.weight"), "b_pred": self._f32("decoder.decoder_projector.bias"),
             "w_joint": self._f32("joint.head.weight"), "b_joint": self._f32("joint.head.bias"),
             "w_enc": self._f32("encoder_projector.weight"), "b_enc": self._f32("encoder_projector.bias")}
        for l in range(layers):
            w[f"w_ih{l}"] = self._f32(f"decoder.lstm.weight_ih_l{l}")
            w[f"w_hh{l}"] = self._f32(f"decoder.lstm.weight_hh_l{l}")
            w[f"b_ih{l}"] = self._f32(f"decoder.lstm.bias_ih_l{l}")
            w[f"b_hh{l}"] = self._f32(f"decoder.lstm.bias_hh_l{l}")
        return w


def encode_fp16(values):
    v = np.ascontiguousarray(values, np.float32).ravel()
    out = np.empty(v.size, np.uint16)
    rc = _l.pk100_encode_fp16(v.ctypes.data, v.size, out.ctypes.data)
    if rc != 0:
        raise ArtifactError(rc, "non-finite F32 value")
    return out.view(np.float16)


def encode_fp16_linear(values, logical_out, logical_in, padded_out, padded_in):
    v = np.ascontiguousarray(values, np.float32).ravel()
    if v.size != logical_out * logical_in:
        raise ArtifactError(ERR_FORMAT, f"shape requires {logical_out * logical_in * 4} F32 bytes, source has {v.size * 4}")
    out = np.empty((padded_out, padded_in), np.uint16)
    rc = _l.pk100_encode_fp16_linear(v.ctypes.data, logical_out, logical_in, padded_out, padded_in, out.ctypes.data)
    if rc != 0:
        raise ArtifactError(rc, "non-finite F32 value or bad padded shape")
    return out.view(np.float16)


def encode_fp32_bias(values, logical, padded):
    v = np.ascontiguousarray(values, np.float32).ravel()
    if v.size != logical:
        raise ArtifactError(ERR_FORMAT, "invalid FP32 bias source/padded lengths")
    out = np.empty(max(padded, 0), np.float32)
    rc = _l.pk100_encode_fp32_bias(v.ctypes.data, logical, padded, out.ctypes.data)
    if rc != 0:
        raise ArtifactError(rc, "invalid FP32 bias source/padded lengths")
    return out


def align_up(value, alignment):
    overflow = C.c_int(0)
    out = _l.pk100_align_up(value, alignment, C.byref(overflow))
    if overflow.value:
        raise ArtifactError(ERR_FORMAT, "alignment overflow")
    return int(out)


# ---- packed-layout size contract (src/packing.rs:71-130, src/exl3.rs:38-75) ----

FORMATS = {"fp16": 0, "fp8_e4m3": 1, "int8": 2, "q4_k": 3, "exl3": 4}


class LinearLayoutC(C.Structure):
    _fields_ = [("logical_in", C.c_longlong), ("logical_out", C.c_longlong), ("padded_in", C.c_longlong),
                ("padded_out", C.c_longlong), ("payload_bytes", C.c_ulonglong), ("metadata_bytes", C.c_ulonglong),
                ("available", C.c_int)]


class Exl3LayoutC(C.Structure):
    _fields_ = [("padded_in", C.c_longlong), ("padded_out", C.c_longlong), ("trellis_shape", C.c_longlong * 3),
                ("trellis_bytes", C.c_ulonglong), ("scale_bytes", C.c_ulonglong)]


_l.pk100_estimate_linear.argtypes = [C.c_int, C.c_longlong, C.c_longlong, C.c_int, C.POINTER(LinearLayoutC)]
_l.pk100_estimate_linear.restype = C.c_int
_l.pk100_exl3_layout.argtypes = [C.c_longlong, C.c_longlong, C.c_int, C.POINTER(Exl3LayoutC)]
_l.pk100_exl3_layout.restype = C.c_int


def estimate_linear(fmt, logical_in, logical_out, exl3_bits=4):
    """`estimate_linear`: dict of padded shape and byte counts, or None where the format has no
    layout for this shape (Q4_K with K % 256 != 0)."""
    out = LinearLayoutC()
    rc = _l.pk100_estimate_linear(FORMATS[fmt], logical_in, logical_out, exl3_bits, C.byref(out))
    if rc != 0:
        raise ValueError("linear dimensions must be nonzero" if rc == -2 else f"estimate_linear: error {rc}")
    if not out.available:
        return None
    return dict(padded_in=out.padded_in, padded_out=out.padded_out, payload_bytes=out.payload_bytes,
                metadata_bytes=out.metadata_bytes)


def exl3_layout(logical_in, logical_out, qbits):
    out = Exl3LayoutC()
    rc = _l.pk100_exl3_layout(logical_in, logical_out, qbits, C.byref(out))
    if rc != 0:
        raise ValueError("linear dimensions must be nonzero" if rc == -2 else
                         f"EXL3 supports integer rates from 1 through 8 bpw, got {qbits}")
    return dict(padded_in=out.padded_in, padded_out=out.padded_out, trellis_shape=list(out.trellis_shape),
                trellis_bytes=out.trellis_bytes, scale_bytes=out.scale_bytes)
