"""CPU restatement of the reference's ".pkl4" artifact format.  TEST INFRASTRUCTURE ONLY: the
product never imports this module.

Follows src/artifact.rs (prefix and header :11-16, :98-156; plan :242-339; writer :345-411;
encoders :413-484; validation :514-724; align_up :734-739), the tensor classes of
src/weights.rs:433-482 and the model manifest of src/weights.rs:510-646.
Pinned to the reference's own unit tests: src/artifact.rs:726-780 (row padding, bias padding,
non-finite rejection, align_up, vocabulary contract) and src/weights.rs:656-670 (tensor and
parameter counts of both profiles)."""
from __future__ import annotations

import json
import struct

import numpy as np

MAGIC = b"PKL4AOT\0"
SCHEMA_VERSION = 2
PREFIX_BYTES = 24
HEADER_ALIGNMENT = 4096
TENSOR_ALIGNMENT = 256
MAX_HEADER_BYTES = 128 * 1024 * 1024
U64_MAX = (1 << 64) - 1

PROFILES = {   # src/config.rs:5-55
    "v2_english": dict(repository="nvidia/parakeet-tdt-0.6b-v2",
                       revision="ae9ad07059c7c739ffaf932226a8fe64ae2620b0", blank=1024),
    "v3_multilingual": dict(repository="nvidia/parakeet-tdt-0.6b-v3",
                            revision="541d1f99c6b0c3cd0b11a95167540bb8edefd82b", blank=8192),
}


class ArtifactInvalid(ValueError):
    pass


def align_up(value: int, alignment: int) -> int:
    """src/artifact.rs:734-739 (u64 arithmetic; overflow is an error)."""
    if value + alignment - 1 > U64_MAX:
        raise ArtifactInvalid("alignment overflow")
    return (value + alignment - 1) // alignment * alignment


# ---------------------------------------------------------------- tensor classes
CANDIDATE_LINEAR = {"ffn", "attention", "pointwise", "subsampling", "encoder_projection",
                    "decoder_projection", "lstm", "joint_head"}


def classify(name: str) -> str:
    """src/weights.rs:433-482."""
    if name.endswith("num_batches_tracked"):
        return "counter"
    if name.endswith(".weight") and ".feed_forward" in name:
        return "ffn"
    if name.endswith((".self_attn.q_proj.weight", ".self_attn.k_proj.weight", ".self_attn.v_proj.weight",
                      ".self_attn.o_proj.weight", ".self_attn.relative_k_proj.weight")):
        return "attention"
    if name.endswith((".conv.pointwise_conv1.weight", ".conv.pointwise_conv2.weight")):
        return "pointwise"
    if name in ("encoder.subsampling.linear.weight", "encoder.subsampling.layers.3.weight",
                "encoder.subsampling.layers.6.weight"):
        return "subsampling"
    if name == "encoder_projector.weight":
        return "encoder_projection"
    if name == "decoder.decoder_projector.weight":
        return "decoder_projection"
    if name.startswith("decoder.lstm.weight_"):
        return "lstm"
    if name == "joint.head.weight":
        return "joint_head"
    if name == "decoder.embedding.weight":
        return "embedding"
    if (name in ("joint.head.bias", "encoder.subsampling.linear.bias", "encoder_projector.bias",
                 "decoder.decoder_projector.bias") or ".conv.norm." in name
            or name.startswith("decoder.lstm.bias_")):
        return "sensitive_fp32"
    if ".conv." in name or name.startswith("encoder.subsampling.layers."):
        return "convolution"
    return "other_fp16"


def linear_shape(shape):
    """src/weights.rs:501-508."""
    shape = tuple(shape)
    if len(shape) == 2 or (len(shape) in (3, 4) and all(d == 1 for d in shape[2:])):
        return shape[0], shape[1]
    return None


def manifest(profile: str, encoder_layers: int = 24):
    """Name -> (dtype, shape) of the source checkpoint (src/weights.rs:510-646)."""
    vocab = PROFILES[profile]["blank"] + 1
    t = {}
    t["decoder.decoder_projector.bias"] = ("F32", (640,))
    t["decoder.decoder_projector.weight"] = ("F32", (640, 640))
    t["decoder.embedding.weight"] = ("F32", (vocab, 640))
    for kind in ("bias_hh", "bias_ih"):
        for layer in range(2):
            t[f"decoder.lstm.{kind}_l{layer}"] = ("F32", (2560,))
    for kind in ("weight_hh", "weight_ih"):
        for layer in range(2):
            t[f"decoder.lstm.{kind}_l{layer}"] = ("F32", (2560, 640))
    for idx, shape in ((0, (256, 1, 3, 3)), (2, (256, 1, 3, 3)), (3, (256, 256, 1, 1)), (5, (256, 1, 3, 3)),
                       (6, (256, 256, 1, 1))):
        t[f"encoder.subsampling.layers.{idx}.bias"] = ("F32", (256,))
        t[f"encoder.subsampling.layers.{idx}.weight"] = ("F32", shape)
    t["encoder.subsampling.linear.bias"] = ("F32", (1024,))
    t["encoder.subsampling.linear.weight"] = ("F32", (1024, 4096))
    if profile == "v2_english":
        t["frontend.mel_filters"] = ("F32", (128, 257))
        t["frontend.window"] = ("F32", (400,))
    for layer in range(encoder_layers):
        p = f"encoder.layers.{layer}"
        t[f"{p}.conv.norm.num_batches_tracked"] = ("I64", ())
        t[f"{p}.conv.depthwise_conv.weight"] = ("F32", (1024, 1, 9))
        for suffix in ("bias", "running_mean", "running_var", "weight"):
            t[f"{p}.conv.norm.{suffix}"] = ("F32", (1024,))
        t[f"{p}.conv.pointwise_conv1.weight"] = ("F32", (2048, 1024, 1))
        t[f"{p}.conv.pointwise_conv2.weight"] = ("F32", (1024, 1024, 1))
        for ff in ("feed_forward1", "feed_forward2"):
            t[f"{p}.{ff}.linear1.weight"] = ("F32", (4096, 1024))
            t[f"{p}.{ff}.linear2.weight"] = ("F32", (1024, 4096))
        for norm in ("norm_conv", "norm_feed_forward1", "norm_feed_forward2", "norm_out", "norm_self_att"):
            t[f"{p}.{norm}.bias"] = ("F32", (1024,))
            t[f"{p}.{norm}.weight"] = ("F32", (1024,))
        t[f"{p}.self_attn.bias_u"] = ("F32", (8, 128))
        t[f"{p}.self_attn.bias_v"] = ("F32", (8, 128))
        for proj in ("k_proj", "o_proj", "q_proj", "relative_k_proj", "v_proj"):
            t[f"{p}.self_attn.{proj}.weight"] = ("F32", (1024, 1024))
    t["encoder_projector.bias"] = ("F32", (640,))
    t["encoder_projector.weight"] = ("F32", (640, 1024))
    t["joint.head.bias"] = ("F32", (vocab + 5,))
    t["joint.head.weight"] = ("F32", (vocab + 5, 640))
    return dict(sorted(t.items()))          # BTreeMap order = byte-wise name order


# ---------------------------------------------------------------- encoders
def _finite(values: np.ndarray, name: str):
    bad = np.flatnonzero(~np.isfinite(values))
    if bad.size:
        raise ArtifactInvalid(f"{name}: non-finite F32 value at element {int(bad[0])}")


def encode_fp16(values, name="tensor") -> bytes:
    """src/artifact.rs:413-428 (half::f16::from_f32 = round to nearest even)."""
    v = np.asarray(values, np.float32).ravel()
    _finite(v, name)
    with np.errstate(over="ignore"):
        return v.astype("<f2").tobytes()


def encode_fp16_linear(values, logical_out, logical_in, padded_out, padded_in, name="tensor") -> bytes:
    """src/artifact.rs:430-467."""
    v = np.asarray(values, np.float32).ravel()
    if v.size != logical_out * logical_in:
        raise ArtifactInvalid(f"{name}: shape requires {logical_out * logical_in * 4} F32 bytes, source has {v.size * 4}")
    _finite(v, name)
    out = np.zeros((padded_out, padded_in), "<f2")
    with np.errstate(over="ignore"):
        out[:logical_out, :logical_in] = v.reshape(logical_out, logical_in).astype("<f2")
    return out.tobytes()


def encode_fp32_bias(values, logical, padded, name="tensor") -> bytes:
    """src/artifact.rs:469-484."""
    v = np.asarray(values, np.float32).ravel()
    if v.size != logical or padded < logical:
        raise ArtifactInvalid(f"{name}: invalid FP32 bias source/padded lengths")
    _finite(v, name)
    out = np.zeros(padded, "<f4")
    out[:logical] = v
    return out.tobytes()


# ---------------------------------------------------------------- plan + writer
def plan(shapes: dict, profile: str, vocabulary):
    """Header of the fp16 plan for tensors name -> shape (src/artifact.rs:242-339)."""
    validate_vocabulary(vocabulary, profile)
    records, cursor = [], 0
    for name in sorted(shapes):
        shape = list(shapes[name])
        family = classify(name)
        if family == "counter":
            continue
        weight_name = name[:-len(".bias")] + ".weight" if name.endswith(".bias") else None
        matching = weight_name if (weight_name in shapes and classify(weight_name) in CANDIDATE_LINEAR) else None
        if family in CANDIDATE_LINEAR:
            ls = linear_shape(shape)
            if ls is None:
                raise ArtifactInvalid(f"{name}: candidate linear has unsupported shape {shape}")
            storage, logical, physical = "sm89_fp16_linear", list(ls), [align_up(ls[0], 128), align_up(ls[1], 128)]
        elif matching is not None:
            out = linear_shape(shapes[matching])[0]
            if shape != [out]:
                raise ArtifactInvalid(f"{name}: bias shape {shape} does not match {matching} output {out}")
            storage, logical, physical = "sm89_fp32_bias", shape, [align_up(out, 128)]
        elif family == "sensitive_fp32" or name.startswith("frontend."):
            storage, logical, physical = "fp32", shape, shape
        else:
            storage, logical, physical = "fp16", shape, shape
        cursor = align_up(cursor, TENSOR_ALIGNMENT)
        nbytes = int(np.prod(physical, dtype=np.uint64)) * (2 if storage in ("fp16", "sm89_fp16_linear") else 4)
        records.append(dict(name=name, storage=storage, logical_shape=logical, physical_shape=physical,
                            offset=cursor, bytes=nbytes))
        cursor += nbytes
    p = PROFILES[profile]
    return dict(schema_version=SCHEMA_VERSION, target="sm_89", profile=profile,
                source_repository=p["repository"], source_revision=p["revision"],
                source_payload_bytes=sum(int(np.prod(s, dtype=np.uint64)) * 4 for s in shapes.values()),
                precision_plan="fp16", tensor_alignment=TENSOR_ALIGNMENT, payload_bytes=cursor,
                vocabulary=list(vocabulary), tensors=records)


def write(path, tensors: dict, profile: str, vocabulary, header_override=None):
    """Writes name -> float32 array as the reference's pack_fp16 does (src/artifact.rs:345-411)."""
    header = plan({k: np.asarray(v).shape for k, v in tensors.items()}, profile, vocabulary)
    if header_override:
        header.update(header_override)
    encoded = json.dumps(header, separators=(",", ":")).encode()
    data_start = align_up(PREFIX_BYTES + len(encoded), HEADER_ALIGNMENT)
    blob = bytearray(data_start + header["payload_bytes"])
    blob[:PREFIX_BYTES] = MAGIC + struct.pack("<IIQ", SCHEMA_VERSION, 0, len(encoded))
    blob[PREFIX_BYTES:PREFIX_BYTES + len(encoded)] = encoded
    for r in header["tensors"]:
        src = np.asarray(tensors[r["name"]], np.float32)
        if r["storage"] == "fp32":
            _finite(src.ravel(), r["name"])
            packed = src.astype("<f4").tobytes()
        elif r["storage"] == "fp16":
            packed = encode_fp16(src, r["name"])
        elif r["storage"] == "sm89_fp16_linear":
            packed = encode_fp16_linear(src, *r["logical_shape"], *r["physical_shape"], r["name"])
        else:
            packed = encode_fp32_bias(src, r["logical_shape"][0], r["physical_shape"][0], r["name"])
        assert len(packed) == r["bytes"], r["name"]
        blob[data_start + r["offset"]:data_start + r["offset"] + len(packed)] = packed
    with open(path, "wb") as f:
        f.write(blob)
    return header


# ---------------------------------------------------------------- reader + validation
def validate_vocabulary(vocabulary, profile):
    """src/artifact.rs:665-685."""
    expected = PROFILES[profile]["blank"]
    if len(vocabulary) != expected:
        raise ArtifactInvalid(f"{profile} requires {expected} vocabulary entries before the blank token, "
                              f"got {len(vocabulary)}")
    for i, piece in enumerate(vocabulary):
        if piece == "" or any(c in piece for c in "\n\r\t"):
            raise ArtifactInvalid(f"vocabulary entry {i} is empty or contains control separators")


def validate_header(header, payload_bytes):
    """src/artifact.rs:514-593, :687-724."""
    if header["schema_version"] != SCHEMA_VERSION:
        raise ArtifactInvalid(f"header schema is {header['schema_version']}, expected {SCHEMA_VERSION}")
    if header["target"] != "sm_89":
        raise ArtifactInvalid(f"target is {header['target']!r}, expected sm_89")
    prof = PROFILES.get(header["profile"])
    if prof is None or header["source_repository"] != prof["repository"] or header["source_revision"] != prof["revision"]:
        raise ArtifactInvalid("profile does not match source repository and revision")
    if header["tensor_alignment"] != TENSOR_ALIGNMENT:
        raise ArtifactInvalid(f"tensor alignment is {header['tensor_alignment']}, expected {TENSOR_ALIGNMENT}")
    if header["payload_bytes"] != payload_bytes:
        raise ArtifactInvalid(f"header declares {header['payload_bytes']} payload bytes, file contains {payload_bytes}")
    validate_vocabulary(header["vocabulary"], header["profile"])
    names, cursor = set(), 0
    for t in header["tensors"]:
        if not t["name"] or t["name"] in names:
            raise ArtifactInvalid(f"empty or duplicate tensor name {t['name']!r}")
        names.add(t["name"])
        if t["offset"] % TENSOR_ALIGNMENT or t["offset"] < cursor:
            raise ArtifactInvalid(f"{t['name']}: invalid aligned offset {t['offset']} after {cursor}")
        lo, ph, st = list(t["logical_shape"]), list(t["physical_shape"]), t["storage"]
        if st in ("fp16", "fp32"):
            if lo != ph:
                raise ArtifactInvalid(f"{t['name']}: plain storage cannot change logical shape {lo} to {ph}")
        elif st == "sm89_fp16_linear":
            if not (len(lo) == 2 and lo[0] > 0 and lo[1] > 0 and ph == [align_up(lo[0], 128), align_up(lo[1], 128)]):
                raise ArtifactInvalid(f"{t['name']}: invalid sm_89 FP16 linear shapes {lo} -> {ph}")
        elif st == "sm89_fp32_bias":
            if not (len(lo) == 1 and lo[0] > 0 and ph == [align_up(lo[0], 128)]):
                raise ArtifactInvalid(f"{t['name']}: invalid sm_89 FP32 bias shapes {lo} -> {ph}")
        else:
            raise ArtifactInvalid(f"{t['name']}: unknown storage {st}")
        elements = 1
        for d in ph:
            elements *= d
        expected = elements * (2 if st in ("fp16", "sm89_fp16_linear") else 4)
        if t["bytes"] != expected:
            raise ArtifactInvalid(f"{t['name']}: physical shape and storage require {expected} bytes, "
                                  f"header declares {t['bytes']}")
        cursor = t["offset"] + t["bytes"]
        if cursor > payload_bytes:
            raise ArtifactInvalid(f"{t['name']}: range ends at {cursor}, beyond {payload_bytes}-byte payload")
    if cursor != payload_bytes:
        raise ArtifactInvalid(f"last tensor ends at {cursor}, payload ends at {payload_bytes}")


def read(path):
    """AotArtifactIndex::open (src/artifact.rs:98-156) + logical views of every tensor."""
    blob = open(path, "rb").read()
    if len(blob) < PREFIX_BYTES:
        raise ArtifactInvalid(f"file has {len(blob)} bytes; prefix requires {PREFIX_BYTES}")
    if blob[:8] != MAGIC:
        raise ArtifactInvalid("bad magic")
    version, flags, header_bytes = struct.unpack("<IIQ", blob[8:24])
    if version != SCHEMA_VERSION:
        raise ArtifactInvalid(f"expected schema version {SCHEMA_VERSION}, got {version}")
    if flags != 0:
        raise ArtifactInvalid(f"unsupported prefix flags {flags:#x}")
    if header_bytes == 0 or header_bytes > MAX_HEADER_BYTES:
        raise ArtifactInvalid(f"header length {header_bytes} is outside 1..={MAX_HEADER_BYTES}")
    data_start = align_up(PREFIX_BYTES + header_bytes, HEADER_ALIGNMENT)
    if data_start > len(blob):
        raise ArtifactInvalid(f"aligned header ends at {data_start}, beyond file length {len(blob)}")
    header = json.loads(blob[PREFIX_BYTES:PREFIX_BYTES + header_bytes])
    validate_header(header, len(blob) - data_start)
    tensors = {}
    for t in header["tensors"]:
        dtype = "<f2" if t["storage"] in ("fp16", "sm89_fp16_linear") else "<f4"
        raw = np.frombuffer(blob, dtype, count=t["bytes"] // np.dtype(dtype).itemsize, offset=data_start + t["offset"])
        phys = raw.reshape(t["physical_shape"])
        tensors[t["name"]] = phys[tuple(slice(0, d) for d in t["logical_shape"])]
    return header, tensors
