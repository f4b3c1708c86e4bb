"""Routed experts of a `.gturbo` artifact, read straight into HBM.

A repacked model keeps its routed experts under `packed_experts/`: `layout.json`
(GTurboPackedExpertsLayoutV1.swift) and one `layer_NN.bin` per layer holding
`expertsPerLayer` blobs `expertStride` bytes apart, expert e at `physicalRank(e) * stride`.
`manifest.json` (GTurboManifestV1.swift) carries the quantisation slots, the architecture and
a size + SHA-256 per file.  The reference streams single experts from those files into a slot
cache (`ExpertStreamer`, expert_io.c); a B200 holds every expert, so this loader reads whole
layers into device memory in LOGICAL expert order, which is the layout
`MoE.register_layer(experts=..., expert_stride=...)` wants.

The validation restates `GTurboV1StructuralValidator.validate` / `crossValidate`
(GTurboPackedExpertsLayoutV1.swift:73-196) and the parts of `GTurboManifestCodec.validate`
(GTurboManifestV1.swift:159-254) that concern this path; a rule that fails raises
`GTurboFormatError(field, reason)` with the reference's field naming.
"""
from __future__ import annotations

import hashlib
import json
import os
from dataclasses import dataclass

import numpy as np

from . import _lib
from . import format as fmt

MAGIC = "GTURBO"                 # GTurboFormatV1.swift:4-7
VERSION_MAJOR = 1
ALIGNMENT = 16_384
KNOWN_FLAGS = {"streamingPresent", "turboQuantKV", "aneSharedExpert"}
TENSOR_KEYS = ("gate", "gate_scales", "gate_biases", "up", "up_scales", "up_biases",
               "down", "down_scales", "down_biases")      # GTurboJSON.swift:129-135, ModelExpertIO.swift:67-82


class GTurboFormatError(ValueError):
    def __init__(self, field: str, reason: str):
        super().__init__(f"{field}: {reason}")
        self.field, self.reason = field, reason


def _basename_ok(name) -> bool:
    return isinstance(name, str) and name not in ("", ".", "..") and "/" not in name and "\\" not in name and "\0" not in name


def _u64(v, field: str) -> int:
    if isinstance(v, bool) or not isinstance(v, int) or v < 0 or v >= 1 << 64:
        raise GTurboFormatError(field, "expected an unsigned 64-bit integer")
    return v


@dataclass
class PackedExpertsLayout:
    expert_stride: int
    num_layers: int
    experts_per_layer: int
    layers: dict            # layer id -> {"file": str, "physical": int array [E] (logical -> rank), "tensors": dict of expert 0}

    def file(self, layer: int) -> str:
        return self.layers[layer]["file"]

    def physical_offsets(self, layer: int) -> np.ndarray:
        """`Model.routedExpertPhysicalOffsets` (ModelExpertIO.swift:84-86): file offset of each logical expert."""
        return self.layers[layer]["physical"].astype(np.uint64) * np.uint64(self.expert_stride)

    def expert_offsets(self, layer: int) -> dict:
        """`Model.routedExpertOffsets` (ModelExpertIO.swift:67-82): the nine offsets inside a blob, from expert 0."""
        t = self.layers[layer]["tensors"]
        return {name: int(t[key]["offset"]) if key in t else 0 for name, key in zip(fmt.OFFSET_NAMES, TENSOR_KEYS)}

    def weight_bits(self, layer: int) -> int | None:
        return self.layers[layer]["tensors"].get("gate", {}).get("bits")


def decode_layout(data) -> PackedExpertsLayout:
    """`GTurboPackedExpertsLayoutCodec.decode` + `GTurboV1StructuralValidator.validate`."""
    try:
        obj = json.loads(data) if isinstance(data, (bytes, str)) else data
        stride, n_layers, per_layer, layers = obj["expertStride"], obj["numLayers"], obj["expertsPerLayer"], obj["layers"]
    except (ValueError, KeyError, TypeError) as e:
        raise GTurboFormatError("packed_experts/layout.json", str(e)) from None
    if not (isinstance(n_layers, int) and isinstance(per_layer, int) and isinstance(stride, int) and n_layers > 0
            and per_layer > 0 and stride > 0 and stride % ALIGNMENT == 0 and isinstance(layers, list)
            and len(layers) == n_layers):
        raise GTurboFormatError("layout", "invalid dimensions or stride")
    out, files = {}, set()
    for lay in layers:
        lid = lay.get("layer")
        if not isinstance(lid, int) or lid < 0 or lid >= n_layers or lid in out:
            raise GTurboFormatError("layout.layers", "duplicate or invalid layer")
        field = f"layout.layers[{lid}]"
        name = lay.get("file")
        if not _basename_ok(name):
            raise GTurboFormatError(field + ".file", "not a plain file name")
        key = name.lower()                      # the reference compares names the way a case-insensitive volume does
        if key == "layout.json":
            raise GTurboFormatError(field + ".file", "reserved packed-expert filename")
        if key in files:
            raise GTurboFormatError(field + ".file", "duplicate layer filename")
        files.add(key)
        experts = lay.get("experts")
        if not isinstance(experts, list) or len(experts) != per_layer:
            raise GTurboFormatError(field + ".experts", "wrong expert count")
        explicit = [e.get("expert") is not None for e in experts]
        if any(explicit) and not all(explicit):
            raise GTurboFormatError(field + ".experts", "expert ids must be either all explicit or all positional")
        physical = np.full(per_layer, -1, dtype=np.int64)
        ranks, offsets = set(), set()
        tensors0 = None
        for pos, e in enumerate(experts):
            logical = e["expert"] if e.get("expert") is not None else pos
            rank = e["physicalRank"] if e.get("physicalRank") is not None else logical
            off, size = _u64(e.get("offset"), "expert.offset"), _u64(e.get("size"), "expert.size")
            if not (isinstance(logical, int) and isinstance(rank, int) and 0 <= logical < per_layer
                    and 0 <= rank < per_layer and physical[logical] < 0 and rank not in ranks and off not in offsets):
                raise GTurboFormatError(field + ".experts", "duplicate or invalid expert mapping")
            physical[logical] = rank
            ranks.add(rank); offsets.add(off)
            if rank * stride >= 1 << 64:
                raise GTurboFormatError("expert.offset", "arithmetic overflow")
            if off != rank * stride or size != stride:
                raise GTurboFormatError(f"expert[{logical}]", "offset or size does not match physical rank")
            spans = []
            tensors = e.get("tensors", {})
            for tname, t in tensors.items():
                shape, bits = t.get("shape"), t.get("bits")
                if not (t.get("dtype") in ("U32", "BF16") and tname and isinstance(t.get("size"), int) and t["size"] > 0
                        and isinstance(shape, list) and shape and all(isinstance(v, int) and v > 0 for v in shape)
                        and (bits is None or (isinstance(bits, int) and 0 < bits <= 32))):
                    raise GTurboFormatError(f"expert[{logical}].tensors.{tname}", "invalid dtype or shape")
                end = _u64(t.get("offset"), f"tensor.{tname}.range") + t["size"]
                if end > size:
                    raise GTurboFormatError(f"expert[{logical}].tensors.{tname}", "range exceeds expert blob")
                spans.append((t["offset"], end, tname))
            spans.sort()
            for a, b in zip(spans, spans[1:]):
                if a[1] > b[0]:
                    raise GTurboFormatError(f"expert[{logical}].tensors", f"overlapping ranges {a[2]} and {b[2]}")
            if logical == 0:
                tensors0 = tensors
        out[lid] = {"file": name, "physical": physical, "tensors": tensors0 or {}}
    return PackedExpertsLayout(stride, n_layers, per_layer, out)


@dataclass
class Manifest:
    model_id: str
    num_layers: int
    experts_per_layer: int
    expert_stride: int
    arch: dict
    quant: dict | None
    files: dict             # relative path -> {"size": int, "sha256": str}


def decode_manifest(data) -> Manifest:
    """`GTurboManifestCodec.decode`: the checks on magic, version, flags, dimensions, the architecture fields this path
    reads, the quantisation slots and the file table (GTurboManifestV1.swift:159-254)."""
    try:
        m = json.loads(data) if isinstance(data, (bytes, str)) else data
        arch, files = m["arch"], m["files"]
        n_layers, per_layer, stride = m["numLayers"], m["expertsPerLayer"], m["expertStride"]
    except (ValueError, KeyError, TypeError) as e:
        raise GTurboFormatError("manifest.json", str(e)) from None
    if m.get("magic") != MAGIC:
        raise GTurboFormatError("manifest.magic", "expected GTURBO")
    if m.get("versionMajor") != VERSION_MAJOR or not isinstance(m.get("versionMinor"), int) or m["versionMinor"] < 0:
        raise GTurboFormatError("manifest.version", "unsupported version")
    for flag in m.get("flags", {}):
        if flag not in KNOWN_FLAGS:
            raise GTurboFormatError(f"manifest.flags.{flag}", "unknown v1 flag")
    if not (m.get("modelID") and isinstance(n_layers, int) and isinstance(per_layer, int) and isinstance(stride, int)
            and n_layers > 0 and per_layer > 0 and stride > 0 and stride % ALIGNMENT == 0):
        raise GTurboFormatError("manifest", "invalid dimensions or stride")
    if arch.get("numLayers") != n_layers or arch.get("numExperts") != per_layer:
        raise GTurboFormatError("manifest.arch", "dimensions disagree with streaming metadata")
    ints = [arch.get(k) for k in ("hiddenSize", "moeIntermediateSize", "topKExperts")]
    if not all(isinstance(v, int) and v > 0 for v in ints) or arch["topKExperts"] > arch["numExperts"] \
            or not arch.get("hiddenActivation"):
        raise GTurboFormatError("manifest.arch", "invalid architecture values")
    quant = m.get("quant")
    if quant is not None:
        for name in ("embedding", "attention", "router", "sharedExpert", "routedExpert"):
            s = quant.get(name, {})
            if not (isinstance(s.get("weightBits"), int) and 0 < s["weightBits"] <= 32 and isinstance(s.get("groupSize"), int)
                    and s["groupSize"] > 0 and s.get("scheme") and s.get("scaleType") and s.get("biasType")):
                raise GTurboFormatError(f"manifest.quant.{name}", "invalid quantization values")
    seen = set()
    for path, entry in files.items():
        parts = path.split("/")
        if path.startswith("/") or not all(_basename_ok(p) for p in parts):
            raise GTurboFormatError(f"manifest.files.{path}", "not a relative path inside the artifact")
        key = path.lower()
        if key in seen:
            raise GTurboFormatError(f"manifest.files.{path}", "filesystem-equivalent duplicate path")
        seen.add(key)
        if key in ("manifest.json", "verified-install.json", "tokenizer"):
            raise GTurboFormatError(f"manifest.files.{path}", "reserved artifact filename")
        sha = entry.get("sha256", "")
        if len(sha) != 64 or any(c not in "0123456789abcdefABCDEF" for c in sha):
            raise GTurboFormatError(f"manifest.files.{path}.sha256", "expected 64 hexadecimal characters")
        _u64(entry.get("size"), f"manifest.files.{path}.size")
    return Manifest(m["modelID"], n_layers, per_layer, stride, arch, quant, files)


def cross_validate(manifest: Manifest, layout: PackedExpertsLayout) -> None:
    """`GTurboV1StructuralValidator.crossValidate` (GTurboPackedExpertsLayoutV1.swift:160-196)."""
    if (manifest.num_layers, manifest.experts_per_layer, manifest.expert_stride) != \
            (layout.num_layers, layout.experts_per_layer, layout.expert_stride):
        raise GTurboFormatError("manifest/layout", "dimension mismatch")
    want = layout.experts_per_layer * layout.expert_stride
    for lid in layout.layers:
        path = "packed_experts/" + layout.file(lid)
        if manifest.files.get(path, {}).get("size") != want:
            raise GTurboFormatError(f"manifest.files.{path}", "missing or wrong layer size")


def sha256_file(path) -> str:
    """`Sha256Verifier.hashFile` (Infrastructure/ModelIO/Sha256Verifier.swift): lower-case hex digest."""
    h = hashlib.sha256()
    with open(path, "rb") as fh:
        for chunk in iter(lambda: fh.read(8 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


class GTurboExperts:
    """The routed experts of one artifact directory."""

    def __init__(self, root):
        self.root = os.fspath(root)
        with open(os.path.join(self.root, "manifest.json"), "rb") as fh:
            self.manifest = decode_manifest(fh.read())
        with open(os.path.join(self.root, "packed_experts", "layout.json"), "rb") as fh:
            self.layout = decode_layout(fh.read())
        cross_validate(self.manifest, self.layout)

    @property
    def layer_bytes(self) -> int:
        return self.layout.experts_per_layer * self.layout.expert_stride

    def layer_path(self, layer: int) -> str:
        return os.path.join(self.root, "packed_experts", self.layout.file(layer))

    def routed_bits(self, layer: int = 0) -> int:
        bits = self.layout.weight_bits(layer)
        if bits is None and self.manifest.quant is not None:
            bits = self.manifest.quant["routedExpert"]["weightBits"]
        if bits not in (4, 8):
            raise GTurboFormatError("manifest.quant.routedExpert", f"{bits}-bit routed experts are not supported")
        return bits

    def meta_dtype(self) -> int:
        scale = (self.manifest.quant or {}).get("routedExpert", {}).get("scaleType", "bf16").lower()
        if scale not in ("bf16", "fp16", "f16"):
            raise GTurboFormatError("manifest.quant.routedExpert.scaleType", f"unsupported scale type {scale}")
        return fmt.META_BF16 if scale == "bf16" else fmt.META_FP16

    def verify_layer(self, layer: int) -> None:
        """size and SHA-256 of the layer file against the manifest (the install-time check of the reference)"""
        rel = "packed_experts/" + self.layout.file(layer)
        entry = self.manifest.files[rel]
        path = self.layer_path(layer)
        if os.path.getsize(path) != entry["size"]:
            raise GTurboFormatError(f"manifest.files.{rel}", "file size differs from the manifest")
        if sha256_file(path) != entry["sha256"].lower():
            raise GTurboFormatError(f"manifest.files.{rel}.sha256", "digest mismatch")

    def copy_plan(self, layer: int) -> list[tuple[int, int, int]]:
        """(file offset, device offset, bytes) runs that put the blobs in logical order; consecutive experts whose
        ranks are consecutive too share a run, so the identity mapping is one run"""
        stride = self.layout.expert_stride
        rank = self.layout.layers[layer]["physical"]
        runs, start = [], 0
        for e in range(1, len(rank) + 1):
            if e == len(rank) or rank[e] != rank[e - 1] + 1:
                runs.append((int(rank[start]) * stride, start * stride, (e - start) * stride))
                start = e
        return runs

    def load_layer(self, layer: int, device_ptr, *, stream=None, verify: bool = False) -> None:
        """Reads the layer's blobs to `device_ptr` (`layer_bytes` bytes of device memory, 16-byte aligned) in logical
        expert order through the library's pinned double-buffered reader."""
        if verify:
            self.verify_layer(layer)
        lib = _lib.lib()
        base = int(device_ptr.data_ptr()) if hasattr(device_ptr, "data_ptr") else int(device_ptr)
        path = self.layer_path(layer).encode()
        st = None if stream is None else (stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream))
        for src, dst, n in self.copy_plan(layer):
            _lib.check(lib.nvmai_cuda_moe_read_file_to_device(path, src, n, base + dst, st), "read_file_to_device")

    def register_layer(self, moe, layer: int, experts_dev, **other_tensors) -> None:
        """`MoE.register_layer` with the stride and the nine offsets of the layout; router, shared expert and gate
        tensors (`model_weights.bin` in the artifact) are the caller's."""
        moe.register_layer(layer, experts=experts_dev, expert_stride=self.layout.expert_stride,
                           offsets=self.layout.expert_offsets(layer), **other_tensors)


def write_packed_experts(root, layers: list, *, d: int, f: int, bits: int, top_k: int = 8, physical_ranks=None,
                         model_id: str = "synthetic") -> None:
    """Writes `manifest.json`, `packed_experts/layout.json` and `layer_NN.bin` for blobs `layers[l]` (uint8
    [experts, blob bytes], logical order; the stride is the blob size rounded up to 16 KiB) the way the reference's
    synthetic artifact does
    (tests/NVMAI/Core/Runtime/QwenToySynthetic.swift:236-400).  `physical_ranks[l][e]` (optional) places expert e at
    that rank of the file."""
    root = os.fspath(root)
    pe = os.path.join(root, "packed_experts")
    os.makedirs(pe, exist_ok=True)
    n_experts, blob_bytes = layers[0].shape
    off, want_bytes = fmt.expert_offsets(d, f, bits)
    assert blob_bytes == want_bytes, "blobs do not have the size of the nine sub-tensors"
    stride = (blob_bytes + ALIGNMENT - 1) // ALIGNMENT * ALIGNMENT
    g = d // 64
    shapes = {"gate": ([f, d], f * d * bits // 8), "up": ([f, d], f * d * bits // 8), "down": ([d, f], d * f * bits // 8)}
    meta = {"gate": [f, g], "up": [f, g], "down": [d, f // 64]}
    tensors = {}
    for role in ("gate", "up", "down"):
        tensors[role] = {"offset": off[role + "_w"], "size": shapes[role][1], "dtype": "U32", "shape": shapes[role][0],
                         "bits": bits}
        for comp, key in (("s", "_scales"), ("b", "_biases")):
            tensors[role + key] = {"offset": off[f"{role}_{comp}"], "size": meta[role][0] * meta[role][1] * 2,
                                   "dtype": "BF16", "shape": meta[role]}
    files, layer_entries = {}, []
    for l, blobs in enumerate(layers):
        rank = np.arange(n_experts) if physical_ranks is None else np.asarray(physical_ranks[l])
        payload = np.zeros((n_experts, stride), dtype=np.uint8)
        payload[rank, :blob_bytes] = blobs
        name = f"layer_{l:02d}.bin"
        payload.tofile(os.path.join(pe, name))
        files["packed_experts/" + name] = {"size": int(payload.size), "sha256": sha256_file(os.path.join(pe, name))}
        experts = []
        for e in range(n_experts):
            entry = {"expert": e, "offset": int(rank[e]) * stride, "size": stride, "tensors": tensors}
            if physical_ranks is not None:
                entry["physicalRank"] = int(rank[e])
            experts.append(entry)
        layer_entries.append({"layer": l, "file": name, "experts": experts})
    layout = {"expertStride": stride, "numLayers": len(layers), "expertsPerLayer": n_experts, "layers": layer_entries}
    with open(os.path.join(pe, "layout.json"), "w") as fh:
        json.dump(layout, fh, sort_keys=True)
    files["packed_experts/layout.json"] = {"size": os.path.getsize(os.path.join(pe, "layout.json")),
                                           "sha256": sha256_file(os.path.join(pe, "layout.json"))}
    slot = lambda b: {"weightBits": b, "scheme": "affine", "scaleType": "bf16", "biasType": "bf16", "groupSize": 64}
    arch = {"hiddenSize": d, "ffnIntermediate": f, "moeIntermediateSize": f, "numHeads": 1, "numKVHeads": 1,
            "numFullKVHeads": 1, "headDim": 64, "fullHeadDim": 64, "vocabSize": 256, "slidingWindow": 0,
            "finalLogitSoftcap": 0.0, "ropeTheta": 10000.0, "fullRopeTheta": 10000.0, "partialRotaryFactor": 1.0,
            "numLayers": len(layers), "numExperts": n_experts, "topKExperts": top_k, "tieWordEmbeddings": True,
            "attentionKEqV": False, "hiddenActivation": "silu", "fullAttentionLayerMask": [0] * len(layers)}
    manifest = {"magic": MAGIC, "versionMajor": 1, "versionMinor": 0,
                "flags": {"streamingPresent": True, "turboQuantKV": False, "aneSharedExpert": False},
                "modelID": model_id, "arch": arch,
                "quant": {k: slot(8 if k == "router" else bits)
                          for k in ("embedding", "attention", "router", "sharedExpert", "routedExpert")},
                "files": files, "expertsPerLayer": n_experts, "numLayers": len(layers), "expertStride": stride}
    with open(os.path.join(root, "manifest.json"), "w") as fh:
        json.dump(manifest, fh, sort_keys=True)
