"""`.gturbo` packed-expert artifacts: layout / manifest validation (the rules of GTurboV1StructuralValidator and
GTurboManifestCodec restated), the copy plan that honours physicalRank, and the SHA-256 check.  CPU only; the read
into device memory is a GPU test."""
import copy
import json

import numpy as np
import pytest

from nvmai_b200 import format as fmt
from nvmai_b200 import gturbo

D, F, E, BITS = 128, 64, 8, 4


def _blobs(seed):
    _, n = fmt.expert_offsets(D, F, BITS)
    return np.random.default_rng(seed).integers(0, 256, size=(E, n), dtype=np.uint8)


@pytest.fixture()
def artifact(tmp_path):
    layers = [_blobs(1), _blobs(2)]
    ranks = [np.arange(E), np.array([3, 4, 5, 0, 7, 6, 1, 2])]
    gturbo.write_packed_experts(tmp_path, layers, d=D, f=F, bits=BITS, physical_ranks=ranks)
    return tmp_path, layers, ranks


def test_open_reads_offsets_ranks_and_quantisation(artifact):
    root, layers, ranks = artifact
    g = gturbo.GTurboExperts(root)
    off, blob = fmt.expert_offsets(D, F, BITS)
    assert g.layout.expert_stride == 16384 * ((blob + 16383) // 16384) and g.layer_bytes == E * g.layout.expert_stride
    assert g.layout.expert_offsets(1) == off
    assert g.layout.physical_offsets(1).tolist() == (ranks[1] * g.layout.expert_stride).tolist()
    assert g.routed_bits() == 4 and g.meta_dtype() == fmt.META_BF16
    g.verify_layer(0); g.verify_layer(1)


def test_copy_plan_puts_blobs_in_logical_order(artifact):
    root, layers, ranks = artifact
    g = gturbo.GTurboExperts(root)
    s = g.layout.expert_stride
    assert g.copy_plan(0) == [(0, 0, E * s)]                      # identity mapping: one read
    plan = g.copy_plan(1)
    assert plan == [(3 * s, 0, 3 * s), (0, 3 * s, s), (7 * s, 4 * s, s), (6 * s, 5 * s, s), (1 * s, 6 * s, 2 * s)]
    raw = np.fromfile(g.layer_path(1), dtype=np.uint8)
    got = np.zeros(E * s, dtype=np.uint8)
    for src, dst, n in plan:
        got[dst:dst + n] = raw[src:src + n]
    blob = layers[1].shape[1]
    assert np.array_equal(got.reshape(E, s)[:, :blob], layers[1])


def test_corrupted_layer_file_fails_the_digest(artifact):
    root, _, _ = artifact
    g = gturbo.GTurboExperts(root)
    path = g.layer_path(0)
    raw = np.fromfile(path, dtype=np.uint8)
    raw[12345] ^= 1
    raw.tofile(path)
    with pytest.raises(gturbo.GTurboFormatError) as ei:
        g.verify_layer(0)
    assert "digest" in ei.value.reason
    raw[:-1].tofile(path)
    with pytest.raises(gturbo.GTurboFormatError) as ei:
        g.verify_layer(0)
    assert "size" in ei.value.reason


def _layout(artifact):
    with open(artifact[0] / "packed_experts" / "layout.json") as fh:
        return json.load(fh)


def _mut(obj, fn):
    o = copy.deepcopy(obj)
    fn(o)
    return o


LAYOUT_CASES = [
    (lambda o: o.update(expertStride=o["expertStride"] + 64), "invalid dimensions or stride"),
    (lambda o: o["layers"].pop(), "invalid dimensions or stride"),
    (lambda o: o["layers"][1].update(layer=0), "duplicate or invalid layer"),
    (lambda o: o["layers"][1].update(file="sub/layer_01.bin"), "plain file name"),
    (lambda o: o["layers"][1].update(file="Layout.JSON"), "reserved"),
    (lambda o: o["layers"][1].update(file="LAYER_00.bin"), "duplicate layer filename"),
    (lambda o: o["layers"][0]["experts"].pop(), "wrong expert count"),
    (lambda o: o["layers"][0]["experts"][2].pop("expert"), "all explicit or all positional"),
    (lambda o: o["layers"][0]["experts"][2].update(expert=1), "duplicate or invalid expert mapping"),
    (lambda o: o["layers"][1]["experts"][2].update(physicalRank=9), "duplicate or invalid expert mapping"),
    (lambda o: o["layers"][0]["experts"][2].update(offset=0), "duplicate or invalid expert mapping"),
    (lambda o: o["layers"][0]["experts"][2].update(offset=o["expertStride"] * 2 + 16384 * 64), "does not match physical rank"),
    (lambda o: o["layers"][0]["experts"][2].update(size=5), "does not match physical rank"),
    (lambda o: o["layers"][0]["experts"][0]["tensors"]["gate"].update(dtype="F32"), "invalid dtype or shape"),
    (lambda o: o["layers"][0]["experts"][0]["tensors"]["gate"].update(bits=33), "invalid dtype or shape"),
    (lambda o: o["layers"][0]["experts"][0]["tensors"]["down_biases"].update(size=1 << 20), "range exceeds expert blob"),
    (lambda o: o["layers"][0]["experts"][0]["tensors"]["up"].update(offset=8), "overlapping ranges"),
]


@pytest.mark.parametrize("case", range(len(LAYOUT_CASES)))
def test_layout_validator_rejects(artifact, case):
    fn, reason = LAYOUT_CASES[case]
    bad = _mut(_layout(artifact), fn)
    with pytest.raises(gturbo.GTurboFormatError) as ei:
        gturbo.decode_layout(json.dumps(bad))
    assert reason in ei.value.reason


MANIFEST_CASES = [
    (lambda m: m.update(magic="GTURB0"), "expected GTURBO"),
    (lambda m: m.update(versionMajor=2), "unsupported version"),
    (lambda m: m["flags"].update(newFlag=True), "unknown v1 flag"),
    (lambda m: m.update(expertStride=1000), "invalid dimensions or stride"),
    (lambda m: m["arch"].update(numExperts=4), "disagree with streaming metadata"),
    (lambda m: m["arch"].update(topKExperts=99), "invalid architecture values"),
    (lambda m: m["quant"]["routedExpert"].update(weightBits=0), "invalid quantization values"),
    (lambda m: m["files"].update({"../evil.bin": {"size": 1, "sha256": "0" * 64}}), "relative path"),
    (lambda m: m["files"].update({"Packed_Experts/LAYER_00.bin": {"size": 1, "sha256": "0" * 64}}), "duplicate path"),
    (lambda m: m["files"].update({"tokenizer": {"size": 1, "sha256": "0" * 64}}), "reserved artifact filename"),
    (lambda m: m["files"]["packed_experts/layer_00.bin"].update(sha256="abc"), "64 hexadecimal"),
]


@pytest.mark.parametrize("case", range(len(MANIFEST_CASES)))
def test_manifest_validator_rejects(artifact, case):
    fn, reason = MANIFEST_CASES[case]
    with open(artifact[0] / "manifest.json") as fh:
        bad = _mut(json.load(fh), fn)
    with pytest.raises(gturbo.GTurboFormatError) as ei:
        gturbo.decode_manifest(json.dumps(bad))
    assert reason in ei.value.reason


def test_cross_validation_needs_matching_dimensions_and_layer_sizes(artifact):
    root = artifact[0]
    with open(root / "manifest.json") as fh:
        m = json.load(fh)
    layout = gturbo.decode_layout(json.dumps(_layout(artifact)))
    gturbo.cross_validate(gturbo.decode_manifest(json.dumps(m)), layout)
    m2 = copy.deepcopy(m); m2["files"]["packed_experts/layer_01.bin"]["size"] -= 1
    with pytest.raises(gturbo.GTurboFormatError) as ei:
        gturbo.cross_validate(gturbo.decode_manifest(json.dumps(m2)), layout)
    assert "missing or wrong layer size" in ei.value.reason
    m3 = copy.deepcopy(m); m3["expertStride"] *= 2
    with pytest.raises(gturbo.GTurboFormatError) as ei:
        gturbo.cross_validate(gturbo.decode_manifest(json.dumps(m3)), layout)
    assert "dimension mismatch" in ei.value.reason


def test_positional_expert_ids_are_accepted(artifact):
    lay = _layout(artifact)
    for e in lay["layers"][0]["experts"]:
        e.pop("expert")
    out = gturbo.decode_layout(json.dumps(lay))
    assert out.layers[0]["physical"].tolist() == list(range(E))
