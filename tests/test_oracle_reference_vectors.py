"""Pins the CPU oracle against the reference's own test material.

Each test restates one test of the reference's suite (file:line in the
docstring): same seed-derived inputs (tests/refvectors.py), same independent
fp32 reference, same tolerance.  Where the reference's test compares its GPU
kernel to that reference, the oracle's shader-semantics functions stand where the
kernel stood; where it drives the CPU path, both the reference's own C GEMV
(oracle/_ref) and the restated one are driven.
"""
import ctypes as C

import numpy as np
import pytest

import refvectors as rv
from oracle import oracle as orc


def _blob_ptrs(blobs: np.ndarray):
    return (C.c_void_p * blobs.shape[0])(*[blobs[k].ctypes.data for k in range(blobs.shape[0])])


def run_router(case):
    L = orc.lib()
    logits = np.zeros(case["E"], dtype=np.float32)
    L.orc_router_logits_affine(8, orc.META_BF16, orc.ptr(case["packed"]), orc.ptr(case["scales"]),
                               orc.ptr(case["biases"]), orc.ptr(case["x_f16"]), orc.ptr(case["eff_bf16"]),
                               case["E"], case["D"], orc.ptr(logits), None)
    idx = np.zeros(case["K"], dtype=np.uint32)
    w16 = np.zeros(case["K"], dtype=np.uint16)
    margin = np.zeros(1, dtype=np.float32)
    L.orc_topk_softmax(orc.ptr(logits), case["E"], case["K"], orc.ptr(case["pes_bf16"]), orc.ptr(idx),
                       orc.ptr(w16), None, orc.ptr(margin))
    return idx, orc.f16_bits_to_f32(w16), float(margin[0]), logits


def test_expert_offsets_production_stride():
    """CPUExpertFFNTests.swift:56-67"""
    o = orc.expert_offsets(2048, 512, 4)
    assert int(o[9]) == 1_769_472
    assert int(o[0]) == 0 and int(o[1]) == 524_288 and int(o[3]) == 589_824 and int(o[6]) == 1_179_648
    assert list(o[:9]) == sorted(o[:9])
    assert int(orc.expert_offsets(2048, 512, 8)[9]) == 3_342_336


def test_router_production_matches_reference():
    """RouterTopKTests.swift:17-44: indices exact, weights max-abs < 5e-3"""
    case = rv.router_case("production")
    idx, w, margin, _ = run_router(case)
    assert idx.tolist() == case["ref_idx"].tolist()
    assert np.max(np.abs(w - case["ref_w"])) < 5e-3
    assert margin > 0


def test_router_near_tie_resolves_like_reference():
    """RouterTopKTests.swift:46-70"""
    case = rv.router_case("near_tie")
    idx, _, _, _ = run_router(case)
    assert idx.tolist() == case["ref_idx"].tolist()


def test_topk_exact_tie_prefers_lower_index():
    """moe.metal:252-258 / RouterTopKTests.swift:86-88: score desc, index asc"""
    L = orc.lib()
    logits = np.array([1.0, 3.0, 3.0, 2.0, 3.0, 0.5, 2.0, 1.0, 0.0, 1.0], dtype=np.float32)
    idx = np.zeros(8, dtype=np.uint32)
    L.orc_topk_softmax(orc.ptr(logits), logits.size, 8, None, orc.ptr(idx), None, None, None)
    assert idx.tolist() == [1, 2, 4, 3, 6, 0, 7, 9]


def run_phases(case, act, active_splits=None, out_dtype=orc.OUT_FP16):
    L = orc.lib()
    K, D, F = case["K"], case["D"], case["F"]
    ptrs = _blob_ptrs(case["blobs"])
    acts = np.zeros(K * F, dtype=np.uint16)
    if active_splits is None:
        L.orc_gpu_phase1(ptrs, orc.ptr(case["off"]), case["bits"], orc.META_BF16, act, orc.ptr(case["x_f16"]),
                         D, F, K, None, 0, orc.OUT_FP16, orc.ptr(acts))
    else:
        for slots in active_splits:
            s = np.array(slots, dtype=np.uint32)
            L.orc_gpu_phase1(ptrs, orc.ptr(case["off"]), case["bits"], orc.META_BF16, act,
                             orc.ptr(case["x_f16"]), D, F, K, orc.ptr(s), s.size, orc.OUT_FP16, orc.ptr(acts))
    y = np.zeros(D, dtype=np.uint16)
    L.orc_gpu_phase2(ptrs, orc.ptr(case["off"]), case["bits"], orc.META_BF16, orc.ptr(acts),
                     orc.ptr(case["w_f16"]), orc.ptr(case["residual_f16"]), D, F, K, out_dtype, orc.ptr(y))
    return orc.f16_bits_to_f32(y), acts


def test_constant_blob_8bit_gives_silu_2():
    """MoEFusedFFNTests.swift:17-54: every output within 0.01 of 2/(1+e^-2)"""
    case = rv.constant_blob_case(8)
    y, _ = run_phases(case, orc.ACT_SILU)
    assert np.all(np.abs(y - case["expected"]) < 0.01)


def test_fused_production_and_hit_split():
    """MoEFusedFFNTests.swift:56-198: rel error < 1e-2 vs MoeRef; subset(0-3)+subset(4-7) == full"""
    case = rv.fused_production_case()
    full, acts_full = run_phases(case, orc.ACT_GELU_TANH)
    split, acts_split = run_phases(case, orc.ACT_GELU_TANH, active_splits=([0, 1, 2, 3], [4, 5, 6, 7]))
    assert np.array_equal(full, split) and np.array_equal(acts_full, acts_split)
    assert orc.rel_error(full, case["expected"]) < 1e-2


@pytest.mark.parametrize("use_ref", [True, False])
def test_cpu_expert_ffn_matches_reference(use_ref):
    """CPUExpertFFNTests.swift:69-113: |out - expected| <= 2e-4 * max(scale, 1)"""
    if use_ref and orc.ref_lib() is None:
        pytest.skip("oracle/_ref not built (reference checkout absent)")
    case = rv.cpu_expert_case()
    L = orc.lib()
    D, F = case["D"], case["F"]
    out = np.zeros(D, dtype=np.float32)
    scratch = np.zeros(2 * F + D, dtype=np.float32)
    fn = orc.ref_gemv4_ptr() if use_ref else C.cast(None, orc.GEMV4_FN)
    L.orc_cpu_expert_accumulate(orc.ptr(case["blob"]), orc.ptr(case["off"]), 4, orc.META_BF16, orc.ACT_SILU,
                                orc.ptr(case["x"]), D, F, 1.0, orc.ptr(scratch), orc.ptr(out), fn)
    scale = max(float(np.max(np.abs(case["expected"]))), 1.0)
    assert np.max(np.abs(out - case["expected"])) <= 2e-4 * scale


def test_cpu_expert_ffn_accumulates_scaled():
    """CPUExpertFFNTests.swift:117-152: 0.75 + 0.25 == 1.0 within 1e-4"""
    case = rv.cpu_expert_case(seeds=(7, 8, 9), x_seed=None)
    L = orc.lib()
    D, F = case["D"], case["F"]
    fn = orc.ref_gemv4_ptr()

    def run(weight, out):
        scratch = np.zeros(2 * F + D, dtype=np.float32)
        L.orc_cpu_expert_accumulate(orc.ptr(case["blob"]), orc.ptr(case["off"]), 4, orc.META_BF16,
                                    orc.ACT_SILU, orc.ptr(case["x"]), D, F, weight, orc.ptr(scratch),
                                    orc.ptr(out), fn)

    once = np.zeros(D, dtype=np.float32)
    run(1.0, once)
    twice = np.zeros(D, dtype=np.float32)
    run(0.75, twice)
    run(0.25, twice)
    scale = max(float(np.max(np.abs(once))), 1.0)
    assert np.max(np.abs(once - twice)) <= 1e-4 * scale


def test_ref_gemv_equals_restated_gemv_bitwise():
    """The restated portable GEMV (int4_affine_gemv.c:114-134) against the
    reference's own object on production-shaped rows: same bits when neither
    contracts a*b+c; within 1e-6 relative otherwise (the reference object is
    built -O3 with FMA contraction allowed)."""
    if orc.ref_lib() is None:
        pytest.skip("oracle/_ref not built")
    rng = np.random.default_rng(5)
    rows, n = 64, 2048
    w = rng.integers(0, 256, size=(rows, n // 2), dtype=np.uint8)
    s = orc.f32_to_bf16_bits(rng.uniform(0.005, 0.02, size=(rows, n // 64)).astype(np.float32))
    b = orc.f32_to_bf16_bits(rng.uniform(-0.08, 0.0, size=(rows, n // 64)).astype(np.float32))
    x = rng.normal(size=n).astype(np.float32)
    a = np.zeros(rows, dtype=np.float32)
    r = np.zeros(rows, dtype=np.float32)
    orc.lib().orc_affine_gemv_f32(4, orc.META_BF16, orc.ptr(w), orc.ptr(s), orc.ptr(b), orc.ptr(x), rows, n, orc.ptr(a))
    orc.ref_lib().nvmai_int4_affine_gemv(w.ctypes.data_as(orc.u8p), s.ctypes.data_as(orc.u16p),
                                         b.ctypes.data_as(orc.u16p), x.ctypes.data_as(orc.f32p), rows, n,
                                         r.ctypes.data_as(orc.f32p))
    assert orc.rel_error(a, r) < 1e-5


@pytest.mark.parametrize("bits", [4, 8])
def test_shared_expert_matches_affine_reference(bits):
    """SharedExpertInt4Tests.swift:11-53 (tol quantInt4*4) / SharedExpertInt8Tests.swift:50-112 (quantInt8*4)"""
    case = rv.shared_expert_case(bits)
    L = orc.lib()
    proj = (C.c_void_p * 9)(*[a.ctypes.data for t in case["proj"] for a in t])
    h1 = np.zeros(case["D"], dtype=np.uint16)
    L.orc_gpu_shared_expert(proj, bits, orc.META_BF16, orc.ACT_GELU_TANH, None, None, None, 0,
                            orc.ptr(case["x_f16"]), case["D"], case["F"], orc.OUT_FP16, orc.ptr(h1))
    tol = (1.5e-3 if bits == 4 else 1e-3) * 4
    assert orc.rel_error(orc.f16_bits_to_f32(h1), case["expected"]) < tol


@pytest.mark.parametrize("bits", [4, 8])
def test_affine_gemv_decodes_packed_codes_exactly(bits):
    """AffineQuantTests.swift:33-56: scale 1, bias 0, x = 1 -> integer row sums"""
    case = rv.affine_quant_case(bits)
    y = np.zeros(case["rows"], dtype=np.float32)
    orc.lib().orc_gpu_affine_gemv_f16(bits, orc.META_BF16, orc.ptr(case["packed"]), orc.ptr(case["scales"]),
                                      orc.ptr(case["biases"]), orc.ptr(case["x_f16"]), case["rows"],
                                      case["cols"], None, orc.ptr(y))
    assert np.array_equal(y, case["expected"])


def test_quantizer_nibble_layout_and_roundtrip():
    """QuantizationTests.swift:35-50 (low nibble = even index) and the 4-bit
    round-trip bound |w - w_hat| <= scale; constant groups reconstruct exactly
    (Quantization.swift:70-72)."""
    row = (np.arange(64, dtype=np.float32) - np.float32(31.5)).reshape(1, 64)
    packed, scales, biases = orc.quantize(4, row)
    scale = float(orc.bf16_bits_to_f32(scales)[0, 0])
    bias = float(orc.bf16_bits_to_f32(biases)[0, 0])
    lo, hi = int(packed[0, 0] & 0x0F), int(packed[0, 0] >> 4)
    assert abs(lo * scale + bias - row[0, 0]) <= scale + 1e-3
    assert abs(hi * scale + bias - row[0, 1]) <= scale + 1e-3
    deq = orc.dequant(4, orc.META_BF16, packed, scales, biases, 1, 64)
    assert np.max(np.abs(deq - row)) <= scale + 1e-3
    const = np.full((1, 64), 0.375, dtype=np.float32)
    p, s, b = orc.quantize(8, const)
    assert np.array_equal(orc.dequant(8, orc.META_BF16, p, s, b, 1, 64), const)


def _group(pairs, query_count, top_k, num_experts, tile, sort_keys=None):
    L = orc.lib()
    n = len(pairs)
    arr = rv.pairs_array(pairs)
    sorted_ = np.zeros(max(n, 1), dtype=orc.PAIR_DTYPE)
    offsets = np.zeros(num_experts, dtype=np.uint32)
    counts = np.zeros(num_experts, dtype=np.uint32)
    groups = np.zeros((max(n, 1), 3), dtype=np.uint32)
    tiles = np.zeros((max(n, 1), 4), dtype=np.uint32)
    ng, nt = C.c_size_t(0), C.c_size_t(0)
    keys = None if sort_keys is None else np.array(sort_keys, dtype=np.uint64)
    rc = L.orc_group_pairs(orc.ptr(arr), n, query_count, top_k, num_experts, tile, orc.ptr(keys),
                           0 if keys is None else keys.size, orc.ptr(sorted_), orc.ptr(offsets), orc.ptr(counts),
                           orc.ptr(groups), C.byref(ng), orc.ptr(tiles), C.byref(nt))
    return rc, sorted_[:n], offsets, counts, groups[:ng.value], tiles[:nt.value]


def test_grouping_literal_table():
    """PrefillMoEGroupingTests.swift:5-53"""
    t = rv.GROUPING_TABLE_1
    rc, s, off, cnt, groups, tiles = _group(t["pairs"], t["query_count"], t["top_k"], t["num_experts"], t["tile"])
    assert rc == 0
    assert s["expert"].tolist() == t["sorted_experts"]
    assert [[int(a), int(b)] for a, b in zip(s["token"], s["rank"])] == t["sorted_token_rank"]
    assert off.tolist() == t["offsets"] and cnt.tolist() == t["counts"]
    assert [tuple(g) for g in groups.tolist()] == t["groups"]
    assert [tuple(g) for g in tiles.tolist()] == t["tiles"]


def test_grouping_deterministic_under_shuffle():
    """PrefillMoEGroupingTests.swift:55-82"""
    t = rv.GROUPING_TABLE_2
    a = _group(t["pairs"], t["query_count"], t["top_k"], t["num_experts"], t["tile"])
    b = _group([t["pairs"][i] for i in t["shuffle"]], t["query_count"], t["top_k"], t["num_experts"], t["tile"])
    for x, y in zip(a[1:], b[1:]):
        assert np.array_equal(x, y)
    assert a[1]["weight_bits"].tolist() == t["sorted_weight_bits"]


def test_grouping_sort_key_override():
    """PrefillMoEGroupingTests.swift:84-115"""
    t = rv.GROUPING_TABLE_3
    rc, s, off, _, groups, tiles = _group(t["pairs"], t["query_count"], t["top_k"], t["num_experts"], t["tile"],
                                          t["sort_keys"])
    assert rc == 0
    assert groups[:, 0].tolist() == t["group_experts"]
    assert s["expert"].tolist() == t["sorted_experts"]
    assert off.tolist() == t["offsets"]
    assert [tuple(g) for g in tiles.tolist()] == t["tiles"]


def test_grouping_rejects_invalid_metadata():
    """PrefillMoEGroupingTests.swift:117-173: tile count 17, expert out of range,
    duplicate (token, rank), sort-key count mismatch"""
    assert _group([(0, 0, 0, 1)], 1, 1, 1, 17)[0] == 4
    assert _group([(0, 2, 0, 1)], 1, 1, 2, 1)[0] == 8
    assert _group([(0, 0, 0, 1), (0, 1, 0, 2)], 1, 2, 2, 1)[0] == 9
    assert _group([(0, 0, 0, 1)], 1, 1, 2, 1, sort_keys=[0])[0] == 10


@pytest.mark.parametrize("d,seed", [(256, 0xC3), (2048, 0xD4)])
def test_rmsnorm_bf16w_oracle_on_reference_vectors(d, seed):
    """RMSNormTests.swift:22-61: the oracle's rmsnorm_bf16w against RmsNormRef on the reference's seed-derived inputs,
    at the reference's bar (Tolerance.fp16Reduction); fp16 rounding of the output is the only difference, so half an
    ulp is the real distance"""
    case = rv.rmsnorm_bf16w_case(d, seed)
    out = np.zeros(d, dtype=np.uint16)
    orc.lib().orc_gpu_rmsnorm_bf16w(orc.ptr(case["x16"].view(np.uint16)), orc.ptr(case["w_bits"]), orc.ptr(out), d,
                                    case["eps"], 0)
    got = orc.f16_bits_to_f32(out)
    assert orc.rel_error(got, case["ref"]) < case["tol"]
    assert np.max(np.abs(got - case["ref"]) / np.maximum(np.abs(case["ref"]), 1e-3)) < 1.0 / 1024


def test_rmsnorm_closed_form():
    """x = (3, 4) repeated, w = 1: mean square 12.5, so out = x / sqrt(12.5) up to fp16 rounding"""
    x = np.tile(np.array([3.0, 4.0], dtype=np.float16), 32)
    w = orc.f32_to_bf16_bits(np.ones(64, dtype=np.float32))
    out = np.zeros(64, dtype=np.uint16)
    orc.lib().orc_gpu_rmsnorm_bf16w(orc.ptr(x.view(np.uint16)), orc.ptr(w), orc.ptr(out), 64, 0.0, 0)
    want = (x.astype(np.float32) / np.float32(np.sqrt(12.5))).astype(np.float16)
    assert np.array_equal(out.view(np.float16), want)
