"""The reference test-suite's seed-derived inputs for the MoE path, regenerated.

The reference keeps no binary fixtures: every hot-path test draws its inputs
from SplitMix64 / SeedTree (or an LCG) and quantizes them with
`Quantization.quantizeInt4Affine/Int8Affine`.  The functions here restate those
set-ups draw for draw (order matters), plus the independent fp32 references the
reference's tests compare their kernels against
(sources/NVMAIValidation/Support/Reference).  Test infrastructure only.
"""
from __future__ import annotations

import numpy as np

from oracle import oracle as orc


def _f16(x: np.ndarray) -> np.ndarray:
    """Float(Float16(x))"""
    return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


def dequant_gemv_ref(bits: int, packed, scales, biases, x: np.ndarray, n: int) -> np.ndarray:
    """DequantInt4GemvRef / DequantInt8GemvRef (Reference/Quant/DequantInt4Gemv.swift:13-44):
    bulk-dequantize each row to fp32, then a plain dot product (vDSP_dotpr: order
    unspecified, carried in double here)."""
    rows = packed.shape[0]
    w = orc.dequant(bits, orc.META_BF16, packed, scales, biases, rows, n)
    return (w.astype(np.float64) @ np.asarray(x, dtype=np.float64)).astype(np.float32)


def gelu_tanh_ref(x: np.ndarray) -> np.ndarray:
    """MoeRef.geluTanh (Reference/MoE/Moe.swift:22-30), fp32."""
    x = x.astype(np.float32)
    inner = np.float32(0.7978845608028654) * (x + np.float32(0.044715) * x * x * x)
    return (np.float32(0.5) * x * (np.float32(1.0) + np.tanh(inner))).astype(np.float32)


def silu_ref(x: np.ndarray) -> np.ndarray:
    x = x.astype(np.float32)
    return (x / (np.float32(1.0) + np.exp(-x))).astype(np.float32)


# ---------------------------------------------------------------------------
# tests/NVMAI/Core/Kernels/MoE/RouterTopKTests.swift
# ---------------------------------------------------------------------------

def router_case(which: str) -> dict:
    E, D, K = 16, 128, 8
    if which == "production":      # RouterTopKTests.swift:17-31
        rng = orc.SplitMix64(0xA5B6_1234)
        weights = np.empty((E, D), dtype=np.float32)
        for e in range(E):
            weights[e] = rng.uniform_array(-0.05, 0.05, D) + np.float32(e) * np.float32(0.01)
        hidden = rng.uniform_array(-1.0, 1.0, D)
        inv_sqrt_d = np.float32(1.0) / np.sqrt(np.float32(D))
        eff = rng.uniform_array(0.5, 1.5, D) * inv_sqrt_d
        pes = rng.uniform_array(0.6, 1.4, E)
    elif which == "near_tie":      # RouterTopKTests.swift:46-61
        rng = orc.SplitMix64(0x71E_0F4A)
        pattern = rng.uniform_array(0.2, 1.0, D)
        hidden = rng.uniform_array(0.5, 1.5, D)
        gains = np.zeros(E, dtype=np.float32)
        for e in range(7):
            gains[e] = np.float32(1.0) - np.float32(e) * np.float32(0.05)
        gains[7] = 0.5
        gains[8] = np.float32(0.5) * (np.float32(1.0) + np.float32(1e-4))
        for e in range(9, E):
            gains[e] = np.float32(0.4) - np.float32(e - 9) * np.float32(0.02)
        weights = (gains[:, None] * pattern[None, :]).astype(np.float32)
        eff = np.ones(D, dtype=np.float32)
        pes = np.ones(E, dtype=np.float32)
    else:
        raise ValueError(which)
    packed, scales, biases = orc.quantize(8, weights)
    # the test's own reference (RouterTopKTests.swift:72-98): fp32 hidden*eff, DequantInt8GemvRef, sort
    logits = dequant_gemv_ref(8, packed, scales, biases, hidden * eff, D)
    order = sorted(range(E), key=lambda e: (-float(logits[e]), e))[:K]
    sel = logits[order]
    ex = np.exp(sel - sel[0]).astype(np.float32)
    ref_w = (ex / ex.sum(dtype=np.float32) * pes[order]).astype(np.float32)
    return dict(E=E, D=D, K=K, packed=packed, scales=scales, biases=biases,
                x_f16=orc.f32_to_f16_bits(hidden), eff_bf16=orc.f32_to_bf16_bits(eff),
                pes_bf16=orc.f32_to_bf16_bits(pes), ref_idx=np.array(order, dtype=np.uint32), ref_w=ref_w)


# ---------------------------------------------------------------------------
# tests/NVMAI/Core/Kernels/MoE/MoEFusedFFNTests.swift
# ---------------------------------------------------------------------------

def fused_production_case() -> dict:
    """MoEFusedFFNTests.swift:56-101: D=128, F=64, K=8, 4-bit, GELU (the `MoE(context:)` default)."""
    D, F, K = 128, 64, 8
    rng = orc.seedtree_key(0x2D3, "production-routed-moe")
    gates, ups, downs = [], [], []
    for _ in range(K):
        gates.append(rng.uniform_array(-0.4, 0.4, F * D).reshape(F, D))
        ups.append(rng.uniform_array(-0.4, 0.4, F * D).reshape(F, D))
        downs.append(rng.uniform_array(-0.4, 0.4, D * F).reshape(D, F))
    x = _f16(rng.uniform_array(-0.5, 0.5, D))
    residual = _f16(rng.uniform_array(-0.5, 0.5, D))
    routing_w = _f16(np.array([np.float32(0.04) + np.float32(i) * np.float32(0.015) for i in range(K)],
                              dtype=np.float32))
    off = orc.expert_offsets(D, F, 4)
    blobs = np.zeros((K, int(off[9])), dtype=np.uint8)
    expected = residual.copy()
    for k in range(K):
        q = [orc.quantize(4, m) for m in (gates[k], ups[k], downs[k])]
        for j, (w, s, b) in enumerate(q):
            for i, arr in enumerate((w, s, b)):
                raw = arr.view(np.uint8).ravel()
                o = int(off[j * 3 + i])
                blobs[k, o:o + raw.size] = raw
        # MoeRef.runFFN + applyStreamedRouted (Reference/MoE/Moe.swift:34-95)
        g = dequant_gemv_ref(4, *q[0], x, D)
        u = dequant_gemv_ref(4, *q[1], x, D)
        act = (gelu_tanh_ref(g) * u).astype(np.float32)
        out = dequant_gemv_ref(4, *q[2], act, F)
        expected = (expected + routing_w[k] * out).astype(np.float32)
    return dict(D=D, F=F, K=K, bits=4, blobs=blobs, off=off, x_f16=orc.f32_to_f16_bits(x),
                residual_f16=orc.f32_to_f16_bits(residual), w_f16=orc.f32_to_f16_bits(routing_w),
                expected=expected)


def constant_blob_case(bits: int = 8) -> dict:
    """MoEFusedFFNTests.swift:17-54, 238-270: zero codes, zero scales, bias-only
    weights (gate 1/64, up 0.5/64, down 1/64; bf16 by truncation), x = 1,
    routing weights 0.125 x 8, residual 0  =>  every output = silu(2)."""
    D, F, K = 128, 64, 8
    L = orc.lib()
    off = orc.expert_offsets(D, F, bits)
    blob = np.zeros(int(off[9]), dtype=np.uint8)

    def fill(o: int, value: float, count: int):
        raw = np.full(count, L.orc_f32_to_bf16_trunc(value), dtype=np.uint16).view(np.uint8)
        blob[o:o + raw.size] = raw

    fill(int(off[2]), 1.0 / 64.0, F * D // 64)
    fill(int(off[5]), 0.5 / 64.0, F * D // 64)
    fill(int(off[8]), 1.0 / 64.0, D * F // 64)
    blobs = np.tile(blob, (K, 1))
    return dict(D=D, F=F, K=K, bits=bits, blobs=blobs, off=off,
                x_f16=orc.f32_to_f16_bits(np.ones(D, dtype=np.float32)),
                residual_f16=np.zeros(D, dtype=np.uint16),
                w_f16=orc.f32_to_f16_bits(np.full(K, 0.125, dtype=np.float32)),
                expected=np.full(D, 2.0 / (1.0 + np.exp(-2.0)), dtype=np.float32))


# ---------------------------------------------------------------------------
# tests/NVMAI/Core/Kernels/CPU/CPUExpertFFNTests.swift
# ---------------------------------------------------------------------------

LCG_INC = 1_442_695_040_888_963_407


def _lcg_rows(count: int, n: int, seed: int):
    vals, _ = orc.lcg_array(seed, LCG_INC, count * n)     # CPUExpertFFNTests.swift:16-27
    return orc.quantize(4, vals.reshape(count, n))


def cpu_expert_case(seeds=(1, 2, 3), x_seed: int | None = 99) -> dict:
    """CPUExpertFFNTests.swift:69-113: gate/up/down rows from LCG seeds 1,2,3; x from
    state 99 with increment 1; expected = DequantInt4GemvRef chain with SiLU."""
    D, F = 128, 64
    gate, up, down = _lcg_rows(F, D, seeds[0]), _lcg_rows(F, D, seeds[1]), _lcg_rows(D, F, seeds[2])
    off = orc.expert_offsets(D, F, 4)
    blob = np.zeros(int(off[9]), dtype=np.uint8)
    for j, (w, s, b) in enumerate((gate, up, down)):
        for i, arr in enumerate((w, s, b)):
            raw = arr.view(np.uint8).ravel()
            o = int(off[j * 3 + i])
            blob[o:o + raw.size] = raw
    if x_seed is None:
        x = np.full(D, 0.05, dtype=np.float32)            # CPUExpertFFNTests.swift:124
    else:
        x, _ = orc.lcg_array(x_seed, 1, D)
    g = dequant_gemv_ref(4, *gate, x, D)
    u = dequant_gemv_ref(4, *up, x, D)
    act = (silu_ref(g) * u).astype(np.float32)
    expected = dequant_gemv_ref(4, *down, act, F)
    return dict(D=D, F=F, blob=blob, off=off, x=x, expected=expected)


# ---------------------------------------------------------------------------
# tests/NVMAI/Core/Kernels/MoE/SharedExpertInt4Tests.swift / SharedExpertInt8Tests.swift
# ---------------------------------------------------------------------------

def shared_expert_case(bits: int) -> dict:
    """SharedExpertInt4Tests.swift:11-53 (seed 0x604, "shared-expert-int4", GELU) and
    SharedExpertInt8Tests.swift:50-112 (seed 0x601, "shared-expert-int8")."""
    D, F = 128, 64
    if bits == 4:
        rng = orc.seedtree_key(0x604, "shared-expert-int4")
    else:
        rng = orc.seedtree_key(0x601, "shared-expert-int8")
    x = rng.uniform_array(-0.4, 0.4, D)
    gate = rng.uniform_array(-0.4, 0.4, F * D).reshape(F, D)
    up = rng.uniform_array(-0.4, 0.4, F * D).reshape(F, D)
    down = rng.uniform_array(-0.4, 0.4, D * F).reshape(D, F)
    q = [orc.quantize(bits, m) for m in (gate, up, down)]
    x16 = _f16(x)
    g = dequant_gemv_ref(bits, *q[0], x16, D)
    u = dequant_gemv_ref(bits, *q[1], x16, D)
    act = _f16(gelu_tanh_ref(g) * u)
    expected = dequant_gemv_ref(bits, *q[2], act, F)
    return dict(D=D, F=F, bits=bits, proj=q, x_f16=orc.f32_to_f16_bits(x), expected=expected)


# ---------------------------------------------------------------------------
# tests/NVMAI/Core/Kernels/Prefill/PrefillMoEGroupingTests.swift (literal tables)
# ---------------------------------------------------------------------------

def pairs_array(rows) -> np.ndarray:
    a = np.zeros(len(rows), dtype=orc.PAIR_DTYPE)
    for i, (t, e, r, w) in enumerate(rows):
        a[i] = (t, e, r, w)
    return a


GROUPING_TABLE_1 = dict(      # PrefillMoEGroupingTests.swift:5-53
    pairs=[(0, 3, 0, 10), (0, 1, 1, 11), (0, 4, 2, 12), (1, 1, 0, 13), (1, 3, 1, 14), (1, 2, 2, 15),
           (2, 4, 0, 16), (2, 3, 1, 17), (2, 1, 2, 18), (3, 5, 0, 19), (3, 1, 1, 20), (3, 4, 2, 21)][::-1],
    query_count=4, top_k=3, num_experts=6, tile=2,
    sorted_experts=[1, 1, 1, 1, 2, 3, 3, 3, 4, 4, 4, 5],
    sorted_token_rank=[[0, 1], [1, 0], [2, 2], [3, 1], [1, 2], [0, 0], [1, 1], [2, 1], [0, 2], [2, 0], [3, 2], [3, 0]],
    offsets=[0xFFFFFFFF, 0, 4, 5, 8, 11], counts=[0, 4, 1, 3, 3, 1],
    groups=[(1, 0, 4), (2, 4, 1), (3, 5, 3), (4, 8, 3), (5, 11, 1)],
    tiles=[(0, 2, 0, 5), (2, 2, 5, 6), (4, 1, 11, 1)])

GROUPING_TABLE_2 = dict(      # PrefillMoEGroupingTests.swift:55-82
    pairs=[(0, 2, 0, 101), (0, 1, 1, 102), (1, 2, 0, 103), (1, 0, 1, 104), (2, 1, 0, 105), (2, 2, 1, 106)],
    shuffle=[5, 1, 3, 0, 4, 2], query_count=3, top_k=2, num_experts=3, tile=2,
    sorted_weight_bits=[104, 102, 105, 101, 103, 106])

GROUPING_TABLE_3 = dict(      # PrefillMoEGroupingTests.swift:84-115
    pairs=[(0, 1, 0, 10), (0, 2, 1, 20), (1, 3, 0, 30), (1, 1, 1, 11), (2, 2, 0, 21), (2, 3, 1, 31)],
    query_count=3, top_k=2, num_experts=4, tile=2, sort_keys=[0, 30, 10, 20],
    group_experts=[2, 3, 1], sorted_experts=[2, 2, 3, 3, 1, 1], offsets=[0xFFFFFFFF, 4, 0, 2],
    tiles=[(0, 2, 0, 4), (2, 1, 4, 2)])


# ---------------------------------------------------------------------------
# tests/NVMAI/Core/Kernels/Quant/AffineQuantTests.swift:8-56
# ---------------------------------------------------------------------------

def affine_quant_case(bits: int) -> dict:
    """Codes (row*11 + column*3) & mask packed LSB-first, scale 1, bias 0, x = 1:
    every output is the integer sum of the row's codes."""
    rows, cols = 3, 128
    mask = (1 << bits) - 1
    values = np.array([[(r * 11 + c * 3) & mask for c in range(cols)] for r in range(rows)], dtype=np.uint32)
    packed = np.zeros((rows, cols * bits // 8), dtype=np.uint8)
    for r in range(rows):
        for c in range(cols):
            bit = c * bits
            packed[r, bit // 8] |= np.uint8((int(values[r, c]) << (bit % 8)) & 0xFF)
    one = np.uint16(np.float32(1.0).view(np.uint32) >> 16)
    scales = np.full((rows, cols // 64), one, dtype=np.uint16)
    biases = np.zeros((rows, cols // 64), dtype=np.uint16)
    return dict(bits=bits, rows=rows, cols=cols, packed=packed, scales=scales, biases=biases,
                x_f16=orc.f32_to_f16_bits(np.ones(cols, dtype=np.float32)),
                expected=values.sum(axis=1).astype(np.float32))


# ---------------------------------------------------------------------------
# tests/NVMAI/Core/Kernels/Primitives/RMSNormTests.swift
# ---------------------------------------------------------------------------

def rmsnorm_bf16w_case(d: int, seed: int) -> dict:
    """RMSNormTests.swift:22-55: x ~ U(-1, 1) rounded to fp16, weight ~ U(0.5, 1.5) rounded to bf16, eps 1e-6;
    the comparator is RmsNormRef.apply in its scalar form (RMSNormReferenceTests.swift:16-22), bar 5e-3."""
    rng = orc.seedtree_key(seed, f"rmsnorm-bf16w-d{d}")
    x32 = rng.uniform_array(-1.0, 1.0, d)
    w32 = rng.uniform_array(0.5, 1.5, d)
    x16 = x32.astype(np.float16)
    w_bits = orc.f32_to_bf16_bits(w32)
    x, w = x16.astype(np.float32), orc.bf16_bits_to_f32(w_bits)
    eps = np.float32(1e-6)
    sum_sq = np.float32(0.0)
    for v in x:
        sum_sq = np.float32(sum_sq + v * v)
    inv = np.float32(1.0) / np.sqrt(np.float32(sum_sq / np.float32(d) + eps))
    return {"x16": x16, "w_bits": w_bits, "eps": float(eps), "ref": (x * inv * w).astype(np.float32), "tol": 5e-3}
