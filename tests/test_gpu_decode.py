"""GPU parity tests of the decode path, through the C ABI, against the CPU oracle
and the reference's regenerated test vectors.

Bars: expert indices bit-exact; dequantised weights bit-exact; FFN outputs
within 1e-3 (RelError, sources/NVMAIValidation/Support/Tolerance/RelError.swift:4-16)
of the reference CPU path; the reference's own per-test tolerances where a test
of the reference is restated.
"""
import numpy as np
import pytest

import gpu_util as gu
import refvectors as rv
from nvmai_b200 import Elementwise, MoE, MoEConfig, affine_gemv, dequant, synthetic
from nvmai_b200 import format as fmt
from oracle import oracle as orc

pytestmark = pytest.mark.gpu

FFN_TOL = 1e-3      # north-star bar vs the reference CPU path, fp32 accumulation


def sync():
    gu.torch_cuda().cuda.synchronize()


# ---------------------------------------------------------------------------
# dequantisation: bit-exact
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("meta", [fmt.META_BF16, fmt.META_FP16])
def test_dequant_bit_exact(bits, meta):
    rng = np.random.default_rng(100 + bits + meta)
    rows, n = 96, 512
    w, s, b = synthetic.affine_tensor(rng, rows, n, bits, meta)
    out = gu.dev_empty(rows * n, "f32")
    dequant(bits, meta, gu.to_dev(w), gu.to_dev(s), gu.to_dev(b), rows, n, out)
    sync()
    got = out.cpu().numpy().reshape(rows, n)
    want = orc.dequant(bits, meta, w, s, b, rows, n)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("bits", [4, 8])
def test_dequant_of_reference_quantizer_output_bit_exact(bits):
    """weights quantised by the restated Quantization.quantizeInt*Affine"""
    rng = orc.SplitMix64(0xD0 + bits)
    wf = rng.uniform_array(-0.4, 0.4, 32 * 256).reshape(32, 256)
    w, s, b = orc.quantize(bits, wf)
    out = gu.dev_empty(32 * 256, "f32")
    dequant(bits, fmt.META_BF16, gu.to_dev(w), gu.to_dev(s), gu.to_dev(b), 32, 256, out)
    sync()
    want = orc.dequant(bits, orc.META_BF16, w, s, b, 32, 256)
    assert np.array_equal(out.cpu().numpy().reshape(32, 256).view(np.uint32), want.view(np.uint32))


# ---------------------------------------------------------------------------
# generic GEMV + elementwise
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("bits", [4, 8])
def test_affine_gemv_decodes_packed_codes_exactly(bits):
    """AffineQuantTests.swift:33-56"""
    case = rv.affine_quant_case(bits)
    y = gu.dev_empty(8, "f16")
    affine_gemv(bits, fmt.META_BF16, gu.to_dev(case["packed"]), gu.to_dev(case["scales"]),
                gu.to_dev(case["biases"]), gu.to_dev(case["x_f16"]), y, case["rows"], case["cols"])
    sync()
    got = orc.f16_bits_to_f32(gu.from_dev(y, np.uint16)[:case["rows"]])
    assert orc.rel_error(got, case["expected"]) < 0.002
    assert np.array_equal(got, case["expected"].astype(np.float16).astype(np.float32))


@pytest.mark.parametrize("bits,m,n", [(4, 512, 2048), (8, 2048, 512), (8, 1, 2048)])
def test_affine_gemv_matches_oracle(bits, m, n):
    """DequantInt4GEMVTests / DequantInt8GEMVTests sweep shapes, incl. the m = 1 scalar gate."""
    rng = np.random.default_rng(7 * bits + m)
    w, s, b = synthetic.affine_tensor(rng, m, n, bits, fmt.META_BF16)
    x = fmt.f32_to_f16_bits(rng.normal(size=n))
    y = gu.dev_empty(max(m, 8), "f16")
    affine_gemv(bits, fmt.META_BF16, gu.to_dev(w), gu.to_dev(s), gu.to_dev(b), gu.to_dev(x), y, m, n)
    sync()
    want = np.zeros(m, dtype=np.float32)
    orc.lib().orc_gpu_affine_gemv_f16(bits, orc.META_BF16, orc.ptr(w), orc.ptr(s), orc.ptr(b), orc.ptr(x), m, n,
                                      None, orc.ptr(want))
    got = orc.f16_bits_to_f32(gu.from_dev(y, np.uint16)[:m])
    assert orc.rel_error(got, want) < 5e-3          # Tolerance.fp16Reduction


def test_elementwise_kernels_bit_exact():
    """utility.metal:32-44, 60-70, 94-103"""
    rng = np.random.default_rng(3)
    n = 2048
    a = rng.normal(size=n).astype(np.float16)
    b = rng.normal(size=n).astype(np.float16)
    g = np.array([0.37], dtype=np.float16)
    da, db = gu.to_dev(a.view(np.uint16)), gu.to_dev(b.view(np.uint16))
    out = gu.dev_empty(n, "f16")
    Elementwise.encode_silu_mul(da, db, out, n)
    sync()
    af, bf = a.astype(np.float32), b.astype(np.float32)
    got = gu.from_dev(out, np.float16).astype(np.float32)
    want = ((af / (1 + np.exp(-af))) * bf).astype(np.float16).astype(np.float32)
    assert np.max(np.abs(got - want)) <= np.max(np.abs(want)) * 2 ** -10   # expf differs by an ulp at most
    hid = gu.to_dev(a.view(np.uint16).copy())
    Elementwise.encode_residual_add(hid, db, n)
    sync()
    assert np.array_equal(gu.from_dev(hid, np.float16), (af + bf).astype(np.float16))
    y = gu.to_dev(a.view(np.uint16).copy())
    Elementwise.encode_sigmoid_scalar_mul(y, gu.to_dev(g.view(np.uint16)), n)
    sync()
    want = (af / (1 + np.exp(-np.float32(g[0])))).astype(np.float16).astype(np.float32)
    assert np.max(np.abs(gu.from_dev(y, np.float16).astype(np.float32) - want)) <= np.max(np.abs(want)) * 2 ** -10


# ---------------------------------------------------------------------------
# router
# ---------------------------------------------------------------------------

def _router_moe(case, tokens=1):
    cfg = MoEConfig(d=case["D"], f=64, shared_f=0, num_experts=case["E"], top_k=case["K"], routed_bits=4,
                    shared_bits=4, router_kind=fmt.ROUTER_AFFINE8, shared_gate_kind=fmt.GATE_NONE,
                    meta_dtype=fmt.META_BF16, max_tokens=tokens)
    moe = MoE(cfg)
    off, stride = fmt.expert_offsets(cfg.d, cfg.f, 4)
    dummy = gu.dev_empty(stride * cfg.num_experts, "u8")
    keep = dict(experts=dummy, router=(gu.to_dev(case["packed"]), gu.to_dev(case["scales"]), gu.to_dev(case["biases"])),
                eff=gu.to_dev(case["eff_bf16"]), pes=gu.to_dev(case["pes_bf16"]))
    moe.register_layer(0, experts=dummy, expert_stride=stride, offsets=off, router=keep["router"],
                       effective_scale=keep["eff"], per_expert_scale=keep["pes"])
    return moe, keep


@pytest.mark.parametrize("which", ["production", "near_tie"])
def test_router_matches_reference(which):
    """RouterTopKTests.swift:17-70: indices exactly equal, weights max-abs < 5e-3"""
    case = rv.router_case(which)
    moe, keep = _router_moe(case)
    idx, w = gu.dev_empty(8, "u32"), gu.dev_empty(8, "f16")
    moe.encode_router(0, gu.to_dev(case["x_f16"]), idx, w)
    sync()
    assert gu.from_dev(idx, np.uint32).tolist() == case["ref_idx"].tolist()
    if which == "production":
        got = orc.f16_bits_to_f32(gu.from_dev(w, np.uint16))
        assert np.max(np.abs(got - case["ref_w"])) < 5e-3


def test_router_block_equals_repeated_decode_router_and_leaves_padding():
    """PrefillRouterTests.swift:33-101: T strided rows == T single-row calls; padding untouched"""
    case = rv.router_case("production")
    T, stride = 5, 192
    moe, keep = _router_moe(case, tokens=T)
    rng = orc.SplitMix64(0xBEEF)
    rows = np.full((T, stride), 0x7BFF, dtype=np.uint16)      # sentinel padding
    for t in range(T):
        rows[t, :case["D"]] = orc.f32_to_f16_bits(rng.uniform_array(-1.0, 1.0, case["D"]))
    xd = gu.to_dev(rows)
    sentinel = 0x5A5A5A5A
    idx = gu.to_dev(np.full(T * 8 + 8, sentinel, dtype=np.uint32))
    w = gu.to_dev(np.full(T * 8 + 8, 0x1234, dtype=np.uint16))
    moe.encode_router(0, xd, idx, w, tokens=T, x_stride=stride)
    sync()
    got_idx = gu.from_dev(idx, np.uint32)
    got_w = gu.from_dev(w, np.uint16)
    assert np.all(got_idx[T * 8:] == sentinel) and np.all(got_w[T * 8:] == 0x1234)
    for t in range(T):
        i1, w1 = gu.dev_empty(8, "u32"), gu.dev_empty(8, "f16")
        moe.encode_router(0, gu.to_dev(rows[t, :case["D"]].copy()), i1, w1)
        sync()
        assert np.array_equal(gu.from_dev(i1, np.uint32), got_idx[t * 8:(t + 1) * 8])
        assert np.array_equal(gu.from_dev(w1, np.uint16), got_w[t * 8:(t + 1) * 8])


# ---------------------------------------------------------------------------
# routed phase 1 / phase 2 against the reference's fused-FFN tests
# ---------------------------------------------------------------------------

def _phase_moe(case, act, out_dtype=fmt.OUT_FP16):
    cfg = MoEConfig(d=case["D"], f=case["F"], shared_f=0, num_experts=8, top_k=8, routed_bits=case["bits"],
                    shared_bits=4, router_kind=fmt.ROUTER_AFFINE8, shared_gate_kind=fmt.GATE_NONE,
                    meta_dtype=fmt.META_BF16, activation=act, out_dtype=out_dtype, max_tokens=1)
    return MoE(cfg)


def _run_phases(moe, case, splits=None):
    blobs_dev = gu.to_dev(case["blobs"])
    stride = case["blobs"].shape[1]
    blobs = [blobs_dev.data_ptr() + k * stride for k in range(case["K"])]
    off = dict(zip(fmt.OFFSET_NAMES, [int(v) for v in case["off"][:9]]))
    x = gu.to_dev(case["x_f16"])
    acts = gu.dev_empty(case["K"] * case["F"], "f16")
    if splits is None:
        moe.encode_routed_phase1(blobs, off, x, acts)
    else:
        for slots in splits:
            moe.encode_routed_phase1(blobs, off, x, acts, active_slots=slots)
    y = gu.dev_empty(case["D"], "f16")
    moe.encode_routed_phase2(blobs, off, acts, gu.to_dev(case["w_f16"]), gu.to_dev(case["residual_f16"]), y)
    sync()
    return gu.from_dev(y, np.uint16), gu.from_dev(acts, np.uint16), blobs_dev


def test_constant_blob_8bit_gives_silu_2():
    """MoEFusedFFNTests.swift:17-54"""
    case = rv.constant_blob_case(8)
    y, _, _ = _run_phases(_phase_moe(case, fmt.ACT_SILU), case)
    assert np.all(np.abs(orc.f16_bits_to_f32(y) - case["expected"]) < 0.01)


def test_fused_production_pipeline_and_hit_split():
    """MoEFusedFFNTests.swift:56-198: < 1e-2 vs MoeRef; subset(0-3)+subset(4-7) bit-identical to full"""
    case = rv.fused_production_case()
    moe = _phase_moe(case, fmt.ACT_GELU_TANH)
    full, acts_full, _ = _run_phases(moe, case)
    split, acts_split, _ = _run_phases(moe, case, splits=([0, 1, 2, 3], [4, 5, 6, 7]))
    assert np.array_equal(full, split) and np.array_equal(acts_full, acts_split)
    assert orc.rel_error(orc.f16_bits_to_f32(full), case["expected"]) < 1e-2
    # and against the oracle's shader-semantics restatement
    import test_oracle_reference_vectors as t
    want, want_acts = t.run_phases(case, orc.ACT_GELU_TANH)
    assert orc.rel_error(orc.f16_bits_to_f32(acts_full), orc.f16_bits_to_f32(want_acts)) < 1e-3
    assert orc.rel_error(orc.f16_bits_to_f32(full), want) < 2e-3


# ---------------------------------------------------------------------------
# shared expert
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("bits", [4, 8])
def test_shared_expert_matches_affine_reference(bits):
    """SharedExpertInt4Tests.swift:11-53 / SharedExpertInt8Tests.swift:50-112"""
    case = rv.shared_expert_case(bits)
    cfg = MoEConfig(d=case["D"], f=64, shared_f=case["F"], num_experts=8, top_k=8, routed_bits=4, shared_bits=bits,
                    router_kind=fmt.ROUTER_DENSE_F16, shared_gate_kind=fmt.GATE_NONE, meta_dtype=fmt.META_BF16,
                    activation=fmt.ACT_GELU_TANH, max_tokens=1)
    moe = MoE(cfg)
    off, stride = fmt.expert_offsets(cfg.d, cfg.f, 4)
    dummy = gu.dev_empty(stride * 8, "u8")
    router = (gu.dev_empty(8 * cfg.d, "f16"), None, None)
    shared = [gu.dev_tensor3(t) for t in case["proj"]]
    moe.register_layer(0, experts=dummy, expert_stride=stride, offsets=off, router=router, shared=shared)
    h1 = gu.dev_empty(cfg.d, "f16")
    moe.encode_shared_expert(0, gu.to_dev(case["x_f16"]), h1)
    sync()
    got = orc.f16_bits_to_f32(gu.from_dev(h1, np.uint16))
    tol = (1.5e-3 if bits == 4 else 1e-3) * 4
    assert orc.rel_error(got, case["expected"]) < tol


# ---------------------------------------------------------------------------
# whole layer at the benchmark shape
# ---------------------------------------------------------------------------

def _layer_case(bits, meta, out_dtype, tokens, seed, router_kind=fmt.ROUTER_DENSE_F16,
                gate_kind=fmt.ROUTER_DENSE_F16, d=2048, f=512, e=256):
    host = synthetic.layer(seed, d=d, f=f, shared_f=f, num_experts=e, routed_bits=bits, meta=meta,
                           router_kind=router_kind, gate_kind=gate_kind)
    cfg = MoEConfig(d=d, f=f, shared_f=f, num_experts=e, top_k=8, routed_bits=bits, shared_bits=bits,
                    router_kind=router_kind, shared_gate_kind=gate_kind, meta_dtype=meta,
                    activation=fmt.ACT_SILU, out_dtype=out_dtype, max_tokens=tokens)
    return host, cfg


def _check_layer(host, cfg, tokens, seed, tol_gpu_oracle):
    moe = MoE(cfg)
    dl = gu.DeviceLayer(host)
    dl.register(moe, 0)
    x = synthetic.hidden_rows(seed + 1, tokens, cfg.d)
    esz = "f16" if cfg.out_dtype == fmt.OUT_FP16 else "f32"
    h2 = gu.dev_empty(tokens * cfg.d, esz)
    idx, w = gu.dev_empty(tokens * 8, "u32"), gu.dev_empty(tokens * 8, "f16")
    moe.layer_decode(0, gu.to_dev(x), tokens, h2_out=h2, out_idx=idx, out_w=w)
    sync()
    got_idx = gu.from_dev(idx, np.uint32).reshape(tokens, 8)
    got_w = gu.from_dev(w, np.uint16).reshape(tokens, 8)
    if cfg.out_dtype == fmt.OUT_FP16:
        got = orc.f16_bits_to_f32(gu.from_dev(h2, np.uint16)).reshape(tokens, cfg.d)
    else:
        got = h2.cpu().numpy().reshape(tokens, cfg.d)
    L, keep = gu.oracle_layer(host, cfg)
    for t in range(tokens):
        o_idx, o_w, o_h2, margin, cpu = gu.oracle_decode(L, cfg, np.ascontiguousarray(x[t]))
        assert margin > 1e-5, f"router decision margin {margin} too small for an exact-index test: change the seed"
        assert got_idx[t].tolist() == o_idx.tolist()
        assert np.max(np.abs(orc.f16_bits_to_f32(got_w[t]) - orc.f16_bits_to_f32(o_w))) < 1e-3
        assert np.all(np.isfinite(got[t]))
        assert orc.rel_error(got[t], cpu) < FFN_TOL, "vs the reference CPU path"
        assert orc.rel_error(got[t], o_h2) < tol_gpu_oracle, "vs the shader-semantics oracle"
    return moe, dl, got


@pytest.mark.parametrize("bits,meta", [(4, fmt.META_FP16), (4, fmt.META_BF16), (8, fmt.META_FP16), (8, fmt.META_BF16)])
def test_layer_decode_benchmark_shape_fp32_out(bits, meta):
    """configs[0] / configs[1] (B = 1): D 2048, 256 experts, top-8, F 512, shared expert + sigmoid gate"""
    host, cfg = _layer_case(bits, meta, fmt.OUT_FP32, 1, seed=11 * bits + meta)
    _check_layer(host, cfg, 1, seed=50 + bits, tol_gpu_oracle=5e-4)


def test_layer_decode_reference_format_fp16_out():
    """the drop-in configuration: bf16 meta, affine 8-bit router and gate, fp16 rounding points"""
    host, cfg = _layer_case(4, fmt.META_BF16, fmt.OUT_FP16, 1, seed=77, router_kind=fmt.ROUTER_AFFINE8,
                            gate_kind=fmt.ROUTER_AFFINE8)
    _check_layer(host, cfg, 1, seed=78, tol_gpu_oracle=2e-3)     # one fp16 ulp of the output


@pytest.mark.parametrize("tokens,grouped_min", [(2, None), (4, None), (16, None), (64, None), (4, 4), (16, 4)])
def test_layer_decode_batch(tokens, grouped_min, monkeypatch):
    """configs[1]: independent rows, 8-bit.  Small batches run every row's blocks separately; from 24 rows on
    (or from NVMAI_CUDA_GROUPED_MIN on) rows that picked the same expert are grouped and share one read of its weights"""
    if grouped_min is not None:
        monkeypatch.setenv("NVMAI_CUDA_GROUPED_MIN", str(grouped_min))
    host, cfg = _layer_case(8, fmt.META_FP16, fmt.OUT_FP32, tokens, seed=5)
    _check_layer(host, cfg, tokens, seed=6 + tokens, tol_gpu_oracle=5e-4)


def test_layer_decode_batch_4bit_reference_rounding(monkeypatch):
    """grouped path with the reference's fp16 rounding points and a ragged batch (11 rows)"""
    monkeypatch.setenv("NVMAI_CUDA_GROUPED_MIN", "4")
    host, cfg = _layer_case(4, fmt.META_BF16, fmt.OUT_FP16, 11, seed=15, router_kind=fmt.ROUTER_AFFINE8,
                            gate_kind=fmt.ROUTER_AFFINE8)
    _check_layer(host, cfg, 11, seed=16, tol_gpu_oracle=2e-3)


def test_batched_result_equals_row_by_row(monkeypatch):
    """grouping must not change a row's result: batch of 9 == nine single-row calls, bitwise"""
    monkeypatch.setenv("NVMAI_CUDA_GROUPED_MIN", "4")
    host, cfg = _layer_case(4, fmt.META_BF16, fmt.OUT_FP32, 9, seed=41, d=256, f=128, e=32)
    moe = MoE(cfg)
    dl = gu.DeviceLayer(host)
    dl.register(moe, 0)
    x = synthetic.hidden_rows(42, 9, cfg.d)
    xd = gu.to_dev(x)
    batch = gu.dev_empty(9 * cfg.d, "f32")
    moe.layer_decode(0, xd, 9, h2_out=batch)
    sync()
    got = batch.cpu().numpy().reshape(9, cfg.d)
    for t in range(9):
        one = gu.dev_empty(cfg.d, "f32")
        moe.layer_decode(0, xd.data_ptr() + t * cfg.d * 2, 1, h2_out=one)
        sync()
        assert np.array_equal(one.cpu().numpy().view(np.uint32), got[t].view(np.uint32)), f"row {t}"


def test_layer_decode_small_shape_and_determinism():
    """D=128, F=64, 16 experts (every element checked), run twice: bitwise equal"""
    host, cfg = _layer_case(4, fmt.META_BF16, fmt.OUT_FP32, 3, seed=9, d=128, f=64, e=16,
                            router_kind=fmt.ROUTER_AFFINE4, gate_kind=fmt.ROUTER_AFFINE8)
    moe, dl, got1 = _check_layer(host, cfg, 3, seed=10, tol_gpu_oracle=5e-4)
    x = synthetic.hidden_rows(11, 3, cfg.d)
    h2 = gu.dev_empty(3 * cfg.d, "f32")
    moe.layer_decode(0, gu.to_dev(x), 3, h2_out=h2)
    sync()
    assert np.array_equal(h2.cpu().numpy().reshape(3, cfg.d).view(np.uint32), got1.view(np.uint32))


def test_hidden_residual_add():
    """hidden = out(hidden + h2) fused into the last stage (utility.metal:94-103)"""
    host, cfg = _layer_case(4, fmt.META_BF16, fmt.OUT_FP16, 1, seed=21, d=128, f=64, e=16)
    moe = MoE(cfg)
    dl = gu.DeviceLayer(host)
    dl.register(moe, 0)
    x = synthetic.hidden_rows(22, 1, cfg.d)
    hid0 = synthetic.hidden_rows(23, 1, cfg.d)
    hid = gu.to_dev(hid0.copy())
    h2 = gu.dev_empty(cfg.d, "f16")
    moe.layer_decode(0, gu.to_dev(x), 1, hidden=hid, h2_out=h2)
    sync()
    want = (orc.f16_bits_to_f32(hid0[0]) + orc.f16_bits_to_f32(gu.from_dev(h2, np.uint16))).astype(np.float16)
    assert np.array_equal(gu.from_dev(hid, np.float16).ravel(), want)


# ---------------------------------------------------------------------------
# pair grouping
# ---------------------------------------------------------------------------

def _device_grouping(pairs, tokens, top_k, num_experts):
    cfg = MoEConfig(d=128, f=64, shared_f=0, num_experts=num_experts, top_k=top_k, routed_bits=4, shared_bits=4,
                    router_kind=fmt.ROUTER_AFFINE8, shared_gate_kind=fmt.GATE_NONE, max_tokens=max(tokens, 1))
    moe = MoE(cfg)
    idx = np.zeros((tokens, top_k), dtype=np.uint32)
    w = np.zeros((tokens, top_k), dtype=np.uint16)
    for t, e, r, bits in pairs:
        idx[t, r] = e
        w[t, r] = bits
    n = tokens * top_k
    out = gu.dev_empty(n * 16, "u8")
    off, cnt = gu.dev_empty(num_experts, "u32"), gu.dev_empty(num_experts, "u32")
    moe.group_pairs(gu.to_dev(idx), gu.to_dev(w), tokens, out, off, cnt)
    sync()
    return (out.cpu().numpy().view(orc.PAIR_DTYPE), gu.from_dev(off, np.uint32), gu.from_dev(cnt, np.uint32))


def test_grouping_literal_tables():
    """PrefillMoEGroupingTests.swift:5-53, 55-82: exact sorted-pair order, offsets, counts, weight bits"""
    t = rv.GROUPING_TABLE_1
    s, off, cnt = _device_grouping(t["pairs"], t["query_count"], t["top_k"], t["num_experts"])
    assert s["expert"].tolist() == t["sorted_experts"]
    assert [[int(a), int(b)] for a, b in zip(s["token"], s["rank"])] == t["sorted_token_rank"]
    assert off.tolist() == t["offsets"] and cnt.tolist() == t["counts"]
    t2 = rv.GROUPING_TABLE_2
    s2, _, _ = _device_grouping(t2["pairs"], t2["query_count"], t2["top_k"], t2["num_experts"])
    assert s2["weight_bits"].tolist() == t2["sorted_weight_bits"]


@pytest.mark.parametrize("tokens", [1, 37, 256, 1500])
def test_grouping_matches_oracle_on_random_routes(tokens):
    """sortedness, a permutation of the input, and equality with the restated
    groupTokenExpertPairs on seeded routes (more than one 1024-pair pass at 1500)"""
    import ctypes as C
    rng = np.random.default_rng(tokens)
    K, E = 8, 256
    idx = np.stack([rng.choice(E, size=K, replace=False) for _ in range(tokens)]).astype(np.uint32)
    pairs = [(t, int(idx[t, r]), r, (t * K + r) & 0xFFFF) for t in range(tokens) for r in range(K)]
    s, off, cnt = _device_grouping(pairs, tokens, K, E)
    arr = rv.pairs_array(pairs)
    n = len(pairs)
    want = np.zeros(n, dtype=orc.PAIR_DTYPE)
    woff, wcnt = np.zeros(E, dtype=np.uint32), np.zeros(E, dtype=np.uint32)
    groups, tiles = np.zeros((n, 3), dtype=np.uint32), np.zeros((n, 4), dtype=np.uint32)
    ng, nt = C.c_size_t(0), C.c_size_t(0)
    rc = orc.lib().orc_group_pairs(orc.ptr(arr), n, tokens, K, E, 16, None, 0, orc.ptr(want), orc.ptr(woff),
                                   orc.ptr(wcnt), orc.ptr(groups), C.byref(ng), orc.ptr(tiles), C.byref(nt))
    assert rc == 0
    assert np.array_equal(s, want) and np.array_equal(off, woff) and np.array_equal(cnt, wcnt)


# ---------------------------------------------------------------------------
# stack driver
# ---------------------------------------------------------------------------

def test_stack_decode_small_matches_oracle_chain():
    layers, d, f, e = 3, 256, 128, 32
    cfg = MoEConfig(d=d, f=f, shared_f=f, num_experts=e, top_k=8, routed_bits=8, shared_bits=8,
                    router_kind=fmt.ROUTER_DENSE_F16, shared_gate_kind=fmt.ROUTER_DENSE_F16,
                    meta_dtype=fmt.META_FP16, out_dtype=fmt.OUT_FP32, max_tokens=2, num_layers=layers)
    moe = MoE(cfg)
    hosts = [synthetic.layer(300 + l, d=d, f=f, shared_f=f, num_experts=e, routed_bits=8, meta=fmt.META_FP16)
             for l in range(layers)]
    devs = [gu.DeviceLayer(h) for h in hosts]
    for l, dv in enumerate(devs):
        dv.register(moe, l)
    x0 = synthetic.hidden_rows(400, 2, d)
    y = gu.dev_empty(2 * d, "f32")
    torch = gu.torch_cuda()
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        xd = gu.to_dev(x0)
        st.synchronize()
        moe.stack_decode(xd, 2, y, stream=st)       # captured + replayed as a CUDA graph
        moe.stack_decode(xd, 2, y, stream=st)       # replay
        st.synchronize()
    got = y.cpu().numpy().reshape(2, d)
    for t in range(2):
        x = np.ascontiguousarray(x0[t])
        for l in range(layers):
            L, keep = gu.oracle_layer(hosts[l], cfg)
            _, _, h2, _, _ = gu.oracle_decode(L, cfg, x)
            if l + 1 < layers:
                scale = 1.0 / np.sqrt(np.mean(h2.astype(np.float64) ** 2) + 1e-6)
                x = orc.f32_to_f16_bits((h2.astype(np.float64) * scale).astype(np.float32))
        assert orc.rel_error(got[t], h2) < 2e-3


# ---------------------------------------------------------------------------
# error behaviour (host-side injection only)
# ---------------------------------------------------------------------------

def test_errors_are_codes_not_traps():
    from nvmai_b200 import NvmaiError
    from nvmai_b200 import _lib
    host, cfg = _layer_case(4, fmt.META_BF16, fmt.OUT_FP16, 1, seed=31, d=128, f=64, e=16)
    moe = MoE(cfg)
    x = gu.to_dev(synthetic.hidden_rows(1, 1, cfg.d))
    with pytest.raises(NvmaiError) as ei:                       # layer never registered
        moe.layer_decode(0, x, 1)
    assert ei.value.code == _lib.EINVAL
    dl = gu.DeviceLayer(host)
    dl.register(moe, 0)
    with pytest.raises(NvmaiError) as ei:                       # more tokens than max_tokens
        moe.layer_decode(0, x, 2)
    assert ei.value.code == _lib.ERANGE
    with pytest.raises(NvmaiError) as ei:                       # layer index out of range
        moe.layer_decode(3, x, 1)
    assert ei.value.code == _lib.ERANGE
    with pytest.raises(NvmaiError) as ei:                       # misaligned input
        moe.layer_decode(0, x.data_ptr() + 2, 1)
    assert ei.value.code == _lib.EINVAL
    bad = dict(host["offsets"]); bad["down_b"] = host["stride"]    # offset + bytes past the blob
    with pytest.raises(NvmaiError) as ei:
        moe.register_layer(0, experts=dl.experts, expert_stride=host["stride"], offsets=bad, router=dl.router,
                           shared=dl.shared, shared_gate=dl.gate)
    assert ei.value.code == _lib.ERANGE


def test_resident_tensors_at_bases_that_are_off_by_two_bytes():
    """the reference packs router / shared-expert tensors back to back without alignment and tests its kernels on a
    base that is off by two bytes (DequantInt4GEMVTests.swift:114-121): such tensors are realigned at registration
    and the layer gives the same bits as with aligned tensors"""
    import torch
    tokens = 3
    host = synthetic.layer(611, d=256, f=128, shared_f=128, num_experts=16, routed_bits=4, shared_bits=4,
                           meta=fmt.META_BF16, router_kind=fmt.ROUTER_AFFINE8, gate_kind=fmt.ROUTER_AFFINE8)
    cfg = MoEConfig(d=256, f=128, shared_f=128, num_experts=16, top_k=8, routed_bits=4, shared_bits=4,
                    router_kind=fmt.ROUTER_AFFINE8, shared_gate_kind=fmt.ROUTER_AFFINE8, meta_dtype=fmt.META_BF16,
                    out_dtype=fmt.OUT_FP32, max_tokens=tokens)
    x = gu.to_dev(synthetic.hidden_rows(612, tokens, 256))
    dl = gu.DeviceLayer(host)

    def off_by_two(t):
        if t is None:
            return None
        flat = t.contiguous().view(torch.uint8).reshape(-1)
        buf = torch.zeros(flat.numel() + 32, dtype=torch.uint8, device=flat.device)
        view = buf[2:2 + flat.numel()]
        view.copy_(flat)
        assert view.data_ptr() % 16 == 2
        return view

    def run(shift):
        moe = MoE(cfg)
        if shift:
            fix = lambda t3: tuple(off_by_two(t) for t in t3)
            moe.register_layer(0, experts=dl.experts, expert_stride=host["stride"], offsets=host["offsets"],
                               router=fix(dl.router), shared=[fix(t) for t in dl.shared], shared_gate=fix(dl.gate))
        else:
            dl.register(moe, 0)
        y = gu.dev_empty(tokens * 256, "f32")
        moe.layer_decode(0, x, tokens, h2_out=y)
        moe.synchronize()
        return y.cpu().numpy()

    np.testing.assert_array_equal(run(True), run(False))
