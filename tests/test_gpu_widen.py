"""GPU parity tests of the callers either side of the decode block: the width-2
verification entry point and the block with the attention residual add and the
post-attention RMS norm folded in.  Through the C ABI, against the CPU oracle.
"""
import ctypes as C

import numpy as np
import pytest

import gpu_util as gu
import refvectors as rv
from nvmai_b200 import MoE, MoEConfig, synthetic
from nvmai_b200 import format as fmt
from oracle import oracle as orc

pytestmark = pytest.mark.gpu

FFN_TOL = 1e-3


def sync():
    gu.torch_cuda().cuda.synchronize()


def _case(bits, meta, out_dtype, tokens, seed, d=2048, f=512, e=256, router_kind=fmt.ROUTER_DENSE_F16,
          gate_kind=fmt.ROUTER_DENSE_F16):
    host = synthetic.layer(seed, d=d, f=f, shared_f=f, num_experts=e, routed_bits=bits, meta=meta,
                           router_kind=router_kind, gate_kind=gate_kind)
    cfg = MoEConfig(d=d, f=f, shared_f=f, num_experts=e, top_k=8, routed_bits=bits, shared_bits=bits,
                    router_kind=router_kind, shared_gate_kind=gate_kind, meta_dtype=meta,
                    activation=fmt.ACT_SILU, out_dtype=out_dtype, max_tokens=tokens)
    return host, cfg


def _out(t, cfg, rows):
    if cfg.out_dtype == fmt.OUT_FP16:
        return orc.f16_bits_to_f32(gu.from_dev(t, np.uint16)).reshape(rows, cfg.d)
    return t.cpu().numpy().reshape(rows, cfg.d)


@pytest.mark.parametrize("bits,out_dtype", [(4, fmt.OUT_FP16), (8, fmt.OUT_FP32)])
def test_verify_pair_equals_two_decode_rows(bits, out_dtype):
    """`encodeRoutedMoEVerifyPair`: each of the two rows gets the decode block's result (the reference encodes the
    decode kernels once per row), indices exact; the second row is the first plus a small perturbation so that the
    rows share most experts, which is the case the entry point exists for"""
    kind = fmt.ROUTER_AFFINE8 if out_dtype == fmt.OUT_FP16 else fmt.ROUTER_DENSE_F16
    host, cfg = _case(bits, fmt.META_BF16, out_dtype, 2, seed=301 + bits, router_kind=kind, gate_kind=kind)
    moe = MoE(cfg)
    dl = gu.DeviceLayer(host)
    dl.register(moe, 0)
    x = synthetic.hidden_rows(302, 2, cfg.d)
    x32 = orc.f16_bits_to_f32(x[0])
    bump = orc.f16_bits_to_f32(synthetic.hidden_rows(303, 1, cfg.d)[0]) * np.float32(0.05)
    x[1] = orc.f32_to_f16_bits(x32 + bump)
    esz = "f16" if out_dtype == fmt.OUT_FP16 else "f32"
    hid0 = synthetic.hidden_rows(304, 2, cfg.d)
    hid_host = hid0 if out_dtype == fmt.OUT_FP16 else orc.f16_bits_to_f32(hid0).astype(np.float32)
    hid = gu.to_dev(hid_host.copy())
    h2 = gu.dev_empty(2 * cfg.d, esz)
    idx, w = gu.dev_empty(16, "u32"), gu.dev_empty(16, "f16")
    moe.layer_verify_pair(0, gu.to_dev(x), hidden=hid, h2_out=h2, out_idx=idx, out_w=w)
    sync()
    got, got_hid = _out(h2, cfg, 2), _out(hid, cfg, 2)
    got_idx = gu.from_dev(idx, np.uint32).reshape(2, 8)
    L, keep = gu.oracle_layer(host, cfg)
    shared = len(set(got_idx[0].tolist()) & set(got_idx[1].tolist()))
    assert shared >= 4, f"the two rows share only {shared} experts: not the case under test"
    tol_gpu = 2e-3 if out_dtype == fmt.OUT_FP16 else 5e-4
    for t in range(2):
        o_idx, o_w, o_h2, margin, cpu = gu.oracle_decode(L, cfg, np.ascontiguousarray(x[t]))
        assert margin > 1e-5
        assert got_idx[t].tolist() == o_idx.tolist()
        assert orc.rel_error(got[t], cpu) < FFN_TOL, "vs the reference CPU path"
        assert orc.rel_error(got[t], o_h2) < tol_gpu, "vs the shader-semantics oracle"
        # the tail: one residual add per row (RealForwardRunner.swift:3207-3213), in the output type
        base = orc.f16_bits_to_f32(hid0[t])
        if out_dtype == fmt.OUT_FP16:
            want = (base + got[t]).astype(np.float16).astype(np.float32)
        else:
            want = base + got[t]
        assert np.array_equal(got_hid[t], want)
    # and bitwise the same as the general entry point with two rows
    h2b = gu.dev_empty(2 * cfg.d, esz)
    moe.layer_decode(0, gu.to_dev(x), 2, h2_out=h2b)
    sync()
    assert np.array_equal(_out(h2b, cfg, 2).view(np.uint32), got.view(np.uint32))


@pytest.mark.parametrize("d,seed", [(256, 0xC3), (2048, 0xD4)])
def test_prenorm_rows_match_reference_rmsnorm_vectors(d, seed):
    """the normalised rows the fused entry point hands to the block, on the inputs of the reference's own rmsnorm
    tests (RMSNormTests.swift:22-61), within the reference's bar of its fp32 comparator and within one fp16 ulp of
    the oracle"""
    case = rv.rmsnorm_bf16w_case(d, seed)
    host, cfg = _case(4, fmt.META_BF16, fmt.OUT_FP16, 1, seed=311, d=d, f=128, e=32)
    moe = MoE(cfg)
    dl = gu.DeviceLayer(host)
    dl.register(moe, 0)
    hid = gu.to_dev(case["x16"].view(np.uint16).copy())
    xo = gu.dev_empty(d, "f16")
    moe.layer_decode_prenorm(0, hid, gu.to_dev(case["w_bits"]), case["eps"], 1, x_out=xo)
    sync()
    got_bits = gu.from_dev(xo, np.uint16).ravel()
    got = orc.f16_bits_to_f32(got_bits)
    assert orc.rel_error(got, case["ref"]) < case["tol"]
    want = np.zeros(d, dtype=np.uint16)
    orc.lib().orc_gpu_rmsnorm_bf16w(orc.ptr(case["x16"].view(np.uint16)), orc.ptr(case["w_bits"]), orc.ptr(want), d,
                                    case["eps"], fmt.OUT_FP16)
    ulp = np.abs(got_bits.astype(np.int32) - want.astype(np.int32))    # same sign bits wherever both are non-zero
    assert ulp.max() <= 1 and np.count_nonzero(ulp) <= d // 100


@pytest.mark.parametrize("tokens,out_dtype,grouped_min", [(1, fmt.OUT_FP16, None), (3, fmt.OUT_FP16, None),
                                                          (1, fmt.OUT_FP32, None), (6, fmt.OUT_FP16, 4)])
def test_prenorm_block_matches_unfused_sequence(tokens, out_dtype, grouped_min, monkeypatch):
    """residual add -> rmsnorm_bf16w -> decode block -> residual add (RealForwardRunner.swift:1900-1909, 1911-1995) in
    three launches: the hidden state after the first add and the final add are exact given the block output, the
    normalised rows are within one fp16 ulp of the oracle's, and the block output on those rows meets the decode bars"""
    if grouped_min is not None:
        monkeypatch.setenv("NVMAI_CUDA_GROUPED_MIN", str(grouped_min))
    kind = fmt.ROUTER_AFFINE8 if out_dtype == fmt.OUT_FP16 else fmt.ROUTER_DENSE_F16
    host, cfg = _case(4, fmt.META_BF16, out_dtype, tokens, seed=321, router_kind=kind, gate_kind=kind)
    moe = MoE(cfg)
    dl = gu.DeviceLayer(host)
    dl.register(moe, 0)
    f16 = out_dtype == fmt.OUT_FP16
    esz = "f16" if f16 else "f32"
    rng = np.random.default_rng(322)
    hid32 = (rng.standard_normal((tokens, cfg.d)) * 3.0).astype(np.float32)
    delta16 = (rng.standard_normal((tokens, cfg.d)) * 0.7).astype(np.float16)
    w_bits = orc.f32_to_bf16_bits(rng.uniform(0.5, 1.5, cfg.d).astype(np.float32))
    hid_host = hid32.astype(np.float16).view(np.uint16) if f16 else hid32
    eps = 1e-6
    hid = gu.to_dev(hid_host.copy())
    h2 = gu.dev_empty(tokens * cfg.d, esz)
    xo = gu.dev_empty(tokens * cfg.d, "f16")
    idx = gu.dev_empty(tokens * 8, "u32")
    moe.layer_decode_prenorm(0, hid, gu.to_dev(w_bits), eps, tokens, attn_delta=gu.to_dev(delta16.view(np.uint16)),
                             h2_out=h2, x_out=xo, out_idx=idx)
    sync()
    got_h2, got_hid = _out(h2, cfg, tokens), _out(hid, cfg, tokens)
    got_x = gu.from_dev(xo, np.uint16).reshape(tokens, cfg.d)
    got_idx = gu.from_dev(idx, np.uint32).reshape(tokens, 8)
    # hidden' = out(hidden + delta) (utility.metal:94-103)
    mid = hid_host.copy()
    orc.lib().orc_gpu_residual_add(orc.ptr(mid), orc.ptr(delta16.view(np.uint16) if f16 else delta16.astype(np.float32)),
                                   tokens * cfg.d, out_dtype)
    mid32 = orc.f16_bits_to_f32(mid).reshape(tokens, cfg.d) if f16 else mid
    L, keep = gu.oracle_layer(host, cfg)
    tol_gpu = 2e-3 if f16 else 5e-4
    for t in range(tokens):
        want_x = np.zeros(cfg.d, dtype=np.uint16)
        orc.lib().orc_gpu_rmsnorm_bf16w(orc.ptr(np.ascontiguousarray(mid[t])), orc.ptr(w_bits), orc.ptr(want_x), cfg.d,
                                        eps, out_dtype)
        ulp = np.abs(got_x[t].astype(np.int32) - want_x.astype(np.int32))
        assert ulp.max() <= 1 and np.count_nonzero(ulp) <= cfg.d // 100, f"row {t}: normalised rows"
        o_idx, o_w, o_h2, margin, cpu = gu.oracle_decode(L, cfg, np.ascontiguousarray(got_x[t]))
        assert margin > 1e-5
        assert got_idx[t].tolist() == o_idx.tolist()
        assert orc.rel_error(got_h2[t], cpu) < FFN_TOL, "vs the reference CPU path"
        assert orc.rel_error(got_h2[t], o_h2) < tol_gpu, "vs the shader-semantics oracle"
        want_hid = (mid32[t] + got_h2[t]).astype(np.float16).astype(np.float32) if f16 else mid32[t] + got_h2[t]
        assert np.array_equal(got_hid[t], want_hid), f"row {t}: hidden = out(out(hidden + delta) + h2)"


@pytest.mark.parametrize("tokens,out_dtype,grouped_min", [(1, fmt.OUT_FP16, None), (3, fmt.OUT_FP32, None),
                                                          (6, fmt.OUT_FP16, 4), (40, fmt.OUT_FP32, None)])
def test_next_block_input_norm_is_written_by_the_last_stage(tokens, out_dtype, grouped_min, monkeypatch):
    """RealForwardRunner.swift:1886-1909: the layer after the MoE block starts with rmsnorm_bf16w of the hidden state the
    block wrote; with the fused entry point the block's last stage writes that row too.  Everything else must be the
    bits of the call without it; the normalised rows within one fp16 ulp of the oracle's rmsnorm of the same hidden
    state.  1 / 3 rows: the down stage's last block per row; 6 rows: the grouped combine; 40 rows: the tensor-core path."""
    if grouped_min is not None:
        monkeypatch.setenv("NVMAI_CUDA_GROUPED_MIN", str(grouped_min))
    kind = fmt.ROUTER_AFFINE8 if out_dtype == fmt.OUT_FP16 else fmt.ROUTER_DENSE_F16
    host, cfg = _case(4, fmt.META_BF16, out_dtype, tokens, seed=325, d=512, f=256, e=32, router_kind=kind, gate_kind=kind)
    f16 = out_dtype == fmt.OUT_FP16
    esz = "f16" if f16 else "f32"
    rng = np.random.default_rng(326)
    hid32 = (rng.standard_normal((tokens, cfg.d)) * 3.0).astype(np.float32)
    delta16 = (rng.standard_normal((tokens, cfg.d)) * 0.7).astype(np.float16)
    w_bits = orc.f32_to_bf16_bits(rng.uniform(0.5, 1.5, cfg.d).astype(np.float32))
    wn_bits = orc.f32_to_bf16_bits(rng.uniform(0.5, 1.5, cfg.d).astype(np.float32))
    hid_host = hid32.astype(np.float16).view(np.uint16) if f16 else hid32
    dl = gu.DeviceLayer(host)
    outs = []
    for fused in (False, True):
        moe = MoE(cfg)
        dl.register(moe, 0)
        hid = gu.to_dev(hid_host.copy())
        h2 = gu.dev_empty(tokens * cfg.d, esz)
        xn = gu.to_dev(np.full(tokens * cfg.d, 0x7E00, dtype=np.uint16))
        delta = gu.to_dev(delta16.view(np.uint16))
        if fused:
            moe.layer_decode_fused_norms(0, hid, gu.to_dev(w_bits), 1e-6, tokens, gu.to_dev(wn_bits), 1e-5, xn,
                                         attn_delta=delta, h2_out=h2)
        else:
            moe.layer_decode_prenorm(0, hid, gu.to_dev(w_bits), 1e-6, tokens, attn_delta=delta, h2_out=h2)
        moe.synchronize()
        raw = np.uint16 if f16 else np.uint32
        outs.append((gu.from_dev(hid, raw).copy(), gu.from_dev(h2, raw).copy(), gu.from_dev(xn, np.uint16).copy()))
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])
    hid_out = outs[1][0].reshape(tokens, cfg.d)
    got = outs[1][2].reshape(tokens, cfg.d)
    for t in range(tokens):
        want = np.zeros(cfg.d, dtype=np.uint16)
        row = np.ascontiguousarray(hid_out[t] if f16 else hid_out[t].view(np.float32))
        orc.lib().orc_gpu_rmsnorm_bf16w(orc.ptr(row), orc.ptr(wn_bits), orc.ptr(want), cfg.d, 1e-5, out_dtype)
        ulp = np.abs(got[t].astype(np.int32) - want.astype(np.int32))
        assert ulp.max() <= 1 and np.count_nonzero(ulp) <= max(1, cfg.d // 100), f"row {t}"


def test_prenorm_rejects_bad_arguments():
    from nvmai_b200 import NvmaiError, _lib
    host, cfg = _case(4, fmt.META_BF16, fmt.OUT_FP16, 2, seed=331, d=256, f=128, e=32)
    moe = MoE(cfg)
    dl = gu.DeviceLayer(host)
    dl.register(moe, 0)
    hid = gu.dev_empty(2 * cfg.d, "f16")
    w = gu.dev_empty(cfg.d, "f16")
    for args, kw, code in [((0, None, w, 1e-6, 1), {}, _lib.EINVAL),           # no hidden state
                           ((0, hid, None, 1e-6, 1), {}, _lib.EINVAL),         # no norm weight
                           ((0, hid, w, -1.0, 1), {}, _lib.EINVAL),            # negative eps
                           ((0, hid, w, 1e-6, 3), {}, _lib.ERANGE),            # more rows than max_tokens
                           ((1, hid, w, 1e-6, 1), {}, _lib.ERANGE)]:           # layer out of range
        with pytest.raises(NvmaiError) as ei:
            moe.layer_decode_prenorm(*args, **kw)
        assert ei.value.code == code
    with pytest.raises(NvmaiError) as ei:
        moe.layer_verify_pair(5, hid)
    assert ei.value.code == _lib.ERANGE


@pytest.mark.parametrize("rows", [12, 48])
def test_route_trace_replay_matches_cpu_path(rows):
    """a recorded routing (`position layer e0..e7`) drives the routed kernels through `routed_partial`; every row's
    share equals the reference CPU path's accumulation over the recorded experts with the replay's weights.
    12 rows run the per-row tiles, 48 rows the tensor-core tiles"""
    from nvmai_b200 import route_trace as rt
    e = 32
    host, cfg = _case(4, fmt.META_BF16, fmt.OUT_FP32, rows, seed=341, d=256, f=128, e=e)
    moe = MoE(cfg)
    dl = gu.DeviceLayer(host)
    dl.register(moe, 0)
    trace = rt.parse(rt.synthesize(40, 2, num_experts=e, reuse=0.38, seed=5).format(), num_experts=e, num_layers=2)
    ids = trace.batch(1, first_row=30, rows=rows)              # wraps past the last recorded token
    x = synthetic.hidden_rows(342, rows, cfg.d)
    w16 = np.full((rows, 8), 1.0 / 8, dtype=np.float16)
    share = gu.dev_empty(rows * cfg.d, "f32")
    moe.routed_partial(0, gu.to_dev(x), rows, gu.to_dev(ids.astype(np.uint32)), gu.to_dev(w16.view(np.uint16)), share)
    sync()
    got = share.cpu().numpy().reshape(rows, cfg.d)
    off = np.array([host["offsets"][n] for n in fmt.OFFSET_NAMES], dtype=np.uint32)
    lib, fn = orc.lib(), orc.ref_gemv4_ptr()
    blobs = host["experts"]
    scratch = np.zeros(2 * cfg.f + cfg.d, dtype=np.float32)
    for t in range(rows):
        want = np.zeros(cfg.d, dtype=np.float32)
        x32 = orc.f16_bits_to_f32(x[t])
        for k in range(8):
            blob = blobs[int(ids[t, k])]
            lib.orc_cpu_expert_accumulate(orc.ptr(blob), orc.ptr(off), 4, orc.META_BF16, orc.ACT_SILU, orc.ptr(x32),
                                          cfg.d, cfg.f, float(np.float16(1.0 / 8)), orc.ptr(scratch), orc.ptr(want), fn)
        assert orc.rel_error(got[t], want) < FFN_TOL, f"row {t}"


def test_zipf_batch_of_256_rows_at_the_benchmark_shape():
    """configs[4] as the benchmark runs it: 256 rows whose experts follow Zipf(1.1) over a seeded permutation, through
    `routed_partial` on one 4-bit layer of the 35B-A3B shape (the hottest expert takes more than 200 rows: work items
    wider than one accumulator).  Sampled rows against the reference CPU path's accumulation."""
    rows, e, k = 256, 256, 8
    host, cfg = _case(4, fmt.META_BF16, fmt.OUT_FP32, rows, seed=371, d=2048, f=512, e=e)
    moe = MoE(cfg)
    dl = gu.DeviceLayer(host)
    dl.register(moe, 0)
    rng = np.random.default_rng(4)
    perm = rng.permutation(e)
    p_ = np.arange(1, e + 1, dtype=np.float64) ** -1.1
    p_ /= p_.sum()
    ids = np.stack([perm[rng.choice(e, size=k, replace=False, p=p_)] for _ in range(rows)]).astype(np.uint32)
    counts = np.bincount(ids.reshape(-1), minlength=e)
    assert counts.max() > 200
    x = synthetic.hidden_rows(372, rows, cfg.d)
    w16 = np.full((rows, k), 1.0 / k, dtype=np.float16)
    share = gu.dev_empty(rows * cfg.d, "f32")
    moe.routed_partial(0, gu.to_dev(x), rows, gu.to_dev(ids), gu.to_dev(w16.view(np.uint16)), share)
    moe.synchronize()
    got = share.cpu().numpy().reshape(rows, cfg.d)
    assert np.all(np.isfinite(got))
    off = np.array([host["offsets"][n] for n in fmt.OFFSET_NAMES], dtype=np.uint32)
    lib, fn = orc.lib(), orc.ref_gemv4_ptr()
    scratch = np.zeros(2 * cfg.f + cfg.d, dtype=np.float32)
    hot = int(np.argmax(counts))
    rows_hot = np.nonzero((ids == hot).any(axis=1))[0]
    sample = sorted(set([0, 1, 31, 32, 100, 255] + rows_hot[[0, len(rows_hot) // 2, -1]].tolist() + list(range(7, 256, 37))))
    worst = 0.0
    for t in sample:
        want = np.zeros(cfg.d, dtype=np.float32)
        x32 = orc.f16_bits_to_f32(x[t])
        for kk in range(k):
            lib.orc_cpu_expert_accumulate(orc.ptr(host["experts"][int(ids[t, kk])]), orc.ptr(off), 4, orc.META_BF16,
                                          orc.ACT_SILU, orc.ptr(x32), cfg.d, cfg.f, float(np.float16(1.0 / k)),
                                          orc.ptr(scratch), orc.ptr(want), fn)
        err = orc.rel_error(got[t], want)
        worst = max(worst, err)
        assert err < FFN_TOL, f"row {t}"
    print(f"[parity] zipf-256 worst sampled error against the CPU path: {worst:.3g}")


@pytest.mark.parametrize("placement", ["contiguous", "strided"])
def test_zipf_batch_on_a_rank_that_holds_a_part_of_the_experts(placement):
    """the 256-row Zipf batch on one of two expert-parallel ranks: the handle holds only its rank's blobs (expert
    map), the tensor-core items cover that rank's pairs, and the share equals what a handle with all experts
    computes when the other rank's pairs get weight zero (their products vanish exactly); the two ranks' shares
    add up to the full result within rounding"""
    from nvmai_b200.ep import ExpertPlacement
    rows, e, k = 256, 256, 8
    host, cfg = _case(4, fmt.META_BF16, fmt.OUT_FP32, rows, seed=381, d=2048, f=512, e=e)
    rng = np.random.default_rng(5)
    perm = rng.permutation(e)
    p_ = np.arange(1, e + 1, dtype=np.float64) ** -1.1
    p_ /= p_.sum()
    ids = np.stack([perm[rng.choice(e, size=k, replace=False, p=p_)] for _ in range(rows)]).astype(np.uint32)
    x = synthetic.hidden_rows(382, rows, cfg.d)
    w16 = np.full((rows, k), 1.0 / k, dtype=np.float16)
    pl = ExpertPlacement(e, 2, placement)

    full = MoE(cfg)
    dl_full = gu.DeviceLayer(host)
    dl_full.register(full, 0)

    def full_share(weights):
        out = gu.dev_empty(rows * cfg.d, "f32")
        full.routed_partial(0, gu.to_dev(x), rows, gu.to_dev(ids), gu.to_dev(weights.view(np.uint16)), out)
        full.synchronize()
        return out.cpu().numpy().reshape(rows, cfg.d)

    whole = full_share(w16)
    total = np.zeros_like(whole)
    for rank in range(2):
        local = dict(host)
        local["experts"] = np.ascontiguousarray(host["experts"][pl.local_experts(rank)])
        moe = MoE(cfg)
        dl = gu.DeviceLayer(local)
        dl.register(moe, 0)
        moe.set_expert_map(pl.expert_map(rank))
        share = gu.dev_empty(rows * cfg.d, "f32")
        moe.routed_partial(0, gu.to_dev(x), rows, gu.to_dev(ids), gu.to_dev(w16.view(np.uint16)), share)
        moe.synchronize()
        got = share.cpu().numpy().reshape(rows, cfg.d)
        owners = np.vectorize(pl.owner)(ids)
        masked = np.where(owners == rank, w16, np.float16(0.0)).astype(np.float16)
        want = full_share(masked)
        assert np.all(np.isfinite(got))
        np.testing.assert_allclose(got, want, rtol=0, atol=1e-6 * float(np.abs(want).max()))
        total += got
    assert orc.rel_error(total.reshape(-1), whole.reshape(-1)) < 1e-5


@pytest.mark.parametrize("out_dtype", [fmt.OUT_FP32, fmt.OUT_FP16])
def test_large_decode_batch_on_tensor_cores_keeps_decode_semantics(out_dtype, monkeypatch):
    """from 32 rows on a 4-bit batched decode call runs the grouped GEMMs of the prefill path; indices stay exact,
    every row stays within the bars of the decode oracle, the residual add keeps the decode order (one add of the
    rounded block output), and the result agrees with the per-row kernels' result for the same call"""
    tokens = 40
    kind = fmt.ROUTER_AFFINE8 if out_dtype == fmt.OUT_FP16 else fmt.ROUTER_DENSE_F16
    host, cfg = _case(4, fmt.META_BF16, out_dtype, tokens, seed=351, router_kind=kind, gate_kind=kind)
    f16 = out_dtype == fmt.OUT_FP16
    esz = "f16" if f16 else "f32"
    x = synthetic.hidden_rows(352, tokens, cfg.d)
    hid0 = synthetic.hidden_rows(353, tokens, cfg.d)
    hid_host = hid0 if f16 else orc.f16_bits_to_f32(hid0).astype(np.float32)
    dl = gu.DeviceLayer(host)

    def run():
        moe = MoE(cfg)
        dl.register(moe, 0)
        hid = gu.to_dev(hid_host.copy())
        h2 = gu.dev_empty(tokens * cfg.d, esz)
        idx = gu.dev_empty(tokens * 8, "u32")
        moe.layer_decode(0, gu.to_dev(x), tokens, hidden=hid, h2_out=h2, out_idx=idx)
        sync()
        return _out(h2, cfg, tokens), _out(hid, cfg, tokens), gu.from_dev(idx, np.uint32).reshape(tokens, 8)

    got, got_hid, got_idx = run()
    monkeypatch.setenv("NVMAI_CUDA_TC_MIN", "100000")       # the same call on the per-row kernels
    per_row, _, per_row_idx = run()
    assert np.array_equal(got_idx, per_row_idx)
    L, keep = gu.oracle_layer(host, cfg)
    for t in range(tokens):
        o_idx, o_w, o_h2, margin, cpu = gu.oracle_decode(L, cfg, np.ascontiguousarray(x[t]))
        assert margin > 1e-5
        assert got_idx[t].tolist() == o_idx.tolist()
        assert orc.rel_error(got[t], cpu) < FFN_TOL, "vs the reference CPU path"
        own = orc.rel_error(o_h2, cpu)
        assert orc.rel_error(got[t], o_h2) < max(2e-3 if f16 else 1e-3, own + 2e-4), "vs the shader-semantics oracle"
        assert orc.rel_error(got[t], per_row[t]) < (2e-3 if f16 else 1e-3), "vs the per-row kernels"
        base = orc.f16_bits_to_f32(hid0[t])
        want = (base + got[t]).astype(np.float16).astype(np.float32) if f16 else base + got[t]
        assert np.array_equal(got_hid[t], want)


def test_gturbo_layers_load_into_hbm_in_logical_order(tmp_path):
    """a synthetic `.gturbo` artifact (layer 1 with permuted physical ranks) read by the library's pinned
    double-buffered reader: device bytes equal the blobs in logical order, the SHA-256 of the manifest holds, and the
    block computed from the loaded experts equals, bit for bit, the block computed from directly uploaded ones"""
    from nvmai_b200 import NvmaiError, _lib, gturbo
    d, f, e = 256, 128, 32
    hosts = [_case(4, fmt.META_BF16, fmt.OUT_FP32, 2, seed=361 + l, d=d, f=f, e=e)[0] for l in range(2)]
    cfg = _case(4, fmt.META_BF16, fmt.OUT_FP32, 2, seed=361, d=d, f=f, e=e)[1]
    ranks = [np.arange(e), np.random.default_rng(7).permutation(e)]
    gturbo.write_packed_experts(tmp_path, [h["experts"] for h in hosts], d=d, f=f, bits=4, physical_ranks=ranks)
    g = gturbo.GTurboExperts(tmp_path)
    assert g.routed_bits() == 4 and g.layout.expert_offsets(0) == dict(hosts[0]["offsets"])
    stride, blob = g.layout.expert_stride, hosts[0]["experts"].shape[1]
    x = gu.to_dev(synthetic.hidden_rows(363, 2, d))
    for l in range(2):
        buf = gu.dev_empty(g.layer_bytes, "u8")
        g.load_layer(l, buf, verify=True)
        sync()
        got = buf.cpu().numpy().reshape(e, stride)
        assert np.array_equal(got[:, :blob], hosts[l]["experts"]), f"layer {l}"
        dl = gu.DeviceLayer(hosts[l])
        direct, loaded = MoE(cfg), MoE(cfg)
        dl.register(direct, 0)
        g.register_layer(loaded, 0, buf, router=dl.router, shared=dl.shared, shared_gate=dl.gate)
        ya, yb = gu.dev_empty(2 * d, "f32"), gu.dev_empty(2 * d, "f32")
        direct.layer_decode(0, x, 2, h2_out=ya)
        loaded.layer_decode(0, x, 2, h2_out=yb)
        sync()
        assert np.array_equal(ya.cpu().numpy().view(np.uint32), yb.cpu().numpy().view(np.uint32))
    lib = _lib.lib()
    buf = gu.dev_empty(64, "u8")
    path = g.layer_path(0).encode()
    assert lib.nvmai_cuda_moe_read_file_to_device(path, g.layer_bytes - 32, 64, buf.data_ptr(), None) == _lib.EIO
    assert lib.nvmai_cuda_moe_read_file_to_device(path + b".missing", 0, 64, buf.data_ptr(), None) == _lib.EIO
    assert lib.nvmai_cuda_moe_read_file_to_device(None, 0, 64, buf.data_ptr(), None) == _lib.EINVAL
    assert lib.nvmai_cuda_moe_read_file_to_device(path, 0, 0, None, None) == _lib.OK


def test_large_decode_batch_inside_a_stream_capture():
    """a 40-row call captured into a CUDA graph: before any eager call the handle has no packed-row scratch and may
    not allocate under capture, so the captured call uses the per-row kernels; after one eager call the capture takes
    the tensor-core launches and replays the eager result bit for bit"""
    torch = gu.torch_cuda()
    tokens = 40
    host, cfg = _case(4, fmt.META_BF16, fmt.OUT_FP32, tokens, seed=371, d=256, f=128, e=32)
    moe = MoE(cfg)
    dl = gu.DeviceLayer(host)
    dl.register(moe, 0)
    x = gu.to_dev(synthetic.hidden_rows(372, tokens, cfg.d))
    y = gu.dev_empty(tokens * cfg.d, "f32")
    stream = torch.cuda.Stream()

    def capture_and_replay():
        y.zero_()
        graph = torch.cuda.CUDAGraph()
        stream.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            moe.layer_decode(0, x, tokens, h2_out=y, stream=torch.cuda.current_stream())
        graph.replay()
        sync()
        return y.cpu().numpy().copy()

    first = capture_and_replay()                 # per-row kernels
    moe.layer_decode(0, x, tokens, h2_out=y, stream=stream)
    sync()
    eager = y.cpu().numpy().copy()               # tensor-core launches, scratch now allocated
    second = capture_and_replay()
    assert np.array_equal(second.view(np.uint32), eager.view(np.uint32))
    assert np.all(np.isfinite(first))
    for t in range(tokens):
        a, b = first.reshape(tokens, -1)[t], eager.reshape(tokens, -1)[t]
        assert orc.rel_error(a, b) < 1e-3
