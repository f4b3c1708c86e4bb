"""Prefill block (router, grouping, tensor-core grouped GEMMs, ordered combine) through
the C ABI against the oracle: the shader-semantics restatement with the prefill path's
rounding points, and the reference CPU path (fp32 throughout)."""
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
for p_ in (ROOT, ROOT / "tests"):
    if str(p_) not in sys.path:
        sys.path.insert(0, str(p_))

pytestmark = pytest.mark.gpu

from nvmai_b200 import MoE, MoEConfig, synthetic      # noqa: E402
from nvmai_b200 import format as fmt                  # noqa: E402
from nvmai_b200 import NvmaiError                     # noqa: E402
from oracle import oracle as orc                      # noqa: E402
import gpu_util as gu                                 # noqa: E402

FFN_TOL = 1e-3      # RelError.compute(actual, reference CPU path) bound of the reference's own tests


def sync():
    import torch
    torch.cuda.synchronize()


def _case(bits, meta, out_dtype, tokens, seed, d=256, f=128, e=32, router_kind=fmt.ROUTER_DENSE_F16,
          gate_kind=fmt.ROUTER_DENSE_F16):
    host = synthetic.layer(seed, d=d, f=f, shared_f=f, num_experts=e, routed_bits=bits, meta=meta,
                           router_kind=router_kind, gate_kind=gate_kind)
    cfg = MoEConfig(d=d, f=f, shared_f=f, num_experts=e, top_k=8, routed_bits=bits, shared_bits=bits,
                    router_kind=router_kind, shared_gate_kind=gate_kind, meta_dtype=meta,
                    activation=fmt.ACT_SILU, out_dtype=out_dtype, max_tokens=tokens)
    return host, cfg


def _run_prefill(host, cfg, tokens, seed, with_hidden=False):
    moe = MoE(cfg)
    dl = gu.DeviceLayer(host)
    dl.register(moe, 0)
    x = synthetic.hidden_rows(seed, tokens, cfg.d)
    f16 = cfg.out_dtype == fmt.OUT_FP16
    esz = "f16" if f16 else "f32"
    y = gu.dev_empty(tokens * cfg.d, esz)
    idx, w = gu.dev_empty(tokens * 8, "u32"), gu.dev_empty(tokens * 8, "f16")
    hid0 = hid = None
    if with_hidden:
        hid0 = synthetic.hidden_rows(seed + 7, tokens, cfg.d)
        if not f16:
            hid0 = orc.f16_bits_to_f32(hid0).astype(np.float32)
        hid = gu.to_dev(hid0.copy())
    moe.layer_prefill(0, gu.to_dev(x), tokens, hidden=hid, y_out=y, out_idx=idx, out_w=w)
    moe.synchronize()
    conv = (lambda t: orc.f16_bits_to_f32(gu.from_dev(t, np.uint16))) if f16 else (lambda t: t.cpu().numpy())
    got = conv(y).reshape(tokens, cfg.d)
    got_hid = conv(hid).reshape(tokens, cfg.d) if with_hidden else None
    return (moe, dl, x, got, gu.from_dev(idx, np.uint32).reshape(tokens, 8), gu.from_dev(w, np.uint16).reshape(tokens, 8),
            hid0, got_hid)


def _check_rows(host, cfg, x, got, got_idx, rows, tol_gpu, hid0=None, got_hid=None, tol_cpu=FFN_TOL):
    """-> (rows that needed the escape below, the worst error against the CPU path among them, worst error overall)"""
    L, keep = gu.oracle_layer(host, cfg)
    escapes, worst_escape, worst = 0, 0.0, 0.0
    for t in rows:
        xr = np.ascontiguousarray(x[t])
        o_idx, o_w, o_y, o_hid = gu.oracle_prefill_row(L, cfg, xr, None if hid0 is None else hid0[t])
        _, _, _, margin, cpu = gu.oracle_decode(L, cfg, xr)
        assert margin > 1e-5, f"row {t}: router decision margin {margin} too small for an exact-index test"
        assert got_idx[t].tolist() == o_idx.tolist(), f"row {t}"
        assert np.all(np.isfinite(got[t]))
        # The bound against the fp32 CPU path is 1e-3.  On a few cancellation-heavy rows the reference's OWN shader
        # semantics (activations rounded to half) sit further than that from its CPU path; there the CUDA path is
        # held to the shader semantics' distance plus 2e-4 instead.
        own = orc.rel_error(o_y, cpu)
        err = orc.rel_error(got[t], cpu)
        worst = max(worst, err)
        if err >= tol_cpu:
            escapes += 1
            worst_escape = max(worst_escape, err)
        assert err < max(tol_cpu, own + 2e-4), f"row {t} vs the reference CPU path"
        assert orc.rel_error(got[t], o_y) < tol_gpu, f"row {t} vs the shader-semantics oracle"
        if got_hid is not None:
            assert orc.rel_error(got_hid[t], o_hid) < tol_gpu, f"row {t}: hidden"
    if escapes:
        print(f"[parity] {escapes} of {len(list(rows))} rows above {tol_cpu:g} against the CPU path (worst {worst_escape:.3g}): "
              "on those the reference's own shader semantics are further than that from its CPU path")
    return escapes, worst_escape, worst


# 8-bit weights on the tensor cores are an opt-in (NVMAI_CUDA_PREFILL_TC8=1): 8-bit codes times a scale need more
# than fp16's 11 bits, so that path is held to 5e-3 here; by default 8-bit prefill calls run the exact kernels.
TC8_TOL = 5e-3


@pytest.mark.parametrize("bits,meta,tc8", [(4, fmt.META_BF16, False), (4, fmt.META_FP16, False), (8, fmt.META_FP16, False),
                                           (8, fmt.META_FP16, True)])
def test_prefill_small_shape_every_row(bits, meta, tc8, monkeypatch):
    """D 256, F 128, 32 experts, 40 rows (ragged items: about 10 rows per expert)"""
    if not tc8 and bits == 8:
        monkeypatch.setenv("NVMAI_CUDA_PREFILL_TC", "0")
    host, cfg = _case(bits, meta, fmt.OUT_FP32, 40, seed=300 + bits)
    moe, dl, x, got, got_idx, got_w, _, _ = _run_prefill(host, cfg, 40, seed=310 + bits)
    tol = TC8_TOL if tc8 else FFN_TOL
    # bf16 scales times the centred 4-bit code are exact in fp16; fp16 scales (11 bits) round once more, which shows
    # against the shader-semantics oracle (1.05e-3 on one row of this case) but stays inside 1e-3 of the CPU path
    tol_gpu = 1.5e-3 if (meta == fmt.META_FP16 and (bits == 4 or tc8)) else tol
    _check_rows(host, cfg, x, got, got_idx, range(40), tol_gpu=tol_gpu, tol_cpu=tol)


def test_prefill_reference_rounding_with_residual():
    """fp16 rounding points of the prefill shaders, affine router and gate, hidden updated in two steps"""
    host, cfg = _case(4, fmt.META_BF16, fmt.OUT_FP16, 24, seed=320, router_kind=fmt.ROUTER_AFFINE8,
                      gate_kind=fmt.ROUTER_AFFINE8)
    moe, dl, x, got, got_idx, got_w, hid0, got_hid = _run_prefill(host, cfg, 24, seed=321, with_hidden=True)
    # against the fp32 CPU path the fp16 rounding points (activations, partials, h2, y) cost about 1e-3 on their
    # own, as they do in the reference's prefill shaders: 2e-3 here, 1e-3 in every fp32-output test
    _check_rows(host, cfg, x, got, got_idx, range(24), tol_gpu=3e-3, hid0=hid0, got_hid=got_hid, tol_cpu=2e-3)


def test_prefill_shared_expert_with_its_own_bit_width(monkeypatch):
    """4-bit routed experts, 8-bit shared expert on the tensor cores: the shared expert cannot ride in the routed
    launches and gets its own"""
    d, f, e, rows = 256, 128, 32, 20
    host = synthetic.layer(390, d=d, f=f, shared_f=f, num_experts=e, routed_bits=4, shared_bits=8, meta=fmt.META_BF16)
    cfg = MoEConfig(d=d, f=f, shared_f=f, num_experts=e, top_k=8, routed_bits=4, shared_bits=8,
                    router_kind=fmt.ROUTER_DENSE_F16, shared_gate_kind=fmt.ROUTER_DENSE_F16, meta_dtype=fmt.META_BF16,
                    activation=fmt.ACT_SILU, out_dtype=fmt.OUT_FP32, max_tokens=rows)
    moe, dl, x, got, got_idx, got_w, _, _ = _run_prefill(host, cfg, rows, seed=391)
    _check_rows(host, cfg, x, got, got_idx, range(rows), tol_gpu=TC8_TOL, tol_cpu=TC8_TOL)


def test_prefill_items_longer_than_one_tile():
    """8 experts and 600 rows: every expert gets all 600 rows, split evenly over 3 work items of 200"""
    host, cfg = _case(4, fmt.META_BF16, fmt.OUT_FP32, 600, seed=330, e=8)
    moe, dl, x, got, got_idx, got_w, _, _ = _run_prefill(host, cfg, 600, seed=331)
    _check_rows(host, cfg, x, got, got_idx, list(range(0, 600, 13)), tol_gpu=1e-3)


@pytest.mark.parametrize("bits,tc8", [(4, False), (8, False), (8, True)])
def test_prefill_benchmark_shape(bits, tc8, monkeypatch):
    """the 35B-A3B layer shape, 512 rows (16 rows per expert on average); sampled rows against the oracle;
    the 8-bit distribution exercises the wide-range activation rows"""
    if not tc8 and bits == 8:
        monkeypatch.setenv("NVMAI_CUDA_PREFILL_TC", "0")
    host, cfg = _case(bits, fmt.META_BF16, fmt.OUT_FP32, 512, seed=340 + bits, d=2048, f=512, e=256)
    moe, dl, x, got, got_idx, got_w, _, _ = _run_prefill(host, cfg, 512, seed=350 + bits)
    assert np.all(np.isfinite(got))
    tol = TC8_TOL if tc8 else FFN_TOL
    _check_rows(host, cfg, x, got, got_idx, [0, 1, 17, 255, 256, 511], tol_gpu=tol, tol_cpu=tol)


def test_prefill_benchmark_chunk_4096_rows():
    """The benchmark's prefill chunk itself: 4096 rows through one 4-bit layer of the 35B-A3B shape (items of
    128-256 rows: the whole-accumulator path, a B ring that wraps a dozen times over the 36 K blocks).  Rows of the
    largest and the smallest work items and a spread of others, against both oracles; indices exact."""
    tokens = 4096
    host, cfg = _case(4, fmt.META_BF16, fmt.OUT_FP32, tokens, seed=344, d=2048, f=512, e=256)
    moe, dl, x, got, got_idx, got_w, _, _ = _run_prefill(host, cfg, tokens, seed=354)
    assert np.all(np.isfinite(got))
    counts = np.bincount(got_idx.reshape(-1), minlength=256)
    assert counts.max() > 128, "no work item longer than one 128-row accumulator: the test would not cover that path"
    hot, cold = int(np.argmax(counts)), int(np.argmin(np.where(counts > 0, counts, 1 << 30)))
    rows_hot = np.nonzero((got_idx == hot).any(axis=1))[0]
    rows_cold = np.nonzero((got_idx == cold).any(axis=1))[0]
    rows = sorted(set([0, 1, 127, 128, 1000, 2047, 2048, 3333, 4094, 4095] + rows_hot[[0, len(rows_hot) // 2, -1]].tolist()
                      + rows_cold[[0, -1]].tolist() + list(range(300, 4096, 511))))
    assert len(rows) >= 16
    escapes, worst_escape, worst = _check_rows(host, cfg, x, got, got_idx, rows, tol_gpu=FFN_TOL)
    assert escapes <= len(rows) // 4, f"{escapes} of {len(rows)} sampled rows needed the shader-semantics escape"


def test_prefill_equals_decode_path_within_tolerance():
    """the batched decode path and the prefill path on the same 64 rows"""
    host, cfg = _case(4, fmt.META_BF16, fmt.OUT_FP32, 64, seed=360)
    moe, dl, x, got, got_idx, got_w, _, _ = _run_prefill(host, cfg, 64, seed=361)
    h2 = gu.dev_empty(64 * cfg.d, "f32")
    idx = gu.dev_empty(64 * 8, "u32")
    moe.layer_decode(0, gu.to_dev(x), 64, h2_out=h2, out_idx=idx)
    moe.synchronize()
    assert np.array_equal(gu.from_dev(idx, np.uint32).reshape(64, 8), got_idx)
    dec = h2.cpu().numpy().reshape(64, cfg.d)
    for t in range(64):
        assert orc.rel_error(got[t], dec[t]) < FFN_TOL


def test_prefill_deterministic():
    host, cfg = _case(4, fmt.META_BF16, fmt.OUT_FP32, 33, seed=370)
    moe, dl, x, got, *_ = _run_prefill(host, cfg, 33, seed=371)
    y = gu.dev_empty(33 * cfg.d, "f32")
    moe.layer_prefill(0, gu.to_dev(x), 33, y_out=y)
    moe.synchronize()
    assert np.array_equal(y.cpu().numpy().reshape(33, cfg.d).view(np.uint32), got.view(np.uint32))


def test_prefill_wait_that_runs_out_frees_tensor_memory_and_the_next_call_runs():
    """a bounded wait of the tensor-core GEMM made to run out from the host side (one block leaves out one copy of its
    own activation rows; nothing faults): the block sets the status word, frees its tensor memory and returns,
    synchronize reports the timeout once, and the same call then gives the same bits as before"""
    from nvmai_b200 import _lib
    from nvmai_b200.moe import debug_set_wait_limit
    host, cfg = _case(4, fmt.META_BF16, fmt.OUT_FP32, 96, seed=390)
    moe, dl, x, good, *_ = _run_prefill(host, cfg, 96, seed=391)
    xd = gu.to_dev(x)
    y = gu.dev_empty(96 * cfg.d, "f32")
    debug_set_wait_limit(20_000_000)            # 20 ms instead of a second
    try:
        moe.debug_drop_prefill_copy()
        moe.layer_prefill(0, xd, 96, y_out=y)
        with pytest.raises(_lib.NvmaiError) as err:
            moe.synchronize()
        assert err.value.code == _lib.ETIMEOUT
    finally:
        debug_set_wait_limit(0)
    moe.layer_prefill(0, xd, 96, y_out=y)        # tensor memory was released: the blocks of this call can allocate it
    moe.synchronize()
    assert np.array_equal(y.cpu().numpy().reshape(96, cfg.d).view(np.uint32), good.view(np.uint32))


@pytest.mark.parametrize("bits", [4, 8])
def test_prefill_shape_of_the_reference_test_runs_on_the_grouped_kernels(bits):
    """PrefillGroupedRoutedMoETests+Execution.swift:8-109 runs d = f = 64, 3 tokens, top-2 of 16 experts, 4- and 8-bit:
    smaller than a tensor-core tile, so the chunk takes the exact grouped kernels (every output compared)"""
    d, f, e, k, rows = 64, 64, 16, 2, 3
    host = synthetic.layer(380 + bits, d=d, f=f, shared_f=f, num_experts=e, routed_bits=bits, meta=fmt.META_BF16)
    cfg = MoEConfig(d=d, f=f, shared_f=f, num_experts=e, top_k=k, routed_bits=bits, shared_bits=bits,
                    router_kind=fmt.ROUTER_DENSE_F16, shared_gate_kind=fmt.ROUTER_DENSE_F16, meta_dtype=fmt.META_BF16,
                    activation=fmt.ACT_SILU, out_dtype=fmt.OUT_FP16 if bits == 4 else fmt.OUT_FP32, max_tokens=rows)
    moe = MoE(cfg)
    dl = gu.DeviceLayer(host)
    dl.register(moe, 0)
    x = synthetic.hidden_rows(381, rows, cfg.d)
    f16 = cfg.out_dtype == fmt.OUT_FP16
    y = gu.dev_empty(rows * cfg.d, "f16" if f16 else "f32")
    idx = gu.dev_empty(rows * k, "u32")
    hid0 = synthetic.hidden_rows(382, rows, cfg.d)
    hid_host = hid0 if f16 else orc.f16_bits_to_f32(hid0).astype(np.float32)
    hid = gu.to_dev(hid_host.copy())
    moe.layer_prefill(0, gu.to_dev(x), rows, hidden=hid, y_out=y, out_idx=idx)
    moe.synchronize()
    conv = (lambda t: orc.f16_bits_to_f32(gu.from_dev(t, np.uint16))) if f16 else (lambda t: t.cpu().numpy())
    got, got_hid = conv(y).reshape(rows, d), conv(hid).reshape(rows, d)
    got_idx = gu.from_dev(idx, np.uint32).reshape(rows, k)
    L, keep = gu.oracle_layer(host, cfg)
    for t in range(rows):
        o_idx, _, o_y, o_hid = gu.oracle_prefill_row(L, cfg, np.ascontiguousarray(x[t]), hid_host[t])
        assert got_idx[t].tolist() == o_idx.tolist()
        assert orc.rel_error(got[t], o_y) < (3e-3 if f16 else 5e-4)
        assert orc.rel_error(got_hid[t], o_hid) < (3e-3 if f16 else 5e-4)
