"""The one-launch decode step (one resident kernel for all layers of a token) against
the staged kernels (bit for bit), the oracle chain, and its failure path.

The stack driver stands in for attention + norm between two MoE blocks with
x = half(y * rsqrt(mean(y^2) + 1e-6)); the oracle chain below does the same in
float64 from the oracle's own block output.
"""
import numpy as np
import pytest

import gpu_util as gu
from nvmai_b200 import MoE, MoEConfig, NvmaiError, synthetic
from nvmai_b200 import _lib
from nvmai_b200 import format as fmt
from nvmai_b200.moe import debug_set_wait_limit
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _stack(cfg, hosts):
    moe = MoE(cfg)
    devs = [gu.DeviceLayer(h) for h in hosts]
    for l, dv in enumerate(devs):
        dv.register(moe, l)
    return moe, devs


def _run(moe, cfg, x0_dev, mode, stream):
    esz = "f16" if cfg.out_dtype == fmt.OUT_FP16 else "f32"
    y = gu.dev_empty(cfg.d, esz)
    moe.set_decode_mode(mode)
    moe.stack_decode(x0_dev, 1, y, stream=stream)
    moe.synchronize(stream)
    raw = gu.from_dev(y, np.uint16 if esz == "f16" else np.uint32).copy()
    val = orc.f16_bits_to_f32(raw) if esz == "f16" else raw.view(np.float32)
    return raw, val


def _oracle_chain(cfg, hosts, x_row):
    """-> (per-layer expert indices, last layer's block output (shader semantics), minimum router margin)"""
    x = np.ascontiguousarray(x_row)
    idxs, margin_min = [], np.inf
    h2 = None
    for l, host in enumerate(hosts):
        L, keep = gu.oracle_layer(host, cfg)
        idx, _, h2, margin, _ = gu.oracle_decode(L, cfg, x)
        idxs.append(idx.copy())
        margin_min = min(margin_min, margin)
        if l + 1 < len(hosts):
            scale = 1.0 / np.sqrt(np.mean(h2.astype(np.float64) ** 2) + 1e-6)
            x = orc.f32_to_f16_bits((h2.astype(np.float64) * scale).astype(np.float32))
    return idxs, h2, margin_min


# the resident kernel fetches whole 128-byte lines per weight row: 4-bit shapes are multiples of 256, 8-bit of 128
SMALL = [
    # bits, meta, out, router kind, gate kind, d, f, shared_f, experts, activation
    (4, fmt.META_BF16, fmt.OUT_FP32, fmt.ROUTER_DENSE_F16, fmt.ROUTER_DENSE_F16, 256, 256, 256, 32, fmt.ACT_SILU),
    (8, fmt.META_FP16, fmt.OUT_FP32, fmt.ROUTER_DENSE_F16, fmt.ROUTER_DENSE_F16, 256, 128, 128, 32, fmt.ACT_SILU),
    (4, fmt.META_BF16, fmt.OUT_FP16, fmt.ROUTER_AFFINE8, fmt.ROUTER_AFFINE8, 512, 256, 512, 48, fmt.ACT_SILU),
    (8, fmt.META_BF16, fmt.OUT_FP32, fmt.ROUTER_AFFINE4, fmt.GATE_NONE, 384, 128, 128, 16, fmt.ACT_GELU_TANH),
    (4, fmt.META_BF16, fmt.OUT_FP16, fmt.ROUTER_AFFINE4, fmt.GATE_NONE, 256, 256, 256, 16, fmt.ACT_GELU_TANH),
    (4, fmt.META_FP16, fmt.OUT_FP32, fmt.ROUTER_AFFINE4, fmt.ROUTER_AFFINE4, 256, 256, 0, 16, fmt.ACT_SILU),
    (4, fmt.META_BF16, fmt.OUT_FP32, fmt.ROUTER_DENSE_F16, fmt.ROUTER_AFFINE8, 1024, 512, 256, 256, fmt.ACT_SILU),
]


@pytest.mark.parametrize("case", SMALL, ids=lambda c: f"b{c[0]}m{c[1]}o{c[2]}r{c[3]}g{c[4] & 0xFF}d{c[5]}")
def test_resident_step_equals_staged_kernels_bitwise(case):
    bits, meta, out, rkind, gkind, d, f, fs, e, act = case
    layers = 3
    cfg = MoEConfig(d=d, f=f, shared_f=fs, num_experts=e, top_k=8, routed_bits=bits, shared_bits=bits,
                    router_kind=rkind, shared_gate_kind=gkind, meta_dtype=meta, activation=act, out_dtype=out,
                    max_tokens=1, num_layers=layers)
    hosts = [synthetic.layer(900 + 7 * l + bits, d=d, f=f, shared_f=fs, num_experts=e, routed_bits=bits, meta=meta,
                             router_kind=rkind, gate_kind=gkind) for l in range(layers)]
    moe, devs = _stack(cfg, hosts)
    x0 = synthetic.hidden_rows(1000 + d, 1, d)
    torch = gu.torch_cuda()
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        xd = gu.to_dev(x0)
        st.synchronize()
        staged_raw, staged = _run(moe, cfg, xd, MoE.DECODE_STAGED, st)
        res_raw, res = _run(moe, cfg, xd, MoE.DECODE_RESIDENT, st)
        res_raw2, _ = _run(moe, cfg, xd, MoE.DECODE_RESIDENT, st)       # a second step: the epoch has moved on
    assert np.all(np.isfinite(res))
    assert np.array_equal(res_raw, staged_raw), "resident kernel and staged kernels differ"
    assert np.array_equal(res_raw, res_raw2), "second step differs from the first"
    idxs, h2, margin = _oracle_chain(cfg, hosts, x0[0])
    assert margin > 1e-5, "router decision margin too small for an exact-index test: change the seed"
    log = moe.read_route_log()
    for l in range(layers):
        assert log[l].tolist() == idxs[l].tolist(), f"layer {l}: selected experts differ from the oracle"
    assert orc.rel_error(res, h2) < (4e-3 if out == fmt.OUT_FP16 else 2e-3)


@pytest.mark.parametrize("bits", [4, 8])
def test_resident_step_full_shape_against_oracle_chain(bits):
    """The benchmark's shape (D 2048, F 512, 256 experts, top-8, shared expert, dense router), 4 layers."""
    layers, d, f, e = 4, 2048, 512, 256
    cfg = MoEConfig(d=d, f=f, shared_f=f, num_experts=e, top_k=8, routed_bits=bits, shared_bits=bits,
                    router_kind=fmt.ROUTER_DENSE_F16, shared_gate_kind=fmt.ROUTER_DENSE_F16, meta_dtype=fmt.META_BF16,
                    out_dtype=fmt.OUT_FP32, max_tokens=1, num_layers=layers)
    hosts = [synthetic.layer(5000 + 3 * l + bits, d=d, f=f, shared_f=f, num_experts=e, routed_bits=bits,
                             meta=fmt.META_BF16) for l in range(layers)]
    moe, devs = _stack(cfg, hosts)
    x0 = synthetic.hidden_rows(78 + bits, 1, d)
    torch = gu.torch_cuda()
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        xd = gu.to_dev(x0)
        st.synchronize()
        staged_raw, _ = _run(moe, cfg, xd, MoE.DECODE_STAGED, st)
        res_raw, res = _run(moe, cfg, xd, MoE.DECODE_RESIDENT, st)
    assert np.array_equal(res_raw, staged_raw)
    idxs, h2, margin = _oracle_chain(cfg, hosts, x0[0])
    assert margin > 1e-5
    log = moe.read_route_log()
    for l in range(layers):
        assert log[l].tolist() == idxs[l].tolist()
    assert orc.rel_error(res, h2) < 2e-3
    # the last layer alone against the reference CPU path (fp32, 1e-3): its input is the oracle chain's own row
    x = np.ascontiguousarray(x0[0])
    for l, host in enumerate(hosts):
        L, keep = gu.oracle_layer(host, cfg)
        _, _, h2l, _, cpu = gu.oracle_decode(L, cfg, x)
        if l + 1 < layers:
            scale = 1.0 / np.sqrt(np.mean(h2l.astype(np.float64) ** 2) + 1e-6)
            x = orc.f32_to_f16_bits((h2l.astype(np.float64) * scale).astype(np.float32))
    assert orc.rel_error(h2, cpu) < 1e-3


def test_resident_mode_refuses_shapes_it_does_not_cover():
    cfg = MoEConfig(d=128, f=64, shared_f=64, num_experts=16, top_k=8, routed_bits=4, shared_bits=8,
                    meta_dtype=fmt.META_BF16, out_dtype=fmt.OUT_FP32, max_tokens=1, num_layers=1)
    host = synthetic.layer(1, d=128, f=64, shared_f=64, num_experts=16, routed_bits=4, shared_bits=8, meta=fmt.META_BF16)
    moe, devs = _stack(cfg, [host])
    x = gu.to_dev(synthetic.hidden_rows(2, 1, 128))
    y = gu.dev_empty(128, "f32")
    moe.set_decode_mode(MoE.DECODE_RESIDENT)
    with pytest.raises(NvmaiError) as ei:       # shared and routed bit widths differ, rows shorter than a 128-byte line
        moe.stack_decode(x, 1, y)
    assert ei.value.code == _lib.EINVAL
    moe.set_decode_mode(MoE.DECODE_AUTO)        # the staged kernels take it
    moe.stack_decode(x, 1, y)
    moe.synchronize()
    assert np.all(np.isfinite(y.cpu().numpy()))


def test_bounded_wait_expires_and_the_handle_recovers():
    """A block that never publishes its router logits (host-made: a test hook, nothing faults): every other
    block's wait runs out, synchronize reports the timeout, and the next step is correct again."""
    layers, d, f, e = 2, 256, 256, 32
    cfg = MoEConfig(d=d, f=f, shared_f=f, num_experts=e, top_k=8, routed_bits=4, shared_bits=4,
                    meta_dtype=fmt.META_BF16, out_dtype=fmt.OUT_FP32, max_tokens=1, num_layers=layers)
    hosts = [synthetic.layer(40 + l, d=d, f=f, shared_f=f, num_experts=e, routed_bits=4, meta=fmt.META_BF16)
             for l in range(layers)]
    moe, devs = _stack(cfg, hosts)
    x0 = synthetic.hidden_rows(41, 1, d)
    torch = gu.torch_cuda()
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        xd = gu.to_dev(x0)
        st.synchronize()
        good_raw, _ = _run(moe, cfg, xd, MoE.DECODE_RESIDENT, st)
        debug_set_wait_limit(20_000_000)            # 20 ms
        try:
            moe.debug_mute_block(3)                 # a block that holds a router row and a shared-expert tile
            y = gu.dev_empty(d, "f32")
            moe.stack_decode(xd, 1, y, stream=st)
            with pytest.raises(NvmaiError) as ei:
                moe.synchronize(st)
            assert ei.value.code == _lib.ETIMEOUT
        finally:
            moe.debug_mute_block()
            debug_set_wait_limit(0)
        again_raw, _ = _run(moe, cfg, xd, MoE.DECODE_RESIDENT, st)
    assert np.array_equal(again_raw, good_raw)


# ---------------------------------------------------------------------------------------------------
# a few rows per step: the rows are the columns of the tensor-core step
# ---------------------------------------------------------------------------------------------------

def _run_rows(moe, cfg, x_dev, rows, mode, stream):
    y = gu.dev_empty(rows * cfg.d, "f32")
    moe.set_decode_mode(mode)
    moe.stack_decode(x_dev, rows, y, stream=stream)
    moe.synchronize(stream)
    return y.cpu().numpy().reshape(rows, cfg.d).copy()


@pytest.mark.parametrize("rows,bits,d,f,fs,e,rkind", [(2, 4, 512, 256, 256, 64, fmt.ROUTER_DENSE_F16),
                                                     (5, 8, 256, 128, 256, 32, fmt.ROUTER_AFFINE8),
                                                     (8, 4, 2048, 512, 512, 256, fmt.ROUTER_DENSE_F16)])
def test_resident_rows_one_layer_equals_staged_kernels_bitwise(rows, bits, d, f, fs, e, rkind):
    """one layer (no input norm in play): every row of the batch kernel carries the bits of the staged per-row kernels"""
    cfg = MoEConfig(d=d, f=f, shared_f=fs, num_experts=e, top_k=8, routed_bits=bits, shared_bits=bits, router_kind=rkind,
                    shared_gate_kind=rkind, meta_dtype=fmt.META_BF16, out_dtype=fmt.OUT_FP32, max_tokens=rows, num_layers=1)
    hosts = [synthetic.layer(1200 + bits, d=d, f=f, shared_f=fs, num_experts=e, routed_bits=bits, meta=fmt.META_BF16,
                             router_kind=rkind, gate_kind=rkind)]
    moe, devs = _stack(cfg, hosts)
    x0 = synthetic.hidden_rows(1201 + rows, rows, d)
    torch = gu.torch_cuda()
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        xd = gu.to_dev(x0)
        st.synchronize()
        staged = _run_rows(moe, cfg, xd, rows, MoE.DECODE_STAGED, st)
        res = _run_rows(moe, cfg, xd, rows, MoE.DECODE_RESIDENT, st)
        res2 = _run_rows(moe, cfg, xd, rows, MoE.DECODE_RESIDENT, st)
    assert np.all(np.isfinite(res))
    assert np.array_equal(res.view(np.uint32), staged.view(np.uint32))
    assert np.array_equal(res.view(np.uint32), res2.view(np.uint32))


@pytest.mark.parametrize("rows,bits", [(3, 4), (8, 4), (4, 8)])
def test_resident_rows_stack_against_oracle_chain(rows, bits):
    """three layers: the per-row input norm is the batch kernel's own reduction, so the bar is the oracle chain's"""
    layers, d, f, e = 3, 512, 256, 64
    cfg = MoEConfig(d=d, f=f, shared_f=f, num_experts=e, top_k=8, routed_bits=bits, shared_bits=bits,
                    meta_dtype=fmt.META_BF16, out_dtype=fmt.OUT_FP32, max_tokens=rows, num_layers=layers)
    hosts = [synthetic.layer(1300 + 5 * l + bits, d=d, f=f, shared_f=f, num_experts=e, routed_bits=bits, meta=fmt.META_BF16)
             for l in range(layers)]
    moe, devs = _stack(cfg, hosts)
    x0 = synthetic.hidden_rows(1301 + rows, rows, d)
    torch = gu.torch_cuda()
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        xd = gu.to_dev(x0)
        st.synchronize()
        res = _run_rows(moe, cfg, xd, rows, MoE.DECODE_RESIDENT, st)
        staged = _run_rows(moe, cfg, xd, rows, MoE.DECODE_STAGED, st)
    checked = []
    for t in range(rows):
        idxs, h2, margin = _oracle_chain(cfg, hosts, x0[t])
        if margin <= 1e-5 or np.abs(h2).max() < 1e-20:
            continue        # a degenerate chain (tie, or a layer that came out all zero) tests nothing
        assert orc.rel_error(res[t], h2) < 2e-3, f"row {t} vs the oracle chain"
        assert orc.rel_error(res[t], staged[t]) < 1e-4, f"row {t} vs the staged kernels"
        checked.append((t, idxs))
    # the step's own routing record, and its dump in the reference's NVMAI_ROUTE_TRACE line format
    from nvmai_b200 import route_trace as rt
    log = moe.read_route_log_rows(rows)
    assert log.shape == (layers, rows, 8)
    for t, idxs in checked:
        for l in range(layers):
            np.testing.assert_array_equal(log[l, t], idxs[l])
    text = rt.from_route_log(log, 100, num_experts=e).format()
    back = rt.parse(text, num_experts=e, top_k=8)
    assert len(back) == layers * rows
    for t in range(rows):
        for l in range(layers):
            np.testing.assert_array_equal(back.batch(l, t, 1)[0], log[l, t])
