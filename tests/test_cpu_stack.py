"""The threaded CPU driver behind the bench's CPU baseline (oracle/cpu_stack.cpp): the same bits whatever the thread
count, and the arithmetic of CPUExpertFFN.accumulate (CPUExpertFFN.swift:101-139) restated here step by step with
the oracle's own GEMV, router and selection."""
import ctypes as C
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
for p_ in (ROOT, ROOT / "tests"):
    if str(p_) not in sys.path:
        sys.path.insert(0, str(p_))

from nvmai_b200 import format as fmt  # noqa: E402
from oracle import oracle as orc  # noqa: E402

D, F, E, K, LAYERS, BITS = 256, 128, 32, 8, 3, 4


def _stack(seed=11):
    rng = np.random.default_rng(seed)
    off, stride = fmt.expert_offsets(D, F, BITS)
    blobs = rng.integers(0, 256, size=(LAYERS, K + 1, stride), dtype=np.uint8)
    gate_m, down_m = F * (D // 64), D * (F // 64)
    for name, n in (("gate", gate_m), ("up", gate_m), ("down", down_m)):
        s = rng.uniform(0.005, 0.02, size=(LAYERS, K + 1, n)).astype(np.float32)
        b = (-7.5 * s * rng.uniform(0.9, 1.1, size=s.shape)).astype(np.float32)
        for suffix, vals in (("_s", s), ("_b", b)):
            bits = fmt.f32_to_bf16_bits(vals)
            o = off[name + suffix]
            blobs[:, :, o:o + 2 * n] = bits.view(np.uint8).reshape(LAYERS, K + 1, 2 * n)
    routers = fmt.f32_to_f16_bits(rng.normal(0.0, 0.05, size=(LAYERS, E, D)))
    gates = fmt.f32_to_f16_bits(rng.normal(0.0, 0.05, size=(LAYERS, D)))
    xs = fmt.f32_to_f16_bits(rng.normal(size=(2, D)))
    desc = orc.StackDesc()
    desc.d, desc.f, desc.e, desc.k, desc.bits, desc.layers, desc.stride = D, F, E, K, BITS, LAYERS, stride
    for i, name in enumerate(fmt.OFFSET_NAMES):
        desc.off[i] = off[name]
    ptrs = [(C.c_void_p * LAYERS)(*[a[l].ctypes.data for l in range(LAYERS)]) for a in (blobs, routers, gates)]
    desc.blobs, desc.router_f16, desc.gate_f16 = (C.cast(p, C.POINTER(C.c_void_p)) for p in ptrs)
    return desc, (blobs, routers, gates, xs, ptrs, off)


def _run(desc, xs, threads):
    y = np.zeros(D, dtype=np.float32)
    sec = orc.cpu_stack_lib().orc_cpu_stack_time(C.byref(desc), threads, 1, 0, xs.ctypes.data, 1, y.ctypes.data, None)
    assert sec > 0
    return y


def _gemv(blob, off, which, x, rows, n):
    names = (("gate_w", "gate_s", "gate_b"), ("up_w", "up_s", "up_b"), ("down_w", "down_s", "down_b"))[which]
    out = np.zeros(rows, dtype=np.float32)
    base = blob.ctypes.data
    orc.lib().orc_affine_gemv_f32(BITS, orc.META_BF16, base + off[names[0]], base + off[names[1]], base + off[names[2]],
                                  orc.ptr(x), rows, n, orc.ptr(out))
    return out


def _restated(keep):
    blobs, routers, gates, xs, _, off = keep
    lib = orc.lib()
    x16 = xs[0].copy()
    y = None
    for l in range(LAYERS):
        x = orc.f16_bits_to_f32(x16).astype(np.float32)
        logits = np.zeros(E, dtype=np.float32)
        lib.orc_router_logits_dense_f16(orc.ptr(routers[l]), orc.ptr(x16), None, E, D, orc.ptr(logits), None)
        idx = np.zeros(K, dtype=np.uint32)
        w = np.zeros(K, dtype=np.float32)
        lib.orc_topk_softmax(orc.ptr(logits), E, K, None, orc.ptr(idx), None, orc.ptr(w), None)
        g = np.float32(0.0)
        gate_row = orc.f16_bits_to_f32(gates[l]).astype(np.float32)
        for i in range(D):
            g = np.float32(g + gate_row[i] * x[i])
        sig = np.float32(1.0) / (np.float32(1.0) + np.exp(-g, dtype=np.float32))
        downs = []
        for e in range(K + 1):          # slot k reads blob k; blob K is the shared expert
            gv = _gemv(blobs[l, e], off, 0, x, F, D)
            uv = _gemv(blobs[l, e], off, 1, x, F, D)
            act = (gv / (np.float32(1.0) + np.exp(-gv, dtype=np.float32)) * uv).astype(np.float32)
            downs.append(_gemv(blobs[l, e], off, 2, act, D, F))
        y = (sig * downs[K]).astype(np.float32)
        for s in range(K):
            y = (y + w[s] * downs[s]).astype(np.float32)
        scale = np.float32(1.0 / np.sqrt(np.sum(y.astype(np.float64) ** 2) / D + 1e-6))
        x16 = orc.f32_to_f16_bits((y * scale).astype(np.float32))
    return y


def test_thread_count_does_not_change_a_bit():
    desc, keep = _stack()
    one = _run(desc, keep[3], 1)
    assert np.all(np.isfinite(one)) and np.abs(one).max() > 0
    for threads in (2, 3, 8):
        assert np.array_equal(_run(desc, keep[3], threads).view(np.uint32), one.view(np.uint32)), threads


def test_driver_follows_the_reference_cpu_accumulation():
    desc, keep = _stack(seed=12)
    got = _run(desc, keep[3], 4)
    want = _restated(keep)
    assert orc.rel_error(got, want) < 1e-5
