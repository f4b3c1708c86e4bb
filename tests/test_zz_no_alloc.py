"""The allocation-free router entry point against the handle-based one.

Some hosts cannot allocate when they call the router: an inference server that
reserved all of HBM for its own arena before the first token, or a decode loop
that must not trigger cudaMalloc's device-wide serialisation.  For them the
library has nvmai_cuda_moe_router_noalloc, whose scratch is a fixed array inside
the library image.  This test drives it through the C ABI twice in a row (the
second call meets whatever the first left in the shared array) and demands the
same bits as nvmai_cuda_moe_router.  It sits in a file that sorts last so that a
run stopping at the first failure has already been through everything else.
"""
import numpy as np
import pytest

import gpu_util as gu
from nvmai_b200 import MoE, MoEConfig, NvmaiError, router_noalloc, synthetic
from nvmai_b200 import _lib
from nvmai_b200 import format as fmt
from nvmai_b200.moe import router_noalloc_status
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _oracle_route(router_host, router_kind, meta, pes_bits, x_row, e, d, k):
    """indices, fp16 weights and decision margin of one row from the CPU oracle"""
    lib = orc.lib()
    logits = np.zeros(e, dtype=np.float32)
    w, s, b = router_host
    if router_kind == fmt.ROUTER_DENSE_F16:
        lib.orc_router_logits_dense_f16(orc.ptr(w), orc.ptr(x_row), None, e, d, orc.ptr(logits), None)
    else:
        lib.orc_router_logits_affine(router_kind, meta, orc.ptr(w), orc.ptr(s), orc.ptr(b), orc.ptr(x_row), None, e, d,
                                     orc.ptr(logits), None)
    idx = np.zeros(k, dtype=np.uint32)
    w16 = np.zeros(k, dtype=np.uint16)
    margin = np.zeros(1, dtype=np.float32)
    lib.orc_topk_softmax(orc.ptr(logits), e, k, orc.ptr(pes_bits), orc.ptr(idx), orc.ptr(w16), None, orc.ptr(margin))
    return idx, w16, float(margin[0]), float(np.max(np.abs(logits)))


# the small shapes are the ones whose staged rows are smaller than the selection scratch laid over them
@pytest.mark.parametrize("router_kind,meta,d,e", [(fmt.ROUTER_DENSE_F16, fmt.META_FP16, 2048, 256),
                                                  (fmt.ROUTER_AFFINE8, fmt.META_BF16, 2048, 256),
                                                  (fmt.ROUTER_AFFINE4, fmt.META_BF16, 64, 40),
                                                  (fmt.ROUTER_AFFINE4, fmt.META_FP16, 128, 256),
                                                  (fmt.ROUTER_AFFINE8, fmt.META_BF16, 64, 16)])
def test_noalloc_router_matches_handle_router_on_two_calls_in_a_row(router_kind, meta, d, e):
    torch = gu.torch_cuda()
    k = 8
    cfg = MoEConfig(d=d, f=64, shared_f=0, num_experts=e, top_k=k, routed_bits=4, shared_bits=4,
                    router_kind=router_kind, shared_gate_kind=fmt.GATE_NONE, meta_dtype=meta, max_tokens=64)
    rng = np.random.default_rng(2024)
    if router_kind == fmt.ROUTER_DENSE_F16:
        router_host = (fmt.f32_to_f16_bits(rng.normal(0.0, 0.02, size=(e, d))), None, None)
    else:
        router_host = synthetic.affine_tensor(rng, e, d, router_kind, meta)
    router = gu.dev_tensor3(router_host)
    pes_host = fmt.f32_to_bf16_bits(rng.uniform(0.6, 1.4, size=e).astype(np.float32))
    pes = gu.to_dev(pes_host)
    moe = MoE(cfg)
    off, stride = fmt.expert_offsets(d, 64, 4)
    dummy = gu.dev_empty(stride * 2, "u8")      # the router never touches the expert blobs
    moe.register_layer(0, experts=dummy, expert_stride=0, offsets=off, router=router, per_expert_scale=pes)

    for call, tokens in enumerate((37, 5)):     # second call: fewer rows, stale logits beyond them in the array
        x_host = synthetic.hidden_rows(300 + call, tokens, d)
        x = gu.to_dev(x_host)
        want_idx, want_w = gu.dev_empty(tokens * k, "u32"), gu.dev_empty(tokens * k, "f16")
        moe.encode_router(0, x, want_idx, want_w, tokens=tokens)
        got_idx = gu.to_dev(np.full(tokens * k, 0xFFFFFFFF, dtype=np.uint32))
        got_w = gu.to_dev(np.full(tokens * k, 0x7E00, dtype=np.uint16))
        router_noalloc(cfg, router, x, got_idx, got_w, tokens=tokens, per_expert_scale=pes)
        router_noalloc_status()                 # waits for the stream; raises if a device-side wait had expired
        torch.cuda.synchronize()
        assert np.array_equal(gu.from_dev(got_idx, np.uint32), gu.from_dev(want_idx, np.uint32)), f"call {call}"
        assert np.array_equal(gu.from_dev(got_w, np.uint16), gu.from_dev(want_w, np.uint16)), f"call {call}"
        # and against the CPU oracle itself: indices exact wherever the decision margin allows an exact test
        got_i = gu.from_dev(got_idx, np.uint32).reshape(tokens, k)
        got_ww = orc.f16_bits_to_f32(gu.from_dev(got_w, np.uint16)).reshape(tokens, k)
        checked = 0
        for t in range(tokens):
            o_idx, o_w, margin, scale = _oracle_route(router_host, router_kind, meta, pes_host,
                                                       np.ascontiguousarray(x_host[t]), e, d, k)
            if margin <= 1e-5 * max(1.0, scale):     # a near tie: fp32 summation order may decide it either way
                continue
            checked += 1
            assert got_i[t].tolist() == o_idx.tolist(), f"call {call} row {t}"
            assert np.max(np.abs(got_ww[t] - orc.f16_bits_to_f32(o_w))) < 5e-3
        assert checked >= tokens // 2


def test_noalloc_router_rejects_batches_beyond_its_fixed_scratch():
    cfg = MoEConfig(d=128, f=64, shared_f=0, num_experts=16, top_k=8, router_kind=fmt.ROUTER_DENSE_F16,
                    shared_gate_kind=fmt.GATE_NONE, max_tokens=1)
    router = (gu.dev_empty(16 * 128, "f16"), None, None)
    x = gu.dev_empty(65 * 128, "f16")
    idx, w = gu.dev_empty(65 * 8, "u32"), gu.dev_empty(65 * 8, "f16")
    with pytest.raises(NvmaiError) as ei:
        router_noalloc(cfg, router, x, idx, w, tokens=65)
    assert ei.value.code == _lib.ERANGE
