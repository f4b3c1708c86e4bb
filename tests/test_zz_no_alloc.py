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

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("router_kind,meta", [(fmt.ROUTER_DENSE_F16, fmt.META_FP16), (fmt.ROUTER_AFFINE8, fmt.META_BF16)])
def test_noalloc_router_matches_handle_router_on_two_calls_in_a_row(router_kind, meta):
    torch = gu.torch_cuda()
    d, e, k = 2048, 256, 8
    cfg = MoEConfig(d=d, f=64, shared_f=0, num_experts=e, top_k=k, routed_bits=4, shared_bits=4,
                    router_kind=router_kind, shared_gate_kind=fmt.GATE_NONE, meta_dtype=meta, max_tokens=64)
    rng = np.random.default_rng(2024)
    if router_kind == fmt.ROUTER_DENSE_F16:
        router_host = (fmt.f32_to_f16_bits(rng.normal(0.0, 0.02, size=(e, d))), None, None)
    else:
        router_host = synthetic.affine_tensor(rng, e, d, router_kind, meta)
    router = gu.dev_tensor3(router_host)
    pes = gu.to_dev(fmt.f32_to_bf16_bits(rng.uniform(0.6, 1.4, size=e).astype(np.float32)))
    moe = MoE(cfg)
    off, stride = fmt.expert_offsets(d, 64, 4)
    dummy = gu.dev_empty(stride * 2, "u8")      # the router never touches the expert blobs
    moe.register_layer(0, experts=dummy, expert_stride=0, offsets=off, router=router, per_expert_scale=pes)

    for call, tokens in enumerate((37, 5)):     # second call: fewer rows, stale logits beyond them in the array
        x = gu.to_dev(synthetic.hidden_rows(300 + call, tokens, d))
        want_idx, want_w = gu.dev_empty(tokens * k, "u32"), gu.dev_empty(tokens * k, "f16")
        moe.encode_router(0, x, want_idx, want_w, tokens=tokens)
        got_idx = gu.to_dev(np.full(tokens * k, 0xFFFFFFFF, dtype=np.uint32))
        got_w = gu.to_dev(np.full(tokens * k, 0x7E00, dtype=np.uint16))
        router_noalloc(cfg, router, x, got_idx, got_w, tokens=tokens, per_expert_scale=pes)
        torch.cuda.synchronize()
        assert np.array_equal(gu.from_dev(got_idx, np.uint32), gu.from_dev(want_idx, np.uint32)), f"call {call}"
        assert np.array_equal(gu.from_dev(got_w, np.uint16), gu.from_dev(want_w, np.uint16)), f"call {call}"


def test_noalloc_router_rejects_batches_beyond_its_fixed_scratch():
    cfg = MoEConfig(d=128, f=64, shared_f=0, num_experts=16, top_k=8, router_kind=fmt.ROUTER_DENSE_F16,
                    shared_gate_kind=fmt.GATE_NONE, max_tokens=1)
    router = (gu.dev_empty(16 * 128, "f16"), None, None)
    x = gu.dev_empty(65 * 128, "f16")
    idx, w = gu.dev_empty(65 * 8, "u32"), gu.dev_empty(65 * 8, "f16")
    with pytest.raises(NvmaiError) as ei:
        router_noalloc(cfg, router, x, idx, w, tokens=65)
    assert ei.value.code == _lib.ERANGE
