"""Child process of test_gpu_ep_failure.py: one rank of a "two-rank" expert-parallel job whose NCCL is the test
double (NVMAI_CUDA_NCCL_LIB), so that nothing waits for a peer.  Prints one JSON line."""
import ctypes
import json
import os
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
for p_ in (ROOT, ROOT / "tests"):
    if str(p_) not in sys.path:
        sys.path.insert(0, str(p_))


def main() -> None:
    scenario = sys.argv[1]
    import torch
    import gpu_util as gu
    from nvmai_b200 import MoE, MoEConfig, synthetic
    from nvmai_b200 import format as fmt
    from nvmai_b200._lib import NvmaiError
    from nvmai_b200.ep import ExpertPlacement
    fake = ctypes.CDLL(os.environ["NVMAI_CUDA_NCCL_LIB"])
    d, f, e, rows = 256, 128, 32, 2
    cfg = MoEConfig(d=d, f=f, shared_f=f, num_experts=e, top_k=8, routed_bits=8, shared_bits=8,
                    router_kind=fmt.ROUTER_DENSE_F16, shared_gate_kind=fmt.ROUTER_DENSE_F16, meta_dtype=fmt.META_FP16,
                    out_dtype=fmt.OUT_FP32, max_tokens=2 * rows, num_layers=2)
    moe = MoE(cfg)
    moe.set_decode_mode(1)          # the staged kernels with NCCL collectives between them: what this test is about
    pl = ExpertPlacement(e, 2, "contiguous")
    keep = []
    for l in range(2):
        host = synthetic.layer(700 + l, d=d, f=f, shared_f=f, num_experts=e, routed_bits=8, meta=fmt.META_FP16)
        local = dict(host)
        local["experts"] = np.ascontiguousarray(host["experts"][pl.local_experts(0)])
        dl = gu.DeviceLayer(local)
        dl.register(moe, l)
        keep.append(dl)
    moe.set_expert_map(pl.expert_map(0))
    moe.ep_init(moe.ep_unique_id(), 0, 2, rows)
    st = torch.cuda.Stream()
    x = gu.to_dev(synthetic.hidden_rows(5, rows, d)).view(torch.float16)
    y = torch.empty(rows, d, dtype=torch.float32, device="cuda")
    out = {"scenario": scenario}
    with torch.cuda.stream(st):
        moe.ep_stack_decode(x, rows, y, stream=st)
        moe.ep_synchronize(st, 5000)            # a healthy step first
        out["healthy_polls"] = fake.fake_nccl_polls()
        if scenario == "async_error":           # the double starts to report a remote error forty polls from now
            os.environ["FAKE_NCCL_ASYNC_ERROR_AFTER"] = str(fake.fake_nccl_polls() + 40)
        moe.debug_host_delay(600 if scenario == "timeout" else 300, st)     # the stream stays busy, the device idle
        moe.ep_stack_decode(x, rows, y, stream=st)
        t0 = time.perf_counter()
        try:
            moe.ep_synchronize(st, 150 if scenario == "timeout" else 5000)
            out["code"] = 0
        except NvmaiError as err:
            out["code"] = err.code
        out["waited_s"] = time.perf_counter() - t0
        out["aborts"] = fake.fake_nccl_aborts()
        try:                                     # the expert-parallel state is gone until ep_init
            moe.ep_stack_decode(x, rows, y, stream=st)
            out["after"] = 0
        except NvmaiError as err:
            out["after"] = err.code
        moe.ep_init(moe.ep_unique_id(), 0, 2, rows)
        os.environ.pop("FAKE_NCCL_ASYNC_ERROR_AFTER", None)
        moe.ep_stack_decode(x, rows, y, stream=st)
        moe.ep_synchronize(st, 5000)
        out["recovered"] = bool(torch.isfinite(y).all().item())
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
