"""Host logic of the expert-parallel driver on CPU: two gloo ranks, the CPU oracle as
the arithmetic, against the single-rank oracle.  Also the placement maps and the
host-side failure cases (a rank that raises, a bad placement)."""
import ctypes as C
import os
import sys
import traceback
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
for p_ in (ROOT, ROOT / "tests"):
    if str(p_) not in sys.path:
        sys.path.insert(0, str(p_))

from nvmai_b200 import MoEConfig, synthetic  # noqa: E402
from nvmai_b200 import format as fmt  # noqa: E402
from nvmai_b200.ep import (NOT_LOCAL, ExpertPlacement, ep_layer_step, ep_replicated_stack_step,  # noqa: E402
                           ep_stack_step)

D, F, E, K = 128, 64, 16, 8


def _cfg():
    return MoEConfig(d=D, f=F, shared_f=F, num_experts=E, top_k=K, routed_bits=4, shared_bits=4,
                     router_kind=fmt.ROUTER_DENSE_F16, shared_gate_kind=fmt.ROUTER_AFFINE8, meta_dtype=fmt.META_BF16,
                     out_dtype=fmt.OUT_FP32, max_tokens=8)


def _host_layer():
    return synthetic.layer(77, d=D, f=F, shared_f=F, num_experts=E, routed_bits=4, meta=fmt.META_BF16,
                           gate_kind=fmt.ROUTER_AFFINE8)


class OracleBackend:
    """CPU stand-in for the CUDA library: same interface, oracle arithmetic (shader
    rounding points, fp32 outputs); serves only the experts the placement gives this rank."""

    def __init__(self, host, cfg, placement, rank):
        import gpu_util as gu
        from oracle import oracle as orc
        self.orc, self.host, self.cfg, self.pl, self.rank = orc, host, cfg, placement, rank
        self.L, self.keep = gu.oracle_layer(host, cfg)

    def router(self, layer, x_all):
        import torch
        orc, c = self.orc, self.cfg
        x = x_all.view(torch.int16).numpy().view(np.uint16)
        idx = np.zeros((x.shape[0], K), dtype=np.uint32)
        w = np.zeros((x.shape[0], K), dtype=np.uint16)
        for t in range(x.shape[0]):
            logits = np.zeros(E, dtype=np.float32)
            orc.lib().orc_router_logits_dense_f16(orc.ptr(self.host["router"][0]), orc.ptr(np.ascontiguousarray(x[t])),
                                                  None, E, c.d, orc.ptr(logits), None)
            orc.lib().orc_topk_softmax(orc.ptr(logits), E, K, None, orc.ptr(idx[t]), orc.ptr(w[t]), None, None)
        return torch.from_numpy(idx.view(np.int32)), torch.from_numpy(w.view(np.int16)).view(torch.float16)

    def routed_partial(self, layer, x_all, idx, w):
        import torch
        orc, c = self.orc, self.cfg
        x = x_all.view(torch.int16).numpy().view(np.uint16)
        idx_np = idx.numpy().view(np.uint32)
        w_np = w.view(torch.int16).numpy().view(np.uint16).copy()
        off = np.array([self.host["offsets"][n] for n in fmt.OFFSET_NAMES], dtype=np.uint32)
        share = np.zeros((x.shape[0], c.d), dtype=np.float32)
        for t in range(x.shape[0]):
            wt = w_np[t].copy()
            for k in range(K):
                if self.pl.owner(int(idx_np[t, k])) != self.rank:
                    wt[k] = 0                      # fp16 +0: a slot held elsewhere contributes nothing here
            blobs = (C.c_void_p * K)(*[self.host["experts"][int(e)].ctypes.data for e in idx_np[t]])
            acts = np.zeros(K * c.f, dtype=np.float32)
            orc.lib().orc_gpu_phase1(blobs, orc.ptr(off), 4, c.meta_dtype, c.activation, orc.ptr(np.ascontiguousarray(x[t])),
                                     c.d, c.f, K, None, 0, orc.OUT_FP32, orc.ptr(acts))
            zero = np.zeros(c.d, dtype=np.float32)
            orc.lib().orc_gpu_phase2(blobs, orc.ptr(off), 4, c.meta_dtype, orc.ptr(acts), orc.ptr(wt), orc.ptr(zero),
                                     c.d, c.f, K, orc.OUT_FP32, orc.ptr(share[t]))
        return torch.from_numpy(share)

    def shared(self, layer, x_own):
        import torch
        orc, c = self.orc, self.cfg
        x = x_own.view(torch.int16).numpy().view(np.uint16)
        proj = (C.c_void_p * 9)(*[a.ctypes.data for t in self.host["shared"] for a in t])
        gw, gs, gb = self.host["gate"]
        h1 = np.zeros((x.shape[0], c.d), dtype=np.float32)
        for t in range(x.shape[0]):
            orc.lib().orc_gpu_shared_expert(proj, 4, c.meta_dtype, c.activation, orc.ptr(gw), orc.ptr(gs), orc.ptr(gb), 8,
                                            orc.ptr(np.ascontiguousarray(x[t])), c.d, c.shared_f, orc.OUT_FP32,
                                            orc.ptr(h1[t]))
        return torch.from_numpy(h1)

    def finalize(self, recv, h1, world, b_own):
        y = h1.clone()
        for r in range(world):
            y = y + recv.view(world, b_own, -1)[r]
        return y

    def renorm(self, y):
        import torch
        v = y.numpy().astype(np.float64)
        scale = 1.0 / np.sqrt(np.mean(v * v, axis=1, keepdims=True) + 1e-6)
        bits = self.orc.f32_to_f16_bits((v * scale).astype(np.float32).reshape(-1)).reshape(v.shape)
        return torch.from_numpy(bits.view(np.int16).copy()).view(torch.float16)


def _rank_main(rank, world, port, mode, fail_rank, out_dir):
    try:
        import torch
        import torch.distributed as dist
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        from datetime import timedelta
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=20))
        cfg, host = _cfg(), _host_layer()
        pl = ExpertPlacement(E, world, mode.replace("stack-", ""))
        backend = OracleBackend(host, cfg, pl, rank)
        b_own = 2
        x_all = synthetic.hidden_rows(5, world * b_own, D)
        x_own = torch.from_numpy(x_all[rank * b_own:(rank + 1) * b_own].view(np.int16).copy()).view(torch.float16)
        if rank == fail_rank:
            raise RuntimeError("injected failure before the first collective")
        if mode.startswith("stack-"):
            # two chained layers both ways: rows owned and shares sent to the owners, and every rank keeping all rows
            y = ep_stack_step(backend, dist, None, x_own, world=world, layers=2)
            z = ep_replicated_stack_step(backend, dist, None, x_own, world=world, layers=2)
            np.save(os.path.join(out_dir, f"z{rank}.npy"), z.numpy())
        else:
            y = ep_layer_step(backend, dist, None, 0, x_own, world=world)
        np.save(os.path.join(out_dir, f"y{rank}.npy"), y.numpy())
        dist.destroy_process_group()
    except Exception:
        with open(os.path.join(out_dir, f"err{rank}.txt"), "w") as f:
            f.write(traceback.format_exc())
        sys.exit(3)


def _spawn(world, mode, tmp_path, fail_rank=-1, port=29541):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, mode, fail_rank, str(tmp_path))) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
    codes = []
    for p in procs:
        if p.is_alive():
            p.kill()            # exactly the child this test started
            p.join()
            codes.append(None)
        else:
            codes.append(p.exitcode)
    return codes


@pytest.mark.parametrize("mode", ["contiguous", "strided"])
def test_two_rank_expert_parallel_layer_equals_single_rank_oracle(mode, tmp_path):
    import gpu_util as gu
    from oracle import oracle as orc
    codes = _spawn(2, mode, tmp_path, port=29541 if mode == "contiguous" else 29543)
    errs = [p.read_text() for p in tmp_path.glob("err*.txt")]
    assert codes == [0, 0], errs
    cfg, host = _cfg(), _host_layer()
    L, keep = gu.oracle_layer(host, cfg)
    x_all = synthetic.hidden_rows(5, 4, D)
    for rank in range(2):
        y = np.load(tmp_path / f"y{rank}.npy")
        for j in range(2):
            _, _, want, _, _ = gu.oracle_decode(L, cfg, np.ascontiguousarray(x_all[rank * 2 + j]))
            assert orc.rel_error(y[j], want) < 1e-5, (rank, j)


def test_two_rank_stack_keeping_all_rows_equals_the_owner_exchange_and_the_oracle_chain(tmp_path):
    """the step structure of the fused expert-parallel kernel (every rank keeps all rows, shares added in rank order on
    every rank) against the owner-mode exchange and against one rank running the chain alone"""
    import gpu_util as gu
    from oracle import oracle as orc
    codes = _spawn(2, "stack-strided", tmp_path, port=29547)
    errs = [p.read_text() for p in tmp_path.glob("err*.txt")]
    assert codes == [0, 0], errs
    cfg, host = _cfg(), _host_layer()
    L, keep = gu.oracle_layer(host, cfg)
    x_all = synthetic.hidden_rows(5, 4, D)
    for rank in range(2):
        y, z = np.load(tmp_path / f"y{rank}.npy"), np.load(tmp_path / f"z{rank}.npy")
        for j in range(2):
            assert orc.rel_error(z[j], y[j]) < 1e-6, (rank, j)
            x = np.ascontiguousarray(x_all[rank * 2 + j])
            _, _, h2, _, _ = gu.oracle_decode(L, cfg, x)
            scale = 1.0 / np.sqrt(np.mean(h2.astype(np.float64) ** 2) + 1e-6)
            x = orc.f32_to_f16_bits((h2.astype(np.float64) * scale).astype(np.float32))
            _, _, want, _, _ = gu.oracle_decode(L, cfg, x)
            assert orc.rel_error(z[j], want) < 2e-4, (rank, j)


def test_a_rank_that_raises_does_not_hang_the_others(tmp_path):
    """Failure injected on the host: rank 1 raises before its first collective; rank 0's
    collective ends with an error after the group's short timeout instead of waiting forever."""
    codes = _spawn(2, "contiguous", tmp_path, fail_rank=1, port=29545)
    assert codes[1] == 3
    assert codes[0] not in (0, None), "rank 0 must fail on its collective, not hang"


def test_placement_maps():
    for mode in ("contiguous", "strided"):
        pl = ExpertPlacement(256, 8, mode)
        seen = set()
        for r in range(8):
            m = pl.expert_map(r)
            local = [e for e in range(256) if m[e] != NOT_LOCAL]
            assert len(local) == 32 and sorted(m[e] for e in local) == list(range(32))
            assert local == sorted(pl.local_experts(r)) and [m[e] for e in pl.local_experts(r)] == list(range(32))
            seen.update(local)
        assert seen == set(range(256))
    assert ExpertPlacement(256, 8, "contiguous").owner(33) == 1 and ExpertPlacement(256, 8, "strided").owner(33) == 1
    with pytest.raises(ValueError):
        ExpertPlacement(256, 3)


def test_zipf_load_is_flatter_with_strided_placement():
    """configs[4]: popularity ~ rank^-1.1 over experts; contiguous placement piles the hot
    experts on one rank, strided spreads them."""
    rng = np.random.default_rng(0)
    p = np.arange(1, 257, dtype=np.float64) ** -1.1
    p /= p.sum()
    idx = np.concatenate([rng.choice(256, size=8, replace=False, p=p) for _ in range(256)])
    ratios = {}
    for mode in ("contiguous", "strided"):
        load = ExpertPlacement(256, 8, mode).pairs_per_rank(idx)
        ratios[mode] = max(load) / (sum(load) / 8)
    assert ratios["contiguous"] > 2.0 > ratios["strided"]
