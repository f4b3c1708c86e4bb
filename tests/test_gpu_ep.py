"""Expert-parallel layer on 2 GPUs (NCCL) through the C ABI against the single-rank
oracle.  Needs two devices; skipped on a one-GPU box."""
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

pytestmark = pytest.mark.gpu

D, F, E, K, B_OWN = 256, 128, 32, 8, 3


def _cfg(tokens, bits=8):
    from nvmai_b200 import MoEConfig
    from nvmai_b200 import format as fmt
    return MoEConfig(d=D, f=F, shared_f=F, num_experts=E, top_k=K, routed_bits=bits, shared_bits=bits,
                     router_kind=fmt.ROUTER_DENSE_F16, shared_gate_kind=fmt.ROUTER_DENSE_F16, meta_dtype=fmt.META_FP16,
                     out_dtype=fmt.OUT_FP32, max_tokens=tokens)


def _rank_main(rank, world, port, out_dir):
    try:
        import torch
        import torch.distributed as dist
        import gpu_util as gu
        from nvmai_b200 import MoE, synthetic
        from nvmai_b200 import format as fmt
        from nvmai_b200.ep import ExpertPlacement, LibraryBackend, ep_layer_step
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        host = synthetic.layer(901, d=D, f=F, shared_f=F, num_experts=E, routed_bits=8, meta=fmt.META_FP16)
        pl = ExpertPlacement(E, world, "strided")
        local = dict(host)
        local["experts"] = np.ascontiguousarray(host["experts"][pl.local_experts(rank)])   # only this rank's blobs
        moe = MoE(_cfg(world * B_OWN))
        dl = gu.DeviceLayer(local)
        dl.register(moe, 0)
        moe.set_expert_map(pl.expert_map(rank))
        x_all = synthetic.hidden_rows(902, world * B_OWN, D)
        st = torch.cuda.Stream()
        with torch.cuda.stream(st):
            x_own = gu.to_dev(x_all[rank * B_OWN:(rank + 1) * B_OWN].copy()).view(torch.float16)
            y = ep_layer_step(LibraryBackend(moe, stream=st), dist, None, 0, x_own, world=world)
            st.synchronize()
        np.save(os.path.join(out_dir, f"y{rank}.npy"), y.cpu().numpy())
        _native_stack(rank, world, out_dir, dist, pl, x_all, st)
        dist.destroy_process_group()
    except Exception:
        with open(os.path.join(out_dir, f"err{rank}.txt"), "w") as f:
            f.write(traceback.format_exc())
        sys.exit(3)


def _native_stack(rank, world, out_dir, dist, pl, x_all, st):
    """Two layers through the library's own communicator (plain launches, then the
    captured graph, then a replay) against the torch.distributed-driven step."""
    import torch
    import gpu_util as gu
    from nvmai_b200 import MoE, synthetic
    from nvmai_b200 import format as fmt
    from nvmai_b200.ep import LibraryBackend, ep_stack_step
    # 4-bit weights: with the benchmark's all-positive 8-bit weights a renormalised all-negative row drives every
    # gate to silu(-400) = 0 and the second layer's output is exactly zero (in the oracle too), which tests nothing
    cfg = _cfg(world * B_OWN, bits=4)
    cfg.num_layers = 2
    moe = MoE(cfg)
    keep = []
    for layer in range(2):
        host = synthetic.layer(910 + layer, d=D, f=F, shared_f=F, num_experts=E, routed_bits=4, meta=fmt.META_FP16)
        local = dict(host)
        local["experts"] = np.ascontiguousarray(host["experts"][pl.local_experts(rank)])
        dl = gu.DeviceLayer(local)
        dl.register(moe, layer)
        keep.append(dl)
    moe.set_expert_map(pl.expert_map(rank))
    ids = [moe.ep_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    moe.ep_init(ids[0], rank, world, B_OWN)
    with torch.cuda.stream(st):
        x_own = gu.to_dev(x_all[rank * B_OWN:(rank + 1) * B_OWN].copy()).view(torch.float16)
        want = ep_stack_step(LibraryBackend(moe, stream=st), dist, None, x_own, world=world, layers=2).clone()
        st.synchronize()
        y = torch.empty_like(want)
        outs = []
        # calls 0-2: shares through an NCCL all-gather; then the receive areas are mapped into each other and
        # calls 3-5 send the shares by peer stores from the down stage (plain launches, capture, replay each time).
        # No assertion between the collective calls: a rank that stopped here would hang its peer.
        for call in range(6):
            if call == 3:
                handles = [None] * world
                dist.all_gather_object(handles, moe.ep_peer_export())
                moe.ep_peer_attach(handles)
            y.zero_()
            moe.ep_stack_decode(x_own, B_OWN, y, stream=st)
            moe.synchronize(stream=st)
            outs.append(y.cpu().numpy().copy())
        # the peer exchange with another number of rows in between (its block counters start over every step)
        alt = []
        for rows in (2, B_OWN):
            y.zero_()
            moe.ep_stack_decode(x_own, rows, y, stream=st)
            moe.synchronize(stream=st)
            alt.append(y.cpu().numpy().copy())
        dist.barrier()      # nobody unmaps a receive area a peer may still write
    np.save(os.path.join(out_dir, f"alt{rank}.npy"), np.stack(alt))
    np.save(os.path.join(out_dir, f"want{rank}.npy"), want.cpu().numpy())
    np.save(os.path.join(out_dir, f"calls{rank}.npy"), np.stack(outs))
    np.save(os.path.join(out_dir, f"native{rank}.npy"), y.cpu().numpy())
    moe.ep_shutdown()


def test_two_gpu_expert_parallel_layer_matches_oracle(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    import gpu_util as gu
    from nvmai_b200 import synthetic
    from nvmai_b200 import format as fmt
    from oracle import oracle as orc
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_rank_main, args=(r, 2, 29561, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        if p.is_alive():
            p.kill()
            p.join()
    errs = [p.read_text() for p in tmp_path.glob("err*.txt")]
    assert [p.exitcode for p in procs] == [0, 0], errs
    host = synthetic.layer(901, d=D, f=F, shared_f=F, num_experts=E, routed_bits=8, meta=fmt.META_FP16)
    cfg = _cfg(2 * B_OWN)
    L, keep = gu.oracle_layer(host, cfg)
    x_all = synthetic.hidden_rows(902, 2 * B_OWN, D)
    for rank in range(2):
        y = np.load(tmp_path / f"y{rank}.npy")
        for j in range(B_OWN):
            o_idx, _, want, _, cpu = gu.oracle_decode(L, cfg, np.ascontiguousarray(x_all[rank * B_OWN + j]))
            assert orc.rel_error(y[j], cpu) < 1e-3
            assert orc.rel_error(y[j], want) < 5e-4
        # the library's own communicator: plain launches, graph capture, replay.  Small batches run the replicated mode
        # (per-row kernels, shares all-gathered): the same arithmetic as the torch-driven grouped kernels up to the
        # association of a few fp32 additions
        want_s = np.load(tmp_path / f"want{rank}.npy")
        calls = np.load(tmp_path / f"calls{rank}.npy")
        assert np.all(np.isfinite(want_s)) and np.abs(want_s).max() > 0, "torch-driven reference stack"
        for c in range(6):
            assert np.all(np.isfinite(calls[c])), f"rank {rank} call {c}: non-finite values ({int((~np.isfinite(calls[c])).sum())})"
            err = np.abs(calls[c] - want_s).max() / np.abs(want_s).max()
            assert err < 1e-5, f"rank {rank} call {c}: {err}"
            assert np.array_equal(calls[c].view(np.uint32), calls[0].view(np.uint32)), "plain launches, capture and replay agree bitwise"
        alt = np.load(tmp_path / f"alt{rank}.npy")
        assert np.array_equal(alt[0][:2].view(np.uint32), calls[0][:2].view(np.uint32)), "two rows after three"
        assert np.array_equal(alt[1].view(np.uint32), calls[0].view(np.uint32)), "three rows after two"


# ---------------------------------------------------------------------------------------------------
# the resident kernel with the shares exchanged by peer stores from inside its down phase
# ---------------------------------------------------------------------------------------------------
RD, RF, RE, R_OWN, R_LAYERS = 256, 256, 32, 3, 3


def _resident_cfg(tokens, layers):
    from nvmai_b200 import MoEConfig
    from nvmai_b200 import format as fmt
    return MoEConfig(d=RD, f=RF, shared_f=RF, num_experts=RE, top_k=K, routed_bits=4, shared_bits=4,
                     router_kind=fmt.ROUTER_DENSE_F16, shared_gate_kind=fmt.ROUTER_DENSE_F16, meta_dtype=fmt.META_BF16,
                     out_dtype=fmt.OUT_FP32, max_tokens=tokens, num_layers=layers)


def _resident_hosts():
    from nvmai_b200 import synthetic
    from nvmai_b200 import format as fmt
    return [synthetic.layer(930 + l, d=RD, f=RF, shared_f=RF, num_experts=RE, routed_bits=4, meta=fmt.META_BF16)
            for l in range(R_LAYERS)]


def _rank_resident(rank, world, port, out_dir):
    try:
        import torch
        import torch.distributed as dist
        import gpu_util as gu
        from nvmai_b200 import MoE, synthetic
        from nvmai_b200.ep import ExpertPlacement
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        hosts = _resident_hosts()
        pl = ExpertPlacement(RE, world, "strided")
        T = world * R_OWN
        moe = MoE(_resident_cfg(T, R_LAYERS))
        keep = []
        for l, host in enumerate(hosts):
            local = dict(host)
            local["experts"] = np.ascontiguousarray(host["experts"][pl.local_experts(rank)])
            dl = gu.DeviceLayer(local)
            dl.register(moe, l)
            keep.append(dl)
        moe.set_expert_map(pl.expert_map(rank))
        ids = [moe.ep_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        moe.ep_init(ids[0], rank, world, R_OWN)
        handles = [None] * world
        dist.all_gather_object(handles, moe.ep_peer_export())
        moe.ep_peer_attach(handles)
        x_all = synthetic.hidden_rows(931, T, RD)
        st = torch.cuda.Stream()
        outs = []
        with torch.cuda.stream(st):
            x_own = gu.to_dev(x_all[rank * R_OWN:(rank + 1) * R_OWN].copy()).view(torch.float16)
            y = torch.zeros(R_OWN, RD, dtype=torch.float32, device="cuda")
            for call in range(3):        # the same step three times: the epoch moves on, the bits must not
                y.zero_()
                moe.ep_stack_decode(x_own, R_OWN, y, stream=st)
                moe.synchronize(stream=st)
                outs.append(y.cpu().numpy().copy())
            dist.barrier()
        np.save(os.path.join(out_dir, f"res{rank}.npy"), np.stack(outs))
        if rank == 0:       # all rows on one GPU with every expert, through the same kernel (one rank)
            one = MoE(_resident_cfg(T, R_LAYERS))
            full = [gu.DeviceLayer(h) for h in hosts]
            for l, dl in enumerate(full):
                dl.register(one, l)
            ya = torch.zeros(T, RD, dtype=torch.float32, device="cuda")
            one.set_decode_mode(MoE.DECODE_RESIDENT)
            one.stack_decode(gu.to_dev(x_all).view(torch.float16), T, ya)
            one.synchronize()
            np.save(os.path.join(out_dir, "single.npy"), ya.cpu().numpy())
        dist.barrier()
        moe.ep_shutdown()
        dist.destroy_process_group()
    except Exception:
        with open(os.path.join(out_dir, f"err{rank}.txt"), "w") as f:
            f.write(traceback.format_exc())
        sys.exit(3)


def test_two_gpu_resident_kernel_exchanges_shares_over_peer_memory(tmp_path):
    """3 layers, 3 rows per rank, experts strided over 2 GPUs: every rank runs ONE resident kernel per step, the ranks'
    shares cross by peer stores from its down phase.  Against the oracle chain per row, against the same rows on one
    GPU with every expert, and bitwise repeatable."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    import gpu_util as gu
    from nvmai_b200 import synthetic
    from oracle import oracle as orc
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_rank_resident, args=(r, 2, 29571, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        if p.is_alive():
            p.kill()
            p.join()
    errs = [p.read_text() for p in tmp_path.glob("err*.txt")]
    assert [p.exitcode for p in procs] == [0, 0], errs
    hosts = _resident_hosts()
    cfg = _resident_cfg(2 * R_OWN, R_LAYERS)
    Ls = [gu.oracle_layer(h, cfg) for h in hosts]
    x_all = synthetic.hidden_rows(931, 2 * R_OWN, RD)
    single = np.load(tmp_path / "single.npy")
    for rank in range(2):
        res = np.load(tmp_path / f"res{rank}.npy")
        assert np.all(np.isfinite(res))
        assert np.array_equal(res[0].view(np.uint32), res[1].view(np.uint32)) and np.array_equal(res[0].view(np.uint32), res[2].view(np.uint32))
        for j in range(R_OWN):
            row = rank * R_OWN + j
            x = np.ascontiguousarray(x_all[row])
            for l in range(R_LAYERS):
                _, _, h2, margin, _ = gu.oracle_decode(Ls[l][0], cfg, x)
                assert margin > 1e-5
                if l + 1 < R_LAYERS:
                    scale = 1.0 / np.sqrt(np.mean(h2.astype(np.float64) ** 2) + 1e-6)
                    x = orc.f32_to_f16_bits((h2.astype(np.float64) * scale).astype(np.float32))
            assert orc.rel_error(res[0][j], h2) < 2e-3, f"rank {rank} row {j} vs the oracle chain"
            assert orc.rel_error(res[0][j], single[row]) < 1e-4, f"rank {rank} row {j} vs one GPU with every expert"
