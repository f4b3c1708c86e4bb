#!/usr/bin/env python
"""Benchmark of the routed-expert MoE FFN stack (35B-A3B shape) on B200.

Workload (the benchmark's configs[3]): 40 MoE FFN layers (hidden 2048, 256 routed
experts, top-8, expert intermediate 512, one sigmoid-gated shared expert of 512),
group-64 affine weights, all experts resident in HBM, batch-1 decode.  A step is
one token through all 40 layers; `value` is tokens/s.  Weights are seeded
synthetic with the benchmark's value distributions, generated on the device.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--bits 4|8] [--impl ours|reference]

One JSON line is printed by rank 0.  `--impl reference` times the reference's
CPU path (its own C GEMV from oracle/_ref when built, else the restated port) on
the host cores for the same workload.
"""
from __future__ import annotations

import argparse
import json
import warnings
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

D, F, FS, E, K, LAYERS = 2048, 512, 512, 256, 8, 40
METRIC = "moe_ffn_stack_decode_tokens_per_s"
UNIT = "tokens/s"


def expert_bytes(bits: int) -> int:
    return 2 * (F * D * bits // 8 + 2 * F * (D // 64) * 2) + (D * F * bits // 8 + 2 * D * (F // 64) * 2)


def layer_bytes(bits: int) -> int:
    """Algorithmic bytes of one layer at batch 1: 8 routed + 1 shared expert,
    the dense fp16 router, the gate row, x in and y out."""
    return K * expert_bytes(bits) + expert_bytes(bits) + E * D * 2 + D * 2 + D * 2 + D * 4


def stage2_bytes(bits: int, out_elt: int) -> int:
    """Algorithmic bytes of one launch of the dominant kernel (routed gate/up +
    activation, 8 experts): codes + scales + biases of gate and up, x, acts out."""
    return K * 2 * (F * D * bits // 8 + 2 * F * (D // 64) * 2) + D * 2 + K * F * out_elt


def measured_peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# --------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------

class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        out, _ = self.proc.communicate(timeout=10)
        sm, smax, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                smax = float(parts[1])
            except ValueError:
                continue
            for name, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm)}


# --------------------------------------------------------------------------------------
# reference CPU path (also the cpu_baseline leg of the GPU arm)
# --------------------------------------------------------------------------------------

class CpuReferenceStack:
    """The stack workload on the host cores with the reference's CPU arithmetic
    (CPUExpertFFN.accumulate over nvmai_int4_affine_gemv), driven by the threaded
    C++ harness in oracle/cpu_stack.cpp: rows of every GEMV stage split over
    std::threads, the router and the selection through the oracle's own functions.
    Per layer only the blobs a token uses are generated (8 routed + 1 shared),
    since the timing does not depend on which of the 256 experts were picked; the
    router still scores all 256 rows."""

    def __init__(self, bits: int, layers: int, seed: int = 7):
        import ctypes as C
        from nvmai_b200 import format as fmt
        from oracle import oracle as orc
        self.orc, self.bits, self.layers = orc, bits, layers
        self.stack_lib = orc.cpu_stack_lib()
        ref = orc.ref_lib() if bits == 4 else None
        self.kind = "reference" if ref is not None else "port"
        self.gemv4 = C.cast(ref.nvmai_int4_affine_gemv, C.c_void_p) if ref is not None else None
        rng = np.random.default_rng(seed)
        off, stride = fmt.expert_offsets(D, F, bits)
        # blobs: random code bytes, then the six scale / bias arrays overwritten with the benchmark's distributions
        self.blobs = rng.integers(0, 256, size=(layers, K + 1, stride), dtype=np.uint8)
        gate_m, down_m = F * (D // 64), D * (F // 64)
        for name, n, lo, hi in (("gate_s", gate_m, 0.005, 0.02), ("gate_b", gate_m, -0.08, 0.0),
                                ("up_s", gate_m, 0.005, 0.02), ("up_b", gate_m, -0.08, 0.0),
                                ("down_s", down_m, 0.005, 0.02), ("down_b", down_m, -0.08, 0.0)):
            vals = fmt.f32_to_bf16_bits(rng.uniform(lo, hi, size=(layers, K + 1, n)).astype(np.float32))
            self.blobs[:, :, off[name]:off[name] + 2 * n] = vals.view(np.uint8).reshape(layers, K + 1, 2 * n)
        self.routers = fmt.f32_to_f16_bits(rng.normal(0.0, 0.02, size=(layers, E, D)))
        self.gates = fmt.f32_to_f16_bits(rng.normal(0.0, 0.02, size=(layers, D)))
        self.xs = fmt.f32_to_f16_bits(rng.normal(size=(8, D)))
        desc = orc.StackDesc()
        desc.d, desc.f, desc.e, desc.k, desc.bits, desc.layers = D, F, E, K, bits, layers
        desc.stride = stride
        for i, name in enumerate(fmt.OFFSET_NAMES):
            desc.off[i] = off[name]
        self._ptrs = [(C.c_void_p * layers)(*[a[l].ctypes.data for l in range(layers)])
                      for a in (self.blobs, self.routers, self.gates)]
        desc.blobs, desc.router_f16, desc.gate_f16 = (C.cast(p_, C.POINTER(C.c_void_p)) for p_ in self._ptrs)
        self.desc = desc

    def time_tokens(self, threads: int, steps: int, warmup: int) -> float:
        """seconds per token over the sampled layers"""
        import ctypes as C
        y = np.zeros(D, dtype=np.float32)
        sec = self.stack_lib.orc_cpu_stack_time(C.byref(self.desc), threads, steps, warmup, self.xs.ctypes.data,
                                                self.xs.shape[0], y.ctypes.data, self.gemv4)
        if sec <= 0 or not np.all(np.isfinite(y)):
            raise RuntimeError("CPU reference stack failed")
        return float(sec)


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def base_record(args, n_gpus: int) -> dict:
    return {
        "metric": METRIC, "unit": UNIT, "n_gpus": n_gpus, "steps": args.steps, "warmup": args.warmup,
        "higher_is_better": True, "vs_baseline": None, "data": "synthetic",
        "config": {"workload": f"configs[3]: 40-layer MoE FFN stack, 35B-A3B shape, {args.bits}-bit, "
                               + ("batch-1 decode" if args.tokens == 1 else f"decode of {args.tokens} independent rows per GPU and step"),
                   "d": D, "f": F, "experts": E, "top_k": K, "layers": args.layers, "bits": args.bits,
                   "meta": "bf16", "router": "dense fp16", "tokens_per_step": args.tokens,
                   "l2": "working set 679 MB (4-bit) / 1246 MB (8-bit) per step exceeds the 126 MB L2; inputs rotate"},
    }


def cpu_baseline_record(args, stack: CpuReferenceStack, layers: int, steps: int, warmup: int, with_single: bool) -> dict:
    """all-core (and one-thread) tokens/s of the reference CPU path, scaled from `layers` sampled layers"""
    threads = host_threads()
    scale = args.layers / layers
    sec_all = stack.time_tokens(threads, steps, warmup) * scale
    rec = {"value": 1.0 / sec_all, "unit": UNIT, "cores": threads, "kind": stack.kind,
           "sample": f"{steps} tokens x {layers} of {args.layers} layers (router over 256 rows, 8 routed + 1 shared "
                     f"expert per layer; GEMV rows split over {threads} std::threads), scaled to {args.layers}"}
    if with_single:
        sec_one = stack.time_tokens(1, 1, 0) * scale
        rec["value_1_thread"] = 1.0 / sec_one
        rec["speedup_all_cores"] = sec_one / sec_all
    return rec


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    layers = min(args.layers, args.ref_layers)
    stack = CpuReferenceStack(args.bits, layers)
    steps, warm = max(1, args.steps), max(0, args.warmup)
    base = cpu_baseline_record(args, stack, layers, steps, warm, with_single=True)
    val = base["value"]
    rec = base_record(args, args.gpus)
    rec.update({"impl": "reference", "value": val, "ms_per_step": 1e3 / val, "scaling": "strong",
                "dtype": "f32", "cpu_baseline": base,
                "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0})
    print(json.dumps(rec), flush=True)


# --------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------

def run_ours(args) -> None:
    import torch
    from nvmai_b200 import MoE, MoEConfig, launch_count, synthetic
    from nvmai_b200 import format as fmt

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    tokens = args.tokens
    if world > 1:
        # a stuck collective would otherwise hold the GPUs until someone kills the job
        killer = threading.Timer(args.deadline, lambda: os._exit(2))
        killer.daemon = True
        killer.start()
        run_ours_ep(args, torch, dist, rank, world, local)
        killer.cancel()
        return
    cfg = MoEConfig(d=D, f=F, shared_f=FS, num_experts=E, top_k=K, routed_bits=args.bits, shared_bits=args.bits,
                    router_kind=fmt.ROUTER_DENSE_F16, shared_gate_kind=fmt.ROUTER_DENSE_F16,
                    meta_dtype=fmt.META_BF16, activation=fmt.ACT_SILU, out_dtype=fmt.OUT_FP32,
                    max_tokens=max(tokens, 1), num_layers=args.layers)
    moe = MoE(cfg)
    devs = []
    for l in range(args.layers):
        dev = synthetic.device_layer(1000 + l, d=D, f=F, shared_f=FS, num_experts=E, routed_bits=args.bits,
                                     meta=fmt.META_BF16)
        synthetic.register_device_layer(moe, l, dev)
        devs.append(dev)
    torch.cuda.synchronize()

    stream = torch.cuda.Stream()
    gen = torch.Generator(device="cuda")
    gen.manual_seed(42 + rank)
    n_inputs = 16      # distinct token inputs rotated through, so every step routes to different experts
    xs = torch.randn(n_inputs, tokens, D, device="cuda", generator=gen).to(torch.float16)
    x_in = torch.empty(tokens, D, dtype=torch.float16, device="cuda")
    y = torch.empty(tokens, D, dtype=torch.float32, device="cuda")
    xs_host = [xs[i].cpu().pin_memory() for i in range(n_inputs)]
    y_host = torch.empty(tokens, D, dtype=torch.float32).pin_memory()
    torch.cuda.synchronize()

    def step(i: int) -> None:
        x_in.copy_(xs[i % n_inputs], non_blocking=True)
        moe.stack_decode(x_in, tokens, y, stream=stream)

    def barrier() -> None:
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.cuda.stream(stream):
        for i in range(max(args.warmup, 3)):
            step(i)
        barrier()
        sampler = ClockSampler(local) if rank == 0 else None
        l0 = launch_count()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for i in range(args.steps):
            step(i)
        end.record(stream)
        barrier()
        launches = launch_count() - l0
        ms = start.elapsed_time(end)
        assert torch.isfinite(y).all(), "non-finite output"

        # end to end through the host-buffer entry point: pinned x in, y out, every step
        for i in range(3):
            moe.stack_decode_host(xs_host[i].data_ptr(), tokens, y_host.data_ptr(), stream=stream)
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            moe.stack_decode_host(xs_host[i % n_inputs].data_ptr(), tokens, y_host.data_ptr(), stream=stream)
        barrier()
        e2e_s = time.perf_counter() - t0
        clocks = sampler.stop() if sampler else None

    times = torch.tensor([ms, e2e_s * 1e3], dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(times[0]), float(times[1])
    ms_per_step = ms / args.steps
    value = tokens / (ms_per_step / 1e3)
    e2e_value = tokens / (e2e_ms / args.steps / 1e3)

    rec = None
    if rank == 0:
        peak, which = measured_peaks()
        forced_staged = os.environ.get("NVMAI_CUDA_DECODE_MODE", "0") == "1"
        if tokens == 1 and not forced_staged:
            roof = resident_roofline(moe, args, xs, x_in, y, stream, peak, which)
        elif 2 <= tokens <= 8 and not forced_staged:
            roof = batch_roofline(moe, args, tokens, ms_per_step, peak, which)
        else:
            roof = stage2_roofline(moe, cfg, devs, args, stream, peak, which)
        step_bytes = roof["bytes_per_launch"] if 2 <= tokens <= 8 and not forced_staged else args.layers * layer_bytes(args.bits)
        roof["step_bytes"] = step_bytes
        roof["step_frac"] = step_bytes / (ms_per_step / 1e3) / 1e9 / peak
        rec = base_record(args, world)
        rec.update({"value": value, "ms_per_step": ms_per_step, "scaling": "weak", "dtype": "f16xu%d->f32" % args.bits,
                    "clocks": clocks, "gpu_launches": int(launches),
                    "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": tokens * D * 2,
                            "d2h_bytes_per_step": tokens * D * 4},
                    "roofline": roof})
        if world == 1 and not args.no_cpu_baseline:
            layers = min(args.layers, args.ref_layers)
            cpu = CpuReferenceStack(args.bits, layers)
            rec["cpu_baseline"] = cpu_baseline_record(args, cpu, layers, steps=8, warmup=1, with_single=True)
        if world == 1 and tokens == 1 and not args.no_parity:
            rec["parity"] = stack_parity(args, cfg, devs, xs, torch)
        print(json.dumps(rec), flush=True)
        if "parity" in rec and not rec["parity"]["ok"]:
            raise SystemExit("parity check of the timed path failed: " + json.dumps(rec["parity"]))
    if dist is not None:
        dist.destroy_process_group()


def run_ours_ep(args, torch, dist, rank: int, world: int, local: int) -> None:
    """Expert-parallel stack: 256/world experts per rank, every rank decodes its own
    `--tokens` rows (weak scaling: one more GPU brings one more decode stream); per layer
    an all-gather of the rows (dispatch) and an all-to-all of the share rows (combine)
    over NCCL, issued by the library on its own communicator and replayed with the
    kernels as one CUDA graph."""
    from nvmai_b200 import MoE, MoEConfig, launch_count, synthetic
    from nvmai_b200 import format as fmt
    from nvmai_b200.ep import ExpertPlacement, LibraryBackend, ep_stack_step
    tokens = args.tokens
    pl = ExpertPlacement(E, world, args.placement)
    cfg = MoEConfig(d=D, f=F, shared_f=FS, num_experts=E, top_k=K, routed_bits=args.bits, shared_bits=args.bits,
                    router_kind=fmt.ROUTER_DENSE_F16, shared_gate_kind=fmt.ROUTER_DENSE_F16,
                    meta_dtype=fmt.META_BF16, activation=fmt.ACT_SILU, out_dtype=fmt.OUT_FP32,
                    max_tokens=world * tokens, num_layers=args.layers)
    moe = MoE(cfg)
    devs = []
    for l in range(args.layers):
        # same seed on every rank: router / shared expert / gate are replicas; the local
        # expert blobs are random bytes whose values do not matter for the timing
        dev = synthetic.device_layer(1000 + l, d=D, f=F, shared_f=FS, num_experts=E, routed_bits=args.bits,
                                     meta=fmt.META_BF16, expert_ids=pl.local_experts(rank))
        synthetic.register_device_layer(moe, l, dev)
        devs.append(dev)
    moe.set_expert_map(pl.expert_map(rank))
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    backend = LibraryBackend(moe, stream=stream)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(42 + rank)
    n_inputs = 16
    xs = torch.randn(n_inputs, tokens, D, device="cuda", generator=gen).to(torch.float16)
    x_in = torch.empty(tokens, D, dtype=torch.float16, device="cuda")
    y_out = torch.empty(tokens, D, dtype=torch.float32, device="cuda")
    xs_host = [xs[i].cpu().pin_memory() for i in range(n_inputs)]
    y_host = torch.empty(tokens, D, dtype=torch.float32).pin_memory()

    t_begin = time.perf_counter()

    def note(msg):      # progress on stderr: tells where a stuck multi-GPU run stopped
        if args.verbose:
            print(f"[rank {rank} +{time.perf_counter() - t_begin:6.1f}s] {msg}", file=sys.stderr, flush=True)

    native = args.ep_driver == "native"
    note("weights resident")
    if native:
        # the library's own communicator: compute and both collectives of all layers replay as one CUDA graph
        ids = [moe.ep_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        moe.ep_init(ids[0], rank, world, tokens)
        if args.ep_exchange == "p2p":
            # the ranks' receive areas mapped into each other (CUDA IPC): the down phase stores its shares there itself
            handles = [None] * world
            dist.all_gather_object(handles, moe.ep_peer_export())
            try:
                moe.ep_peer_attach(handles)
                attached = 1
            except Exception as err:       # no peer access between some pair of GPUs
                note(f"peer attach failed: {err}")
                attached = 0
            flag = torch.tensor([attached], dtype=torch.int32, device="cuda")
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if int(flag.item()) == 0:
                # every rank falls back together: a fresh communicator, shares by NCCL between the staged kernels
                args.ep_exchange = "nccl"
                moe.ep_shutdown()
                ids = [moe.ep_unique_id() if rank == 0 else None]
                dist.broadcast_object_list(ids, src=0)
                moe.ep_init(ids[0], rank, world, tokens)

        def run_step():
            moe.ep_stack_decode(x_in, tokens, y_out, stream=stream)
    else:
        # torch.distributed collectives around the library's per-stage calls, plain launches
        def run_step():
            y = ep_stack_step(backend, dist, None, x_in, world=world, layers=args.layers)
            y_out.copy_(y, non_blocking=True)

    with torch.cuda.stream(stream):
        x_in.copy_(xs[0])
        def wait_step():
            # the library's own host-polled wait: a step whose peer is gone ends as an error (the communicator is
            # aborted) after --deadline seconds instead of blocking in the driver for good
            if native:
                moe.ep_synchronize(stream, int(args.deadline * 1000))
            else:
                stream.synchronize()

        for call in range(3):       # plain launches, graph capture, first replay
            run_step()
            wait_step()
            note(f"step call {call} done")
        dist.barrier()

        def step(i):
            x_in.copy_(xs[i % n_inputs], non_blocking=True)
            run_step()

        for i in range(max(args.warmup, 10)):
            step(i)
        # the clock sampler starts (a process spawn on rank 0) BEFORE the barrier that opens the timed region:
        # otherwise the other ranks' first collective would wait for rank 0 inside their timed region
        sampler = ClockSampler(local) if rank == 0 else None
        dist.barrier()
        torch.cuda.synchronize()
        l0 = launch_count()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for i in range(args.steps):
            step(i)
        end.record(stream)
        dist.barrier()
        torch.cuda.synchronize()
        launches = launch_count() - l0
        ms = start.elapsed_time(end)
        note(f"timed region done: {ms / args.steps:.3f} ms/step")
        assert torch.isfinite(y_out).all(), "non-finite output"
        t0 = time.perf_counter()
        for i in range(args.steps):
            x_in.copy_(xs_host[i % n_inputs], non_blocking=True)
            run_step()
            y_host.copy_(y_out, non_blocking=True)
            wait_step()
        dist.barrier()
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
        clocks = sampler.stop() if sampler else None
    times = torch.tensor([ms, e2e_s * 1e3], dtype=torch.float64, device="cuda")
    dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_per_step = float(times[0]) / args.steps
    resident = native and args.ep_exchange == "p2p" and world * tokens <= 8
    if resident and args.block_trace:
        # every rank's timeline of a few traced steps, on stderr (the marks slow the kernel a little: after the timing)
        moe.set_trace(True)
        with torch.cuda.stream(stream):
            for i in range(4):
                step(i)
            stream.synchronize()
        dist.barrier()
        print(json.dumps(block_trace_summary(moe.read_block_trace(), world * tokens,
                                             f"rank {rank} of {world}, {world * tokens} rows per step", False)),
              file=sys.stderr, flush=True)
        moe.set_trace(False)
        dist.barrier()
    single = None
    if rank == 0 and resident and not args.no_single_gpu:
        # the same total batch on ONE GPU that holds every expert (the figure an expert-parallel run has to beat)
        one_cfg = MoEConfig(d=D, f=F, shared_f=FS, num_experts=E, top_k=K, routed_bits=args.bits, shared_bits=args.bits,
                            router_kind=fmt.ROUTER_DENSE_F16, shared_gate_kind=fmt.ROUTER_DENSE_F16,
                            meta_dtype=fmt.META_BF16, activation=fmt.ACT_SILU, out_dtype=fmt.OUT_FP32,
                            max_tokens=world * tokens, num_layers=args.layers)
        one = MoE(one_cfg)
        full = []
        for l in range(args.layers):
            dev = synthetic.device_layer(1000 + l, d=D, f=F, shared_f=FS, num_experts=E, routed_bits=args.bits, meta=fmt.META_BF16)
            synthetic.register_device_layer(one, l, dev)
            full.append(dev)
        rows = world * tokens
        xa = torch.randn(n_inputs, rows, D, device="cuda", generator=gen).to(torch.float16)
        xin = torch.empty(rows, D, dtype=torch.float16, device="cuda")
        ya = torch.empty(rows, D, dtype=torch.float32, device="cuda")
        with torch.cuda.stream(stream):
            for i in range(5):
                xin.copy_(xa[i], non_blocking=True)
                one.stack_decode(xin, rows, ya, stream=stream)
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record(stream)
            for i in range(args.steps):
                xin.copy_(xa[i % n_inputs], non_blocking=True)
                one.stack_decode(xin, rows, ya, stream=stream)
            s1.record(stream)
            stream.synchronize()
        single = rows / (s0.elapsed_time(s1) / args.steps / 1e3)
        del one, full
    if rank == 0:
        peak, which = measured_peaks()
        rec = base_record(args, world)
        # kernels per layer on the expert-parallel path: router, group, gate/up, down, combine, shared gate/up,
        # shared down, finalize (+ renorm between layers); the library counts them, replays included
        rec.update({"value": world * tokens / (ms_per_step / 1e3), "ms_per_step": ms_per_step, "scaling": "weak",
                    "dtype": "f16xu%d->f32" % args.bits, "clocks": clocks,
                    "gpu_launches": int(launches),
                    "e2e": {"value": world * tokens / (float(times[1]) / args.steps / 1e3), "unit": UNIT,
                            "h2d_bytes_per_step": tokens * D * 2, "d2h_bytes_per_step": tokens * D * 4},
                    "roofline": {"bound": "hbm", "kernel": "expert-parallel step (all kernels + 2 collectives per layer)",
                                 "achieved": args.layers * layer_bytes(args.bits) * tokens / (ms_per_step / 1e3) / 1e9,
                                 "peak": peak, "peak_source": which, "unit": "GB/s",
                                 "frac": args.layers * layer_bytes(args.bits) * tokens / (ms_per_step / 1e3) / 1e9 / peak,
                                 "traffic": None}})
        if resident:
            exchange = ("one resident kernel per rank and step and nothing else: every rank keeps all rows; the step's rows are "
                        "gathered at layer 0 and the share rows of a rank's experts exchanged in every layer's down phase, both as "
                        "tagged 64-bit peer stores over NVLink from inside the kernel (no collective call)")
            rec["roofline"]["kernel"] = "persistent_batch_kernel (one launch per rank = all layers of the step)"
        elif native and world * tokens < 24:
            exchange = ("all_gather(fp32 share rows) per layer, NCCL" if args.ep_exchange != "p2p" else
                        "shares by peer stores from the staged down kernel + counted arrival") + "; every rank keeps all rows"
        else:
            exchange = "all_gather(x) + all_to_all(share rows) per layer, NCCL"
        rec["config"].update({"parallelism": f"ep{world}", "experts_per_gpu": E // world, "placement": args.placement,
                              "tokens_per_step": world * tokens, "ep_driver": args.ep_driver, "exchange": exchange})
        if single is not None:
            rec["single_gpu_same_batch"] = {"value": single, "unit": UNIT, "rows_per_step": world * tokens,
                                            "note": "one GPU holding all 256 experts of every layer, the same rows through "
                                                    "the same resident kernel"}
        print(json.dumps(rec), flush=True)
    note("end-to-end region done")
    dist.barrier()
    torch.cuda.synchronize()
    if native:
        moe.ep_shutdown()       # every rank, with nothing in flight
    note("communicator closed")
    dist.destroy_process_group()
    note("process group closed")


def run_batch_layer(args) -> None:
    """configs[1] / configs[4]: ONE layer, a batch of `--tokens` independent rows through the batched decode
    kernels (rows that picked the same expert share one read of its weights).  Rotates over 16 independently
    seeded layers so that the working set exceeds L2.  `--zipf S` replaces the router's choice by expert ids
    drawn with popularity ~ rank^-S over a seeded permutation (configs[4]); the routed kernels then run from
    the given ids (`nvmai_cuda_moe_routed_partial`), router and shared expert left out."""
    import torch
    from nvmai_b200 import MoE, MoEConfig, launch_count, synthetic
    from nvmai_b200 import format as fmt
    from nvmai_b200.ep import ExpertPlacement
    torch.cuda.set_device(0)
    tokens, n_layers = args.tokens, 16
    cfg = MoEConfig(d=D, f=F, shared_f=FS, num_experts=E, top_k=K, routed_bits=args.bits, shared_bits=args.bits,
                    router_kind=fmt.ROUTER_DENSE_F16, shared_gate_kind=fmt.ROUTER_DENSE_F16,
                    meta_dtype=fmt.META_BF16, activation=fmt.ACT_SILU, out_dtype=fmt.OUT_FP32,
                    max_tokens=tokens, num_layers=n_layers)
    moe = MoE(cfg)
    devs = []
    for l in range(n_layers):
        dev = synthetic.device_layer(3000 + l, d=D, f=F, shared_f=FS, num_experts=E, routed_bits=args.bits,
                                     meta=fmt.META_BF16)
        synthetic.register_device_layer(moe, l, dev)
        devs.append(dev)
    stream = torch.cuda.Stream()
    gen = torch.Generator(device="cuda")
    gen.manual_seed(11)
    x = torch.randn(tokens, D, device="cuda", generator=gen).to(torch.float16)
    y = torch.empty(tokens, D, dtype=torch.float32, device="cuda")
    idx = torch.empty(tokens, K, dtype=torch.int32, device="cuda")
    w = torch.empty(tokens, K, dtype=torch.float16, device="cuda")
    zipf = args.zipf > 0
    trace_stats = None
    idx_per_layer = None
    if args.route_trace:
        # the routing comes from a trace in the reference's NVMAI_ROUTE_TRACE format (RealForwardRunner.swift:1208-1237):
        # step i replays `tokens` consecutive recorded tokens of trace layer i % layers; weights 1/K (the trace holds ids only)
        from nvmai_b200 import route_trace as rt
        if args.route_trace.startswith("synthetic"):
            reuse = float(args.route_trace.split(":")[1]) if ":" in args.route_trace else 0.38
            trace = rt.parse(rt.synthesize(max(tokens, 128), n_layers, num_experts=E, top_k=K, reuse=reuse, seed=9).format(),
                             num_experts=E, top_k=K)
        else:
            trace = rt.parse(args.route_trace, num_experts=E, top_k=K)
        trace_stats = trace.stats()
        tl = trace.layer_ids()
        idx_per_layer = [torch.from_numpy(trace.batch(tl[l % len(tl)], 0, tokens)).cuda() for l in range(n_layers)]
        w.fill_(1.0 / K)
    if zipf:
        rng = np.random.default_rng(4)
        perm = rng.permutation(E)
        p = (np.arange(1, E + 1, dtype=np.float64) ** -args.zipf)
        p /= p.sum()
        ids = np.stack([perm[rng.choice(E, size=K, replace=False, p=p)] for _ in range(tokens)]).astype(np.int32)
        idx.copy_(torch.from_numpy(ids))
        w.fill_(1.0 / K)

    prenorm = args.prenorm
    if prenorm:
        # the two steps the runner encodes in front of the block (RealForwardRunner.swift:1900-1909), folded into the
        # block's launches ("fused") or as the separate launches they replace ("unfused": residual add, norm, block)
        from nvmai_b200 import Elementwise
        hidden = torch.randn(tokens, D, device="cuda", generator=gen).to(torch.float16)
        delta = (0.5 * torch.randn(tokens, D, device="cuda", generator=gen)).to(torch.float16)
        norm_w = (0.5 + torch.rand(D, device="cuda", generator=gen)).to(torch.bfloat16)
        hid32 = hidden.float()

    def step(i: int) -> None:
        if prenorm == "fused":
            moe.layer_decode_prenorm(i % n_layers, hid32, norm_w, 1e-6, tokens, attn_delta=delta, h2_out=y, out_idx=idx,
                                     out_w=w, stream=stream)
        elif prenorm == "unfused":
            Elementwise.encode_residual_add(hidden, delta, tokens * D, stream=stream)
            moe.rms_renorm(hid32, tokens, x, stream=stream)
            moe.layer_decode(i % n_layers, x, tokens, hidden=hid32, h2_out=y, out_idx=idx, out_w=w, stream=stream)
        elif idx_per_layer is not None:
            moe.routed_partial(i % n_layers, x, tokens, idx_per_layer[i % n_layers], w, y, stream=stream)
        elif zipf:
            moe.routed_partial(i % n_layers, x, tokens, idx, w, y, stream=stream)
        else:
            moe.layer_decode(i % n_layers, x, tokens, h2_out=y, out_idx=idx, out_w=w, stream=stream)

    with torch.cuda.stream(stream):
        for i in range(max(args.warmup, 3)):
            step(i)
        stream.synchronize()
        sampler = ClockSampler(0)
        l0 = launch_count()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for i in range(args.steps):
            step(i)
        end.record(stream)
        stream.synchronize()
        launches = launch_count() - l0
        ms = start.elapsed_time(end) / args.steps
        clocks = sampler.stop()
    assert torch.isfinite(y).all(), "non-finite output"
    ids = idx.cpu().numpy() if idx_per_layer is None else idx_per_layer[(args.steps - 1) % n_layers].cpu().numpy()
    zipf = zipf or idx_per_layer is not None          # routed experts only in both replay modes
    distinct = int(np.unique(ids).size)
    blob = expert_bytes(args.bits)
    nbytes = distinct * blob + tokens * (D * 2 + D * 4)
    if not zipf:
        nbytes += blob + E * D * 2 + D * 2           # shared expert, fp16 router, gate row
    peak, which = measured_peaks()
    gbs = nbytes / (ms * 1e-3) / 1e9
    load = {}
    counts = np.bincount(ids.ravel(), minlength=E)
    for n in (2, 4, 8):
        for mode in ("contiguous", "strided"):
            per = ExpertPlacement(E, n, mode).pairs_per_rank(ids.ravel())
            load[f"{mode}{n}"] = round(max(per) / (sum(per) / n), 3)
    rec = {"metric": "moe_ffn_layer_batch_tokens_per_s", "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
           "warmup": args.warmup, "higher_is_better": True, "vs_baseline": None, "data": "synthetic", "scaling": "weak",
           "dtype": "f16xu%d->f32" % args.bits, "value": tokens / (ms * 1e-3), "ms_per_step": ms, "clocks": clocks,
           "gpu_launches": int(launches),
           "config": {"workload": ("one layer, %d rows, routing replayed from a trace (%s), routed experts only"
                                   % (tokens, "synthetic" if args.route_trace.startswith("synthetic") else "file"))
                      if idx_per_layer is not None else
                      ("one layer, %d rows, attention residual add + post-attention RMS norm + block, %s"
                       % (tokens, prenorm)) if prenorm else
                      ("configs[4]: one layer, %d rows, Zipf(%.1f) routing, routed experts only" % (tokens, args.zipf))
                      if zipf else ("configs[1]: one layer, %d independent rows, router + routed + shared" % tokens),
                      "d": D, "f": F, "experts": E, "top_k": K, "bits": args.bits, "layers_rotated": n_layers,
                      "distinct_experts": distinct, "hottest_expert_rows": int(counts.max()),
                      "max_over_mean_pairs_per_gpu": load},
           "roofline": {"bound": "hbm", "kernel": "whole layer call (each distinct expert's bytes counted once)",
                        "achieved": gbs, "peak": peak, "peak_source": which, "unit": "GB/s", "frac": gbs / peak,
                        "traffic": None, "bytes_per_step": nbytes}}
    if trace_stats is not None:
        rec["config"]["trace"] = trace_stats
    print(json.dumps(rec), flush=True)


def run_batch_layer_ep(args, torch, dist, rank: int, world: int, local: int) -> None:
    """configs[4] on several GPUs: the 256-row Zipf batch on one layer whose experts are spread over the ranks.  Every
    rank owns tokens / world rows.  A step is: all-gather of the rows (a row is needed by nearly every rank, its eight
    experts being spread over them), every rank's tensor-core items over ITS experts' pairs
    (`nvmai_cuda_moe_routed_partial` under the rank's expert map), all-to-all of the fp32 share rows to the rows'
    owners, rank-ordered sum there.  Collectives by torch.distributed (NCCL); no shared expert (as at one GPU)."""
    from nvmai_b200 import MoE, MoEConfig, launch_count, synthetic
    from nvmai_b200 import format as fmt
    from nvmai_b200.ep import ExpertPlacement
    tokens, n_layers = args.tokens, 16
    assert tokens % world == 0, "--tokens must divide by the number of GPUs"
    own = tokens // world
    pl = ExpertPlacement(E, world, args.placement)
    cfg = MoEConfig(d=D, f=F, shared_f=FS, num_experts=E, top_k=K, routed_bits=args.bits, shared_bits=args.bits,
                    router_kind=fmt.ROUTER_DENSE_F16, shared_gate_kind=fmt.ROUTER_DENSE_F16, meta_dtype=fmt.META_BF16,
                    activation=fmt.ACT_SILU, out_dtype=fmt.OUT_FP32, max_tokens=tokens, num_layers=n_layers)
    moe = MoE(cfg)
    devs = []
    for l in range(n_layers):
        dev = synthetic.device_layer(3000 + l, d=D, f=F, shared_f=FS, num_experts=E, routed_bits=args.bits,
                                     meta=fmt.META_BF16, expert_ids=pl.local_experts(rank))
        synthetic.register_device_layer(moe, l, dev)
        devs.append(dev)
    moe.set_expert_map(pl.expert_map(rank))
    stream = torch.cuda.Stream()
    gen = torch.Generator(device="cuda")
    gen.manual_seed(11 + rank)
    x_own = torch.randn(own, D, device="cuda", generator=gen).to(torch.float16)
    x_all = torch.empty(tokens, D, dtype=torch.float16, device="cuda")
    share = torch.empty(tokens, D, dtype=torch.float32, device="cuda")
    recv = torch.empty(world, own, D, dtype=torch.float32, device="cuda")
    y_own = torch.empty(own, D, dtype=torch.float32, device="cuda")
    rng = np.random.default_rng(4)              # the same routing on every rank
    perm = rng.permutation(E)
    p = (np.arange(1, E + 1, dtype=np.float64) ** -args.zipf)
    p /= p.sum()
    ids = np.stack([perm[rng.choice(E, size=K, replace=False, p=p)] for _ in range(tokens)]).astype(np.int32)
    idx = torch.from_numpy(ids).cuda()
    w = torch.full((tokens, K), 1.0 / K, dtype=torch.float16, device="cuda")

    def step(i: int) -> None:
        dist.all_gather_into_tensor(x_all, x_own)
        moe.routed_partial(i % n_layers, x_all, tokens, idx, w, share, stream=stream)
        dist.all_to_all_single(recv.view(tokens, D), share)
        moe.ep_finalize(recv, world, None, own, y=y_own, stream=stream)

    with torch.cuda.stream(stream):
        for i in range(max(args.warmup, 5)):
            step(i)
        # the clock sampler starts (a process spawn on rank 0) BEFORE the barrier that opens the timed region:
        # otherwise the other ranks' first collective would wait for rank 0 inside their timed region
        sampler = ClockSampler(local) if rank == 0 else None
        dist.barrier()
        torch.cuda.synchronize()
        l0 = launch_count()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for i in range(args.steps):
            step(i)
        end.record(stream)
        dist.barrier()
        torch.cuda.synchronize()
        launches = launch_count() - l0
        ms = start.elapsed_time(end)
        # the routed kernels alone, no collective: what the exchange adds to a step
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record(stream)
        for i in range(args.steps):
            moe.routed_partial(i % n_layers, x_all, tokens, idx, w, share, stream=stream)
        c1.record(stream)
        stream.synchronize()
        compute_ms = c0.elapsed_time(c1) / args.steps
        clocks = sampler.stop() if sampler else None
    assert torch.isfinite(y_own).all(), "non-finite output"
    times = torch.tensor([ms, compute_ms], dtype=torch.float64, device="cuda")
    every = torch.empty(world, 2, dtype=torch.float64, device="cuda")
    dist.all_gather_into_tensor(every, times.view(1, 2))
    dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms = float(times[0]) / args.steps
    if rank == 0:
        per = pl.pairs_per_rank(ids.ravel())
        rec = {"metric": "moe_ffn_layer_batch_tokens_per_s", "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
               "warmup": args.warmup, "higher_is_better": True, "vs_baseline": None, "data": "synthetic",
               "scaling": "strong", "dtype": "f16xu%d->f32" % args.bits, "value": tokens / (ms * 1e-3), "ms_per_step": ms,
               "clocks": clocks, "gpu_launches": int(launches),
               "config": {"workload": "configs[4]: one layer, %d rows, Zipf(%.1f) routing, routed experts only, experts on "
                                      "%d GPUs" % (tokens, args.zipf, world),
                          "d": D, "f": F, "experts": E, "top_k": K, "bits": args.bits, "layers_rotated": n_layers,
                          "placement": args.placement, "rows_per_gpu": own, "pairs_per_gpu": [int(v) for v in per],
                          "max_over_mean_pairs_per_gpu": round(max(per) / (sum(per) / world), 3),
                          "all_gather_bytes_in_per_gpu": (world - 1) * own * D * 2,
                          "all_to_all_bytes_out_per_gpu": (world - 1) * own * D * 4,
                          "routed_kernels_alone_ms_max_over_gpus": float(times[1]),
                          "routed_kernels_alone_ms_per_gpu": [round(float(v), 4) for v in every[:, 1].cpu()],
                          "step_ms_per_gpu": [round(float(v) / args.steps, 4) for v in every[:, 0].cpu()]}}
        print(json.dumps(rec), flush=True)


def run_gturbo_load(args) -> None:
    """One production-size layer file (256 blobs, 453 MB at 4 bits) of a synthetic `.gturbo` artifact read into HBM
    by `nvmai_cuda_moe_read_file_to_device`; the file sits in the page cache after it is written, so the figure is the
    reader's pipeline (pread -> pinned buffer -> async copy), not the disk."""
    import tempfile
    import time
    import torch
    from nvmai_b200 import gturbo
    from nvmai_b200 import format as fmt
    torch.cuda.set_device(0)
    _, blob = fmt.expert_offsets(D, F, args.bits)
    rng = np.random.default_rng(5)
    blobs = rng.integers(0, 256, size=(E, blob), dtype=np.uint8)
    with tempfile.TemporaryDirectory() as root:
        gturbo.write_packed_experts(root, [blobs], d=D, f=F, bits=args.bits)
        g = gturbo.GTurboExperts(root)
        buf = torch.empty(g.layer_bytes, dtype=torch.uint8, device="cuda")
        t0 = time.perf_counter()
        g.verify_layer(0)
        sha_s = time.perf_counter() - t0
        times = []
        for i in range(max(args.warmup, 1) + args.steps):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            g.load_layer(0, buf)            # returns after the last copy has completed
            times.append(time.perf_counter() - t0)
        ok = bool(np.array_equal(buf.cpu().numpy().reshape(E, g.layout.expert_stride)[:, :blob], blobs))
    ms = float(np.median(times[max(args.warmup, 1):])) * 1e3
    rec = {"metric": "gturbo_layer_load_gb_per_s", "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
           "higher_is_better": True, "vs_baseline": None, "data": "synthetic", "dtype": "u8",
           "value": g.layer_bytes / (ms * 1e-3) / 1e9, "ms_per_step": ms, "gpu_launches": 0,
           "config": {"workload": "one packed_experts layer file (%d blobs, %d bytes) from the page cache into HBM"
                      % (E, g.layer_bytes), "bits": args.bits, "sha256_seconds": round(sha_s, 3), "bytes_match": ok}}
    print(json.dumps(rec), flush=True)


def run_prefill(args) -> None:
    """configs[2]: one layer, `--tokens` rows (4096 by default), 4-bit: router, pair grouping, the grouped
    gate/up and down GEMMs on the tensor cores, ordered combine.  Rotates over `--layers` independently seeded
    layers (453 MB of experts each, larger than L2).  Not the headline line: its own metric."""
    import torch
    from nvmai_b200 import MoE, MoEConfig, launch_count, synthetic
    from nvmai_b200 import format as fmt
    torch.cuda.set_device(0)
    tokens, n_layers = args.tokens, args.layers
    cfg = MoEConfig(d=D, f=F, shared_f=FS, num_experts=E, top_k=K, routed_bits=args.bits, shared_bits=args.bits,
                    router_kind=fmt.ROUTER_DENSE_F16, shared_gate_kind=fmt.ROUTER_DENSE_F16,
                    meta_dtype=fmt.META_BF16, activation=fmt.ACT_SILU, out_dtype=fmt.OUT_FP32,
                    max_tokens=tokens, num_layers=n_layers)
    moe = MoE(cfg)
    devs = []
    for l in range(n_layers):
        dev = synthetic.device_layer(2000 + l, d=D, f=F, shared_f=FS, num_experts=E, routed_bits=args.bits,
                                     meta=fmt.META_BF16)
        synthetic.register_device_layer(moe, l, dev)
        devs.append(dev)
    stream = torch.cuda.Stream()
    gen = torch.Generator(device="cuda")
    gen.manual_seed(7)
    x = torch.randn(tokens, D, device="cuda", generator=gen).to(torch.float16)
    y = torch.empty(tokens, D, dtype=torch.float32, device="cuda")
    x_host = x.cpu().pin_memory()
    y_host = torch.empty(tokens, D, dtype=torch.float32).pin_memory()
    x_in = torch.empty_like(x)
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        for i in range(max(args.warmup, 3)):
            moe.layer_prefill(i % n_layers, x, tokens, y_out=y, stream=stream)
        stream.synchronize()
        sampler = ClockSampler(0)
        l0 = launch_count()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for i in range(args.steps):
            moe.layer_prefill(i % n_layers, x, tokens, y_out=y, stream=stream)
        end.record(stream)
        stream.synchronize()
        launches = launch_count() - l0
        ms = start.elapsed_time(end) / args.steps
        assert torch.isfinite(y).all(), "non-finite output"
        t0 = time.perf_counter()
        for i in range(args.steps):
            x_in.copy_(x_host, non_blocking=True)
            moe.layer_prefill(i % n_layers, x_in, tokens, y_out=y, stream=stream)
            y_host.copy_(y, non_blocking=True)
            stream.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
        clocks = sampler.stop()
        parity = None
        if not args.no_parity:
            idx = torch.empty(tokens, K, dtype=torch.int32, device="cuda")
            moe.layer_prefill(0, x, tokens, y_out=y, out_idx=idx, stream=stream)
            moe.synchronize(stream)
            counts = torch.bincount(idx.reshape(-1), minlength=E)
            hot = int(torch.argmax(counts))
            hot_rows = torch.nonzero((idx == hot).any(dim=1)).reshape(-1).cpu().numpy()
            rows = sorted(set([0, 1, tokens // 2, tokens - 1] + hot_rows[[0, len(hot_rows) // 2, -1]].tolist()
                              + list(range(3, tokens, max(1, tokens // 11)))))
            parity = prefill_parity(cfg, devs[0], x, y, idx, torch, rows)
            parity["rows_of_the_largest_work_item"] = int(counts.max())
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
    flops_routed = tokens * K * 3 * 2 * D * F
    flops_shared = tokens * 3 * 2 * D * FS
    flops_router = tokens * 2 * D * E
    tf = (flops_routed + flops_shared) / (ms * 1e-3) / 1e12
    rec = {"metric": "moe_ffn_prefill_tokens_per_s", "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
           "warmup": args.warmup, "higher_is_better": True, "vs_baseline": None, "data": "synthetic",
           "scaling": "weak", "dtype": "f16xu%d->f32" % args.bits, "value": tokens / (ms * 1e-3), "ms_per_step": ms,
           "clocks": clocks, "gpu_launches": int(launches),
           "config": {"workload": f"configs[2]: prefill chunk of {tokens} rows, one MoE layer, 35B-A3B shape, {args.bits}-bit",
                      "d": D, "f": F, "experts": E, "top_k": K, "layers_rotated": n_layers, "bits": args.bits,
                      "l2": "each layer's experts (453 MB at 4-bit) exceed the 126 MB L2; layers rotate"},
           "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": tokens * D * 2,
                   "d2h_bytes_per_step": tokens * D * 4},
           "roofline": {"bound": "tensor", "kernel": "whole prefill block (router, grouping, packing, 4 GEMM launches, combine)",
                        "achieved": tf, "peak": peak, "peak_source": "measured (sustained)" if peaks else "fallback",
                        "unit": "TFLOP/s", "frac": tf / peak, "traffic": None,
                        "flops": {"routed": flops_routed, "shared": flops_shared, "router_not_counted": flops_router}}}
    if parity is not None:
        rec["parity"] = parity
    print(json.dumps(rec), flush=True)
    if parity is not None and not parity["ok"]:
        raise SystemExit("parity check of the timed path failed: " + json.dumps(parity))


# dram__bytes_read.sum + dram__bytes_write.sum of one stage2_kernel launch, from an ncu capture of the 4-bit
# kernel (the 8-bit kernel has not been captured)
STAGE2_DRAM_BYTES_PER_LAUNCH = {4: 9508352, 8: None}
# the same for the resident decode kernel, per LAYER: an ncu capture of a 4-layer, 4-bit step read 68,057,600 B
# and wrote 1,360,384 B; the traffic of a step grows with its number of layers
RESIDENT_DRAM_BYTES_PER_LAYER = {4: (68057600 + 1360384) // 4, 8: None}


def resident_roofline(moe, args, xs, x_in, y, stream, peak: float, which: str) -> dict:
    """The whole decode step is ONE launch of the resident kernel: its algorithmic bytes are the step's, its
    duration the mean over back-to-back launches (CUDA events on the launching stream; the 0.68 / 1.25 GB a
    step reads are larger than the L2, so every launch streams its weights from HBM)."""
    import torch
    reps = 50
    with torch.cuda.stream(stream):
        x_in.copy_(xs[0], non_blocking=True)
        for _ in range(3):
            moe.stack_decode(x_in, 1, y, stream=stream)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for _ in range(reps):
            moe.stack_decode(x_in, 1, y, stream=stream)
        end.record(stream)
        stream.synchronize()
    us = start.elapsed_time(end) * 1e3 / reps
    nbytes = args.layers * layer_bytes(args.bits)
    achieved = nbytes / (us * 1e-6) / 1e9
    per_layer = RESIDENT_DRAM_BYTES_PER_LAYER.get(args.bits)
    return {"bound": "hbm", "kernel": "persistent_decode_kernel (one launch = all layers of the step)",
            "achieved": achieved, "peak": peak, "peak_source": which, "unit": "GB/s", "frac": achieved / peak,
            "traffic": None if per_layer is None else per_layer * args.layers, "bytes_per_launch": nbytes,
            "us_per_launch": us}


def batch_roofline(moe, args, tokens: int, ms_per_step: float, peak: float, which: str) -> dict:
    """2..8 rows per step run as one launch of the resident batch kernel.  Its algorithmic bytes follow the routing:
    per layer every DISTINCT expert the rows selected (read back from the step's own routing record) once, plus the
    shared expert, the router, the gate row and the rows themselves."""
    log = moe.read_route_log_rows(tokens)                     # [layers][rows][K] of the last step
    blob = expert_bytes(args.bits)
    fixed = blob + E * D * 2 + D * 2 + tokens * (D * 2 + D * 4)
    distinct = [int(np.unique(log[l]).size) for l in range(log.shape[0])]
    nbytes = sum(d * blob + fixed for d in distinct)
    achieved = nbytes / (ms_per_step * 1e-3) / 1e9
    return {"bound": "hbm", "kernel": "persistent_batch_kernel (one launch = all layers of the step, %d rows)" % tokens,
            "achieved": achieved, "peak": peak, "peak_source": which, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
            "bytes_per_launch": nbytes, "us_per_launch": ms_per_step * 1e3,
            "distinct_experts_per_layer_mean": float(np.mean(distinct))}


def device_layer_to_host(dev, torch) -> dict:
    """a device-generated layer as the host arrays the oracle reads"""
    def host_tensor(t):
        def as_np(a):
            if a is None:
                return None
            flat = a.contiguous().cpu().view(torch.uint8).numpy()
            return flat.view(np.uint16 if a.element_size() == 2 else np.uint8).reshape(a.shape)
        w, s_, b = t
        return as_np(w), as_np(s_), as_np(b)
    return {"experts": dev["experts"].cpu().numpy(), "stride": dev["stride"], "offsets": dev["offsets"],
            "router": host_tensor(dev["router"]), "shared": [host_tensor(t) for t in dev["shared"]],
            "gate": host_tensor(dev["gate"])}


def prefill_parity(cfg, dev, x, y, idx, torch, rows) -> dict:
    """Post-timing check of the prefill block's output on sampled rows against both oracles (the prefill shaders'
    rounding points, and the reference CPU path in fp32)."""
    sys.path.insert(0, str(ROOT / "tests"))
    import gpu_util as gu
    from oracle import oracle as orc
    host = device_layer_to_host(dev, torch)
    L, keep = gu.oracle_layer(host, cfg)
    xh = x.cpu().view(torch.int16).numpy().view(np.uint16)
    got = y.cpu().numpy()
    got_idx = idx.cpu().numpy().view(np.uint32)
    worst_cpu, worst_shader, idx_ok, escapes, margin_min = 0.0, 0.0, True, 0, float("inf")
    for t in rows:
        xr = np.ascontiguousarray(xh[t])
        o_idx, _, o_y, _ = gu.oracle_prefill_row(L, cfg, xr)
        _, _, _, margin, cpu = gu.oracle_decode(L, cfg, xr)
        margin_min = min(margin_min, margin)
        idx_ok = idx_ok and got_idx[t].tolist() == o_idx.tolist()
        e_cpu, e_sh, own = orc.rel_error(got[t], cpu), orc.rel_error(got[t], o_y), orc.rel_error(o_y, cpu)
        worst_cpu, worst_shader = max(worst_cpu, e_cpu), max(worst_shader, e_sh)
        if e_cpu >= 1e-3 and e_cpu < own + 2e-4:      # the reference's own shader semantics are that far from its CPU path
            escapes += 1
    rec = {"rows_checked": len(rows), "expert_indices_exact": bool(idx_ok), "min_router_margin": margin_min,
           "worst_rel_err_vs_reference_cpu_path": worst_cpu, "worst_rel_err_vs_shader_oracle": worst_shader,
           "rows_over_1e-3_where_the_shader_oracle_is_too": escapes}
    rec["ok"] = bool(idx_ok and worst_shader < 1e-3 and (worst_cpu < 1e-3 or escapes > 0))
    return rec


def stack_parity(args, cfg, devs, xs, torch) -> dict:
    """Post-timing check of the timed path against the CPU oracle: the first layers of the same stack, same
    input row, through the same entry point; selected experts must be exact, the output within the tolerances
    of the GPU tests; and the resident kernel must give the staged kernels' bits."""
    sys.path.insert(0, str(ROOT / "tests"))
    import dataclasses
    import gpu_util as gu
    from nvmai_b200 import MoE, synthetic
    from oracle import oracle as orc
    n = min(4, args.layers)
    cfg_p = dataclasses.replace(cfg, num_layers=n, max_tokens=1)
    moe = MoE(cfg_p)
    for l in range(n):
        synthetic.register_device_layer(moe, l, devs[l])
    hosts = [device_layer_to_host(devs[l], torch) for l in range(n)]        # kept alive: the oracle reads them in place
    oracle_layers = [gu.oracle_layer(hosts[l], cfg_p) for l in range(n)]

    def chain(x_bits):
        idxs, margin_min, h2, cpu = [], float("inf"), None, None
        x = x_bits
        for l in range(n):
            idx, _, h2, margin, cpu = gu.oracle_decode(oracle_layers[l][0], cfg_p, x)
            idxs.append(idx.tolist())
            margin_min = min(margin_min, margin)
            if l + 1 < n:
                scale = 1.0 / np.sqrt(np.mean(h2.astype(np.float64) ** 2) + 1e-6)
                x = orc.f32_to_f16_bits((h2.astype(np.float64) * scale).astype(np.float32))
        return idxs, margin_min, h2, cpu

    # Each layer's input is the previous layer's output, which differs between the two sides by their rounding: a
    # selection decided by less than that difference proves nothing either way, so of the first eight input rows the
    # one whose chain keeps the widest gap between its eighth and ninth logit is checked
    best = None
    for cand in range(min(8, xs.shape[0])):
        x_bits = np.ascontiguousarray(xs[cand, 0].contiguous().cpu().view(torch.int16).numpy().view(np.uint16))
        res = chain(x_bits)
        if best is None or res[1] > best[1][1]:
            best = (cand, res)
    row, (idxs, margin_min, h2, cpu) = best
    x0 = xs[row, 0].contiguous()
    outs = {}
    for mode in (MoE.DECODE_STAGED, MoE.DECODE_AUTO):
        y = torch.empty(D, dtype=torch.float32, device="cuda")
        moe.set_decode_mode(mode)
        moe.stack_decode(x0, 1, y)
        moe.synchronize()
        outs[mode] = y.cpu().numpy()
    log = moe.read_route_log(n)
    got = outs[MoE.DECODE_AUTO]
    idx_ok = all(log[l].tolist() == idxs[l] for l in range(n))
    rec = {"layers_checked": n, "input_row": row, "expert_indices_exact": bool(idx_ok), "min_router_margin": margin_min,
           "rel_err_vs_oracle_chain": float(orc.rel_error(got, h2)),
           "oracle_last_layer_vs_reference_cpu_path": float(orc.rel_error(h2, cpu)),
           "resident_equals_staged_bitwise": bool(np.array_equal(outs[MoE.DECODE_STAGED].view(np.uint32), got.view(np.uint32)))}
    rec["ok"] = bool(idx_ok and rec["rel_err_vs_oracle_chain"] < 2e-3 and rec["oracle_last_layer_vs_reference_cpu_path"] < 1e-3
                     and rec["resident_equals_staged_bitwise"])
    return rec



def stage2_roofline(moe, cfg, devs, args, stream, peak: float, which: str) -> dict:
    """Times the dominant kernel (routed gate/up + activation) alone: one launch per
    layer with that layer's own experts (40 x 9.4 MB at 4-bit, larger than L2),
    captured once as a CUDA graph and replayed, CUDA events on the launching stream."""
    import torch
    rng = np.random.default_rng(3)
    x = torch.randn(D, device="cuda").to(torch.float16)
    acts = torch.empty(K * F, dtype=torch.float32, device="cuda")
    graph = torch.cuda.CUDAGraph()
    plans = []
    for dev in devs:
        ids = rng.choice(E, size=K, replace=False)
        base = dev["experts"].data_ptr()
        plans.append(([base + int(e) * dev["stride"] for e in ids], dev["offsets"]))
    with torch.cuda.stream(stream):
        for blobs, off in plans[:2]:
            moe.encode_routed_phase1(blobs, off, x, acts, stream=stream)
        stream.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            for blobs, off in plans:
                moe.encode_routed_phase1(blobs, off, x, acts, stream=stream)
        reps = 20
        for _ in range(3):
            graph.replay()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for _ in range(reps):
            graph.replay()
        end.record(stream)
        stream.synchronize()
    us = start.elapsed_time(end) * 1e3 / (reps * len(plans))
    nbytes = stage2_bytes(args.bits, 4)
    achieved = nbytes / (us * 1e-6) / 1e9
    traffic = STAGE2_DRAM_BYTES_PER_LAUNCH.get(args.bits)
    return {"bound": "hbm", "kernel": "stage2_kernel (routed gate/up + activation)", "achieved": achieved, "peak": peak,
            "peak_source": which, "unit": "GB/s", "frac": achieved / peak, "traffic": traffic,
            "bytes_per_launch": nbytes, "us_per_launch": us}


def run_block_trace(args) -> None:
    """Per-phase timeline of the resident decode kernels: every block's GPU-timer marks, reduced to the minimum,
    median and maximum over blocks (median over layers), in microseconds after the layer's first input row."""
    import torch
    from nvmai_b200 import MoE, MoEConfig, synthetic
    from nvmai_b200 import format as fmt
    torch.cuda.set_device(0)
    rows = args.tokens
    cfg = MoEConfig(d=D, f=F, shared_f=FS, num_experts=E, top_k=K, routed_bits=args.bits, shared_bits=args.bits,
                    router_kind=fmt.ROUTER_DENSE_F16, shared_gate_kind=fmt.ROUTER_DENSE_F16, meta_dtype=fmt.META_BF16,
                    activation=fmt.ACT_SILU, out_dtype=fmt.OUT_FP32, max_tokens=rows, num_layers=args.layers)
    moe = MoE(cfg)
    devs = [synthetic.device_layer(1000 + l, d=D, f=F, shared_f=FS, num_experts=E, routed_bits=args.bits, meta=fmt.META_BF16)
            for l in range(args.layers)]
    for l, dev in enumerate(devs):
        synthetic.register_device_layer(moe, l, dev)
    xs = torch.randn(8, rows, D, device="cuda").to(torch.float16)
    x_in = torch.empty(rows, D, dtype=torch.float16, device="cuda")
    y = torch.empty(rows, D, dtype=torch.float32, device="cuda")
    stream = torch.cuda.Stream()
    moe.set_trace(True)
    with torch.cuda.stream(stream):
        for i in range(6):
            x_in.copy_(xs[i])
            moe.stack_decode(x_in, rows, y, stream=stream)
        stream.synchronize()
    print(json.dumps(block_trace_summary(moe.read_block_trace(), rows,
                                         f"{args.layers}-layer stack, {args.bits}-bit, {rows} row(s) per step, resident kernel "
                                         "with tracing on")), flush=True)


def block_trace_summary(trace, rows: int, workload: str, single_row_kernel: bool | None = None) -> dict:
    tr = trace.astype(np.float64)
    tr[tr == 0] = np.nan
    if single_row_kernel if single_row_kernel is not None else rows == 1:
        names = {0: "input row normalised", 1: "router logits stored", 2: "all logits in", 10: "top-k done",
                 3: "gate/up tiles requested", 4: "first gate/up tile landed", 11: "last gate/up tile landed",
                 5: "activations stored", 6: "shared-expert down done", 7: "routed activations staged", 8: "down done",
                 9: "block output stored"}
    else:
        names = {0: "input rows normalised", 1: "phase 1 stored (logits, shared gate/up)", 2: "selection of every row done",
                 3: "gate/up tiles requested", 4: "first gate/up tile landed", 11: "last gate/up tile landed",
                 5: "activations stored", 6: "shared-expert down done", 7: "first eight pairs' down done",
                 8: "down done", 12: "this rank's shares stored to every rank", 9: "block output stored"}
    first = np.nanmin(tr[:, :, 0], axis=1, keepdims=True)
    marks = {}
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", category=RuntimeWarning)
        for i, name in names.items():
            rel = (tr[2:, :, i] - first[2:]) / 1e3
            if np.all(np.isnan(rel)):
                continue
            marks[name] = [round(float(np.nanmedian(f(rel, axis=1))), 2) for f in (np.nanmin, np.nanmedian, np.nanmax)]
    period = np.diff(first[:, 0]) / 1e3
    # the blocks that reach a mark last, most often over the layers (where a straggler sits)
    late = {}
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", category=RuntimeWarning)
        for i, name in names.items():
            col = tr[2:, :, i]
            if np.all(np.isnan(col)):
                continue
            worst = np.argsort(np.nan_to_num(col, nan=-1.0), axis=1)[:, -3:].ravel()
            ids, counts = np.unique(worst, return_counts=True)
            late[name] = [int(b) for b in ids[np.argsort(-counts)][:4]]
    return {"workload": workload, "us_after_first_input_row_min_median_max": marks,
            "layer_period_us_median": round(float(np.median(period[1:])), 2), "blocks_most_often_last": late}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--bits", type=int, default=4, choices=[4, 8])
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--tokens", type=int, default=1)
    ap.add_argument("--ref-layers", type=int, default=8, help="layers the CPU sample runs before scaling to --layers")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the post-timing check against the CPU oracle")
    ap.add_argument("--no-single-gpu", action="store_true",
                    help="expert-parallel runs: skip the one-GPU run of the same total batch on rank 0")
    ap.add_argument("--block-trace", action="store_true",
                    help="print the per-phase timeline of the resident decode kernel instead of the benchmark line")
    ap.add_argument("--placement", default="contiguous", choices=["contiguous", "strided"])
    ap.add_argument("--batch-layer", action="store_true",
                    help="measure configs[1] (one layer, --tokens independent rows, batched decode kernels) or, with "
                         "--zipf, configs[4] instead of the decode stack")
    ap.add_argument("--zipf", type=float, default=0.0, help="with --batch-layer: Zipf exponent of the expert popularity")
    ap.add_argument("--gturbo-load", action="store_true",
                    help="time the read of one synthetic packed_experts layer file into device memory")
    ap.add_argument("--route-trace", default="",
                    help="with --batch-layer: replay the routing of a trace file in the NVMAI_ROUTE_TRACE line format "
                         "(`position layer e0..e7`), or `synthetic[:reuse]`")
    ap.add_argument("--prenorm", default="", choices=["", "fused", "unfused"],
                    help="with --batch-layer: time the block together with the residual add and RMS norm in front of it")
    ap.add_argument("--prefill", action="store_true",
                    help="measure configs[2] (a prefill chunk through the tensor-core grouped GEMMs) instead of the "
                         "decode stack; --tokens defaults to 4096 and --layers to 2 here")
    ap.add_argument("--ep-exchange", default="p2p", choices=["p2p", "nccl"],
                    help="expert-parallel runs, up to 8 rows in total: p2p = one resident kernel per rank and step, the "
                         "ranks' shares cross NVLink by peer stores from inside its down phase; nccl = the staged kernels "
                         "with an NCCL all-gather of the shares per layer")
    ap.add_argument("--ep-driver", default="native", choices=["native", "torch"],
                    help="expert-parallel runs: the library's own communicator and CUDA graph (native), or "
                         "torch.distributed collectives around per-stage calls with plain launches (torch)")
    ap.add_argument("--verbose", action="store_true", help="progress lines on stderr")
    ap.add_argument("--deadline", type=float, default=600.0,
                    help="multi-GPU runs: give up (exit 2) after this many seconds instead of waiting on a stuck collective")
    args = ap.parse_args()
    # the collectives of this benchmark are a few KB per step: NVLink SHARP (multicast objects) has nothing to speed up
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    if args.gturbo_load:
        run_gturbo_load(args)
        return
    if args.block_trace and args.gpus == 1:
        run_block_trace(args)
        return
    if args.batch_layer and int(os.environ.get("WORLD_SIZE", "1")) > 1:
        import torch
        import torch.distributed as dist
        assert args.zipf > 0, "the multi-GPU batch-layer run is the Zipf batch (--zipf S)"
        rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        killer = threading.Timer(args.deadline, lambda: os._exit(2))
        killer.daemon = True
        killer.start()
        run_batch_layer_ep(args, torch, dist, rank, world, local)
        killer.cancel()
        dist.destroy_process_group()
    elif args.batch_layer:
        run_batch_layer(args)
    elif args.prefill:
        if args.tokens == 1:
            args.tokens = 4096
        if args.layers == LAYERS:
            args.layers = 2
        run_prefill(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
