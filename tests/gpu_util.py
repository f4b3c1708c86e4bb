"""Helpers for the GPU parity tests: device upload through torch (plumbing only)
and construction of matching oracle / library layer descriptions."""
from __future__ import annotations

import numpy as np

from nvmai_b200 import MoE, MoEConfig
from nvmai_b200 import format as fmt
from oracle import oracle as orc


def torch_cuda():
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("CUDA device required")
    return torch


def to_dev(a: np.ndarray):
    """numpy -> CUDA tensor of the same bytes (uint8/16/32 kept as raw integer views)."""
    torch = torch_cuda()
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        t = torch.from_numpy(a.view(np.int16))
    elif a.dtype == np.uint32:
        t = torch.from_numpy(a.view(np.int32))
    else:
        t = torch.from_numpy(a)
    return t.cuda()


def dev_empty(n: int, dtype: str):
    torch = torch_cuda()
    dt = {"u8": torch.uint8, "f16": torch.int16, "u32": torch.int32, "f32": torch.float32}[dtype]
    return torch.zeros(n, dtype=dt, device="cuda")


def from_dev(t, dtype) -> np.ndarray:
    a = t.cpu().numpy()
    return a.view(dtype)


def dev_tensor3(t):
    """(w, s, b) numpy (s/b may be None) -> device triple"""
    w, s, b = t
    return (to_dev(w), None if s is None else to_dev(s), None if b is None else to_dev(b))


class DeviceLayer:
    """One synthetic layer resident on the device and described to both sides."""

    def __init__(self, host: dict):
        self.host = host
        self.experts = to_dev(host["experts"])
        self.router = dev_tensor3(host["router"])
        self.shared = [dev_tensor3(t) for t in host["shared"]] if "shared" in host else None
        self.gate = dev_tensor3(host["gate"]) if "gate" in host else None
        self.eff = to_dev(host["eff"]) if host.get("eff") is not None else None
        self.pes = to_dev(host["pes"]) if host.get("pes") is not None else None

    def register(self, moe: MoE, layer: int) -> None:
        moe.register_layer(layer, experts=self.experts, expert_stride=self.host["stride"],
                           offsets=self.host["offsets"], router=self.router, effective_scale=self.eff,
                           per_expert_scale=self.pes, shared=self.shared, shared_gate=self.gate)


def oracle_layer(host: dict, cfg: MoEConfig):
    off = [host["offsets"][n] for n in fmt.OFFSET_NAMES]
    shared = None
    if "shared" in host:
        shared = [a for t in host["shared"] for a in t]
    gate_kind = -1 if ("gate" not in host or cfg.shared_gate_kind == fmt.GATE_NONE) else cfg.shared_gate_kind
    return orc.make_layer(D=cfg.d, F=cfg.f, E=cfg.num_experts, K=cfg.top_k, Fs=cfg.shared_f,
                          routed_bits=cfg.routed_bits, shared_bits=cfg.shared_bits, meta=cfg.meta_dtype,
                          act=cfg.activation, out_dtype=cfg.out_dtype, router_kind=cfg.router_kind,
                          shared_gate_kind=gate_kind, experts=host["experts"], stride=host["stride"], off=off,
                          router=host["router"], eff_scale=host.get("eff"), per_expert_scale=host.get("pes"),
                          shared=shared, sgate=host.get("gate"))


def oracle_decode(L, cfg: MoEConfig, x_f16_row: np.ndarray):
    """-> (idx, w16, h2 in out dtype as fp32, margin, cpu-path fp32 output)"""
    lib = orc.lib()
    import ctypes as C
    idx = np.zeros(cfg.top_k, dtype=np.uint32)
    w16 = np.zeros(cfg.top_k, dtype=np.uint16)
    h2 = np.zeros(cfg.d, dtype=np.uint16 if cfg.out_dtype == fmt.OUT_FP16 else np.float32)
    margin = np.zeros(1, dtype=np.float32)
    lib.orc_gpu_layer_decode(C.byref(L), orc.ptr(x_f16_row), None, orc.ptr(idx), orc.ptr(w16), orc.ptr(h2),
                             orc.ptr(margin))
    cpu = np.zeros(cfg.d, dtype=np.float32)
    lib.orc_cpu_layer_decode(C.byref(L), orc.ptr(x_f16_row), orc.ptr(idx), orc.ptr(w16), orc.ptr(cpu),
                             orc.ref_gemv4_ptr())
    h2f = orc.f16_bits_to_f32(h2) if cfg.out_dtype == fmt.OUT_FP16 else h2
    return idx, w16, h2f, float(margin[0]), cpu


def oracle_prefill_row(L, cfg: MoEConfig, x_f16_row: np.ndarray, hidden_row: np.ndarray | None = None):
    """One row with the prefill path's rounding points -> (idx, w16, y as fp32, hidden out as fp32 or None)."""
    lib = orc.lib()
    import ctypes as C
    f16 = cfg.out_dtype == fmt.OUT_FP16
    idx = np.zeros(cfg.top_k, dtype=np.uint32)
    w16 = np.zeros(cfg.top_k, dtype=np.uint16)
    y = np.zeros(cfg.d, dtype=np.uint16 if f16 else np.float32)
    hid = None if hidden_row is None else np.ascontiguousarray(hidden_row).copy()
    lib.orc_gpu_layer_prefill_row(C.byref(L), orc.ptr(x_f16_row), orc.ptr(hid), orc.ptr(y), orc.ptr(idx), orc.ptr(w16),
                                  None)
    to32 = (lambda a: orc.f16_bits_to_f32(a)) if f16 else (lambda a: a)
    return idx, w16, to32(y), (None if hid is None else to32(hid))
