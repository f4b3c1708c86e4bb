"""Seeded synthetic MoE layers with the benchmark's value distributions.

Codes uniform over the code range; router and gate dense fp16 ~ N(0, 0.02); hidden
rows fp16 ~ N(0, 1).  numpy builds a layer on the host (tests, single-layer runs:
scale ~ U(0.005, 0.02) and bias ~ U(-0.08, 0) per (row, group), drawn in fp32 and
rounded once to the 16-bit meta type); `device_layer` builds the benchmark's layers
directly in device memory with torch's CUDA generator (tens of GB would be too slow
to make on the host and upload), with the scales and biases of a min/max quantizer
over zero-mean weights so that a deep stack keeps its routing diverse.
"""
from __future__ import annotations

import numpy as np

from . import format as fmt


def affine_tensor(rng: np.random.Generator, rows: int, n: int, bits: int, meta: int):
    """(packed u8 [rows, n*bits/8], scales u16 [rows, n/64], biases u16 [rows, n/64])."""
    packed = rng.integers(0, 256, size=(rows, n * bits // 8), dtype=np.uint8)
    scales = rng.uniform(0.005, 0.02, size=(rows, n // fmt.GROUP)).astype(np.float32)
    biases = rng.uniform(-0.08, 0.0, size=(rows, n // fmt.GROUP)).astype(np.float32)
    return packed, fmt.f32_to_meta_bits(scales, meta), fmt.f32_to_meta_bits(biases, meta)


def layer(seed: int, *, d: int = 2048, f: int = 512, shared_f: int = 512, num_experts: int = 256,
          routed_bits: int = 4, shared_bits: int | None = None, meta: int = fmt.META_FP16,
          router_kind: int = fmt.ROUTER_DENSE_F16, gate_kind: int = fmt.ROUTER_DENSE_F16) -> dict:
    """One layer's host arrays: experts u8 [E, stride], router, shared projections, gate row."""
    rng = np.random.default_rng(seed)
    shared_bits = routed_bits if shared_bits is None else shared_bits
    off, stride = fmt.expert_offsets(d, f, routed_bits)
    experts = np.empty((num_experts, stride), dtype=np.uint8)
    for e in range(num_experts):
        experts[e] = fmt.pack_expert_blob(affine_tensor(rng, f, d, routed_bits, meta),
                                          affine_tensor(rng, f, d, routed_bits, meta),
                                          affine_tensor(rng, d, f, routed_bits, meta), d, f, routed_bits)
    out = {"experts": experts, "stride": stride, "offsets": off}
    if router_kind == fmt.ROUTER_DENSE_F16:
        out["router"] = (fmt.f32_to_f16_bits(rng.normal(0.0, 0.02, size=(num_experts, d))), None, None)
    else:
        out["router"] = affine_tensor(rng, num_experts, d, router_kind, meta)
    if shared_f:
        out["shared"] = (affine_tensor(rng, shared_f, d, shared_bits, meta),
                         affine_tensor(rng, shared_f, d, shared_bits, meta),
                         affine_tensor(rng, d, shared_f, shared_bits, meta))
        if gate_kind == fmt.ROUTER_DENSE_F16:
            out["gate"] = (fmt.f32_to_f16_bits(rng.normal(0.0, 0.02, size=(1, d))), None, None)
        elif gate_kind != fmt.GATE_NONE:
            out["gate"] = affine_tensor(rng, 1, d, gate_kind, meta)
    return out


def hidden_rows(seed: int, tokens: int, d: int = 2048) -> np.ndarray:
    """fp16 bit patterns [tokens, d] ~ N(0, 1)."""
    rng = np.random.default_rng(seed)
    return fmt.f32_to_f16_bits(rng.normal(0.0, 1.0, size=(tokens, d)))


# ---------------------------------------------------------------------------
# device-side generation (torch is plumbing here: allocation + RNG only)
# ---------------------------------------------------------------------------

def _device_meta(torch, gen, shape, bits: int, mdt, device):
    """Scales and biases of a min/max group quantizer over zero-mean weights: the scale spans U(0.005, 0.02) at 4 bits
    (the same weight range at 8), the bias sits half the code range below zero, within 10 %.  The weights of a row
    then have no common sign, so a stack of such layers keeps routing different rows to different experts (with a
    one-sided bias every block output is nearly a constant vector and every row of a layer picks the same experts)."""
    top = float((1 << bits) - 1)
    s = (torch.rand(shape, device=device, generator=gen) * 0.015 + 0.005) * (15.0 / top)
    b = -s * (top / 2.0) * (torch.rand(shape, device=device, generator=gen) * 0.2 + 0.9)
    return s.to(mdt), b.to(mdt)


def _device_affine(torch, gen, rows: int, n: int, bits: int, meta: int, device):
    mdt = torch.bfloat16 if meta == fmt.META_BF16 else torch.float16
    w = torch.randint(0, 256, (rows, n * bits // 8), dtype=torch.uint8, device=device, generator=gen)
    s, b = _device_meta(torch, gen, (rows, n // fmt.GROUP), bits, mdt, device)
    return w, s, b


def device_layer(seed: int, *, d: int = 2048, f: int = 512, shared_f: int = 512, num_experts: int = 256,
                 routed_bits: int = 4, shared_bits: int | None = None, meta: int = fmt.META_BF16,
                 expert_ids=None, device="cuda") -> dict:
    """One layer generated in device memory with the benchmark distributions
    (dense fp16 router and gate row).  `expert_ids` restricts generation to a
    subset of blobs (expert-parallel ranks own 256/N of them); the returned
    `experts` tensor then holds only those, in the given order."""
    import torch
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    shared_bits = routed_bits if shared_bits is None else shared_bits
    off, stride = fmt.expert_offsets(d, f, routed_bits)
    n_local = num_experts if expert_ids is None else len(expert_ids)
    mdt = torch.bfloat16 if meta == fmt.META_BF16 else torch.float16
    experts = torch.randint(0, 256, (n_local, stride), dtype=torch.uint8, device=device, generator=gen)
    gate_m = f * (d // fmt.GROUP) * 2
    down_m = d * (f // fmt.GROUP) * 2
    for name, nbytes in (("gate", gate_m), ("up", gate_m), ("down", down_m)):
        sc, bi = _device_meta(torch, gen, (n_local, nbytes // 2), routed_bits, mdt, device)
        experts[:, off[name + "_s"]:off[name + "_s"] + nbytes] = sc.view(torch.uint8)
        experts[:, off[name + "_b"]:off[name + "_b"] + nbytes] = bi.view(torch.uint8)
    out = {"experts": experts, "stride": stride, "offsets": off}
    out["router"] = ((torch.randn(num_experts, d, device=device, generator=gen) * 0.02).to(torch.float16), None, None)
    if shared_f:
        out["shared"] = [_device_affine(torch, gen, shared_f, d, shared_bits, meta, device),
                         _device_affine(torch, gen, shared_f, d, shared_bits, meta, device),
                         _device_affine(torch, gen, d, shared_f, shared_bits, meta, device)]
        out["gate"] = ((torch.randn(1, d, device=device, generator=gen) * 0.02).to(torch.float16), None, None)
    return out


def register_device_layer(moe, layer: int, dev: dict) -> None:
    moe.register_layer(layer, experts=dev["experts"], expert_stride=dev["stride"], offsets=dev["offsets"],
                       router=dev["router"], shared=dev.get("shared"), shared_gate=dev.get("gate"))
