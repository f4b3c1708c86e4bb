"""NVMAIRepack expert-blob layout and 16-bit float helpers (host side, numpy).

Layout of one routed expert (sources/NVMAIRepack/Core/Planning/RepackPlanner.swift:365-426,
sources/NVMAI/Kernels/CPU/CPUExpertFFN.swift:42-59): gate W | gate scales | gate
biases | up W | up scales | up biases | down W | down scales | down biases, every
tensor contiguous, W rows packed LSB-first (`bits` per code), one 16-bit scale
and bias per 64 inputs.
"""
from __future__ import annotations

import numpy as np

GROUP = 64
META_BF16, META_FP16 = 0, 1
ACT_SILU, ACT_GELU_TANH = 0, 1
OUT_FP16, OUT_FP32 = 0, 1
ROUTER_DENSE_F16, ROUTER_AFFINE4, ROUTER_AFFINE8 = 0, 4, 8
GATE_NONE = 0xFFFFFFFF

OFFSET_NAMES = ("gate_w", "gate_s", "gate_b", "up_w", "up_s", "up_b", "down_w", "down_s", "down_b")


def expert_offsets(d: int, f: int, bits: int) -> tuple[dict[str, int], int]:
    """Byte offsets of the nine sub-tensors and the blob stride (CPUExpertFFN.swift:42-59)."""
    if d % GROUP or f % GROUP:
        raise ValueError(f"d={d} and f={f} must be multiples of {GROUP}")
    gate_w = f * d * bits // 8
    gate_m = f * (d // GROUP) * 2
    down_w = d * f * bits // 8
    down_m = d * (f // GROUP) * 2
    sizes = (gate_w, gate_m, gate_m, gate_w, gate_m, gate_m, down_w, down_m, down_m)
    off, o = {}, 0
    for name, size in zip(OFFSET_NAMES, sizes):
        off[name] = o
        o += size
    return off, o


def f32_to_bf16_bits(x) -> np.ndarray:
    """Round-to-nearest-even bf16 bit patterns (Quantization.swift:16-23)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    lsb = (u >> 16) & 1
    return ((u + (0x7FFF + lsb)) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_f16_bits(x) -> np.ndarray:
    return np.asarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def f16_bits_to_f32(b) -> np.ndarray:
    return np.asarray(b, dtype=np.uint16).view(np.float16).astype(np.float32)


def f32_to_meta_bits(x, meta: int) -> np.ndarray:
    return f32_to_bf16_bits(x) if meta == META_BF16 else f32_to_f16_bits(x)


def pack_expert_blob(gate, up, down, d: int, f: int, bits: int) -> np.ndarray:
    """gate/up/down = (packed u8 [rows, n*bits/8], scales u16 [rows, n/64], biases u16)."""
    off, stride = expert_offsets(d, f, bits)
    blob = np.zeros(stride, dtype=np.uint8)
    for prefix, (w, s, b) in (("gate", gate), ("up", up), ("down", down)):
        for name, arr in ((f"{prefix}_w", w), (f"{prefix}_s", s), (f"{prefix}_b", b)):
            raw = np.ascontiguousarray(arr).view(np.uint8).ravel()
            blob[off[name]:off[name] + raw.size] = raw
    return blob
