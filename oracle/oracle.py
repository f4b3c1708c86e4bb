"""ctypes bindings for the CPU oracle (oracle/nvmai_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg.  The product package never imports this module.

`lib()` loads (building on demand) oracle/liboracle.so; `ref_gemv4()` returns
the reference's own nvmai_int4_affine_gemv from oracle/_ref/libnvmai_ref.so
when that object exists (it is compiled from the reference checkout by
oracle/Makefile and cannot be rebuilt where the checkout is absent).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
META_BF16, META_FP16 = 0, 1
ACT_SILU, ACT_GELU_TANH = 0, 1
OUT_FP16, OUT_FP32 = 0, 1

_lib = None
_ref = None

u8p = C.POINTER(C.c_uint8)
u16p = C.POINTER(C.c_uint16)
u32p = C.POINTER(C.c_uint32)
f32p = C.POINTER(C.c_float)
f64p = C.POINTER(C.c_double)

GEMV4_FN = C.CFUNCTYPE(None, u8p, u16p, u16p, f32p, C.c_size_t, C.c_size_t, f32p)


def reference_root() -> Path | None:
    """The reference checkout: $NVMAI_REF_ROOT, else a `reference` directory beside this repository."""
    env = os.environ.get("NVMAI_REF_ROOT")
    for cand in ([Path(env)] if env else []) + [HERE.parent.parent / "reference"]:
        if (cand / "sources/NVMAIKernelsC/int4_affine_gemv.c").exists():
            return cand
    return None


def build(force: bool = False) -> None:
    for so, srcs in (("liboracle.so", ["nvmai_oracle.c"]), ("libcpu_stack.so", ["cpu_stack.cpp", "nvmai_oracle.c"])):
        out = HERE / so
        if force or not out.exists() or any(out.stat().st_mtime < (HERE / s).stat().st_mtime for s in srcs):
            subprocess.run(["make", "-C", str(HERE), so], check=True, stdout=subprocess.DEVNULL)
    ref_root = reference_root()
    if ref_root is not None:
        ref_so = HERE / "_ref" / "libnvmai_ref.so"
        if force or not ref_so.exists():
            subprocess.run(["make", "-C", str(HERE), "ref", f"REF_ROOT={ref_root}"], check=True,
                           stdout=subprocess.DEVNULL)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(str(HERE / "liboracle.so"))
        _declare(_lib)
    return _lib


class StackDesc(C.Structure):
    _fields_ = [("d", C.c_int), ("f", C.c_int), ("e", C.c_int), ("k", C.c_int), ("bits", C.c_int), ("layers", C.c_int),
                ("blobs", C.POINTER(C.c_void_p)), ("stride", C.c_uint64), ("off", C.c_uint32 * 9),
                ("router_f16", C.POINTER(C.c_void_p)), ("gate_f16", C.POINTER(C.c_void_p))]


_stack = None


def cpu_stack_lib() -> C.CDLL:
    """The threaded CPU-baseline driver (cpu_stack.cpp)."""
    global _stack
    if _stack is None:
        build()
        _stack = C.CDLL(str(HERE / "libcpu_stack.so"))
        _stack.orc_cpu_stack_time.argtypes = [C.POINTER(StackDesc), C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int,
                                              C.c_void_p, C.c_void_p]
        _stack.orc_cpu_stack_time.restype = C.c_double
    return _stack


def ref_lib():
    """The reference's own C kernel (or None when it was never built)."""
    global _ref
    if _ref is None:
        p = HERE / "_ref" / "libnvmai_ref.so"
        if not p.exists():
            return None
        _ref = C.CDLL(str(p))
        _ref.nvmai_int4_affine_gemv.argtypes = [u8p, u16p, u16p, f32p, C.c_size_t, C.c_size_t, f32p]
        _ref.nvmai_int4_affine_gemv.restype = None
    return _ref


def ref_gemv4_ptr():
    r = ref_lib()
    if r is None:
        return C.cast(None, GEMV4_FN)
    return C.cast(r.nvmai_int4_affine_gemv, GEMV4_FN)


class Layer(C.Structure):
    _fields_ = [
        ("D", C.c_uint32), ("F", C.c_uint32), ("E", C.c_uint32), ("K", C.c_uint32), ("Fs", C.c_uint32),
        ("routed_bits", C.c_int), ("shared_bits", C.c_int), ("meta", C.c_int), ("act", C.c_int),
        ("out_dtype", C.c_int), ("router_kind", C.c_int), ("shared_gate_kind", C.c_int),
        ("experts", C.c_void_p), ("stride", C.c_uint64), ("off", C.c_uint32 * 9),
        ("router_W", C.c_void_p), ("router_S", C.c_void_p), ("router_B", C.c_void_p),
        ("eff_scale", C.c_void_p), ("per_expert_scale", C.c_void_p),
        ("shared", C.c_void_p * 9),
        ("sgate_W", C.c_void_p), ("sgate_S", C.c_void_p), ("sgate_B", C.c_void_p),
    ]


class Pair(C.Structure):
    _fields_ = [("token", C.c_uint32), ("expert", C.c_uint32), ("rank", C.c_uint32),
                ("weight_bits", C.c_uint32)]


PAIR_DTYPE = np.dtype([("token", "<u4"), ("expert", "<u4"), ("rank", "<u4"), ("weight_bits", "<u4")])


def _declare(L: C.CDLL) -> None:
    vp = C.c_void_p
    sz = C.c_size_t
    L.orc_bf16_to_f32.argtypes = [C.c_uint16]; L.orc_bf16_to_f32.restype = C.c_float
    L.orc_f32_to_bf16.argtypes = [C.c_float]; L.orc_f32_to_bf16.restype = C.c_uint16
    L.orc_f32_to_bf16_trunc.argtypes = [C.c_float]; L.orc_f32_to_bf16_trunc.restype = C.c_uint16
    L.orc_f16_to_f32.argtypes = [C.c_uint16]; L.orc_f16_to_f32.restype = C.c_float
    L.orc_f32_to_f16.argtypes = [C.c_float]; L.orc_f32_to_f16.restype = C.c_uint16
    L.orc_round11.argtypes = [C.c_float]; L.orc_round11.restype = C.c_float
    L.orc_splitmix_next.argtypes = [C.POINTER(C.c_uint64)]; L.orc_splitmix_next.restype = C.c_uint64
    L.orc_splitmix_uniform.argtypes = [C.POINTER(C.c_uint64), C.c_float, C.c_float]
    L.orc_splitmix_uniform.restype = C.c_float
    L.orc_splitmix_fill_uniform.argtypes = [C.POINTER(C.c_uint64), C.c_float, C.c_float, vp, sz]
    L.orc_splitmix_fill_uniform.restype = None
    L.orc_seedtree_key.argtypes = [C.c_uint64, C.c_char_p]; L.orc_seedtree_key.restype = C.c_uint64
    L.orc_lcg_fill.argtypes = [C.POINTER(C.c_uint64), C.c_uint64, vp, sz]; L.orc_lcg_fill.restype = None
    L.orc_quantize_affine.argtypes = [C.c_int, vp, sz, sz, C.c_int, vp, vp, vp]
    L.orc_quantize_affine.restype = None
    L.orc_dequant_affine.argtypes = [C.c_int, C.c_int, vp, vp, vp, sz, sz, vp]
    L.orc_dequant_affine.restype = None
    L.orc_expert_offsets.argtypes = [sz, sz, C.c_int, vp]; L.orc_expert_offsets.restype = None
    L.orc_affine_gemv_f32.argtypes = [C.c_int, C.c_int, vp, vp, vp, vp, sz, sz, vp]
    L.orc_affine_gemv_f32.restype = None
    L.orc_cpu_expert_accumulate.argtypes = [vp, vp, C.c_int, C.c_int, C.c_int, vp, sz, sz,
                                            C.c_float, vp, vp, GEMV4_FN]
    L.orc_cpu_expert_accumulate.restype = None
    L.orc_router_logits_affine.argtypes = [C.c_int, C.c_int, vp, vp, vp, vp, vp, sz, sz, vp, vp]
    L.orc_router_logits_affine.restype = None
    L.orc_router_logits_dense_f16.argtypes = [vp, vp, vp, sz, sz, vp, vp]
    L.orc_router_logits_dense_f16.restype = None
    L.orc_topk_softmax.argtypes = [vp, sz, sz, vp, vp, vp, vp, vp]; L.orc_topk_softmax.restype = None
    L.orc_gpu_phase1.argtypes = [vp, vp, C.c_int, C.c_int, C.c_int, vp, sz, sz, sz, vp, sz, C.c_int, vp]
    L.orc_gpu_phase1.restype = None
    L.orc_gpu_phase2.argtypes = [vp, vp, C.c_int, C.c_int, vp, vp, vp, sz, sz, sz, C.c_int, vp]
    L.orc_gpu_phase2.restype = None
    L.orc_gpu_affine_gemv_f16.argtypes = [C.c_int, C.c_int, vp, vp, vp, vp, sz, sz, vp, vp]
    L.orc_gpu_affine_gemv_f16.restype = None
    L.orc_gpu_shared_expert.argtypes = [vp, C.c_int, C.c_int, C.c_int, vp, vp, vp, C.c_int, vp,
                                        sz, sz, C.c_int, vp]
    L.orc_gpu_shared_expert.restype = None
    L.orc_gpu_residual_add.argtypes = [vp, vp, sz, C.c_int]; L.orc_gpu_residual_add.restype = None
    L.orc_gpu_rmsnorm_bf16w.argtypes = [vp, vp, vp, sz, C.c_float, C.c_int]; L.orc_gpu_rmsnorm_bf16w.restype = None
    L.orc_group_pairs.argtypes = [vp, sz, C.c_long, C.c_long, C.c_long, C.c_long, vp, sz, vp, vp,
                                  vp, vp, C.POINTER(sz), vp, C.POINTER(sz)]
    L.orc_group_pairs.restype = C.c_int
    L.orc_gpu_prefill_reduce.argtypes = [vp, vp, sz, sz, sz, vp]; L.orc_gpu_prefill_reduce.restype = None
    L.orc_gpu_layer_decode.argtypes = [C.POINTER(Layer), vp, vp, vp, vp, vp, vp]
    L.orc_gpu_layer_decode.restype = None
    L.orc_gpu_layer_prefill_row.argtypes = [C.POINTER(Layer), vp, vp, vp, vp, vp, vp]
    L.orc_gpu_layer_prefill_row.restype = None
    L.orc_cpu_layer_decode.argtypes = [C.POINTER(Layer), vp, vp, vp, vp, GEMV4_FN]
    L.orc_cpu_layer_decode.restype = None
    L.orc_rel_error.argtypes = [vp, vp, sz]; L.orc_rel_error.restype = C.c_float


def ptr(a: np.ndarray | None):
    """void* of a C-contiguous numpy array (None -> NULL)."""
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle wants C-contiguous arrays"
    return a.ctypes.data_as(C.c_void_p)


# --------------------------------------------------------------------------
# numpy-level conveniences
# --------------------------------------------------------------------------

class SplitMix64:
    """sources/NVMAIValidation/Support/PRNG/SplitMix64.swift restated (state in C)."""

    def __init__(self, seed: int):
        self.state = C.c_uint64(seed & 0xFFFFFFFFFFFFFFFF)

    def next(self) -> int:
        return lib().orc_splitmix_next(C.byref(self.state))

    def uniform(self, lo: float, hi: float) -> float:
        return float(lib().orc_splitmix_uniform(C.byref(self.state), lo, hi))

    def uniform_array(self, lo: float, hi: float, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        lib().orc_splitmix_fill_uniform(C.byref(self.state), lo, hi, ptr(out), n)
        return out


def seedtree_key(root: int, label: str) -> SplitMix64:
    return SplitMix64(lib().orc_seedtree_key(root, label.encode()))


def lcg_array(state: int, inc: int, n: int) -> tuple[np.ndarray, int]:
    s = C.c_uint64(state)
    out = np.empty(n, dtype=np.float32)
    lib().orc_lcg_fill(C.byref(s), inc, ptr(out), n)
    return out, s.value


def f32_to_f16_bits(x: np.ndarray) -> np.ndarray:
    return np.asarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def f16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return np.asarray(b, dtype=np.uint16).view(np.float16).astype(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Quantization.swift:16-23 vectorised (RNE, no NaN handling)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    lsb = (u >> 16) & 1
    return ((u + (0x7FFF + lsb)) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def quantize(bits: int, w: np.ndarray, use_division: bool = False):
    """Rows of fp32 -> (packed u8 [rows, n*bits/8], scales u16 [rows, n/64], biases)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, n = w.shape
    packed = np.zeros((rows, n * bits // 8), dtype=np.uint8)
    scales = np.zeros((rows, n // 64), dtype=np.uint16)
    biases = np.zeros((rows, n // 64), dtype=np.uint16)
    lib().orc_quantize_affine(bits, ptr(w), rows, n, int(use_division), ptr(packed), ptr(scales), ptr(biases))
    return packed, scales, biases


def dequant(bits: int, meta: int, packed, scales, biases, rows: int, n: int) -> np.ndarray:
    out = np.empty((rows, n), dtype=np.float32)
    lib().orc_dequant_affine(bits, meta, ptr(packed), ptr(scales), ptr(biases), rows, n, ptr(out))
    return out


def expert_offsets(d: int, f: int, bits: int) -> np.ndarray:
    out = np.zeros(10, dtype=np.uint32)
    lib().orc_expert_offsets(d, f, bits, ptr(out))
    return out


def rel_error(actual, reference) -> float:
    a = np.ascontiguousarray(actual, dtype=np.float32).ravel()
    r = np.ascontiguousarray(reference, dtype=np.float32).ravel()
    assert a.size == r.size
    return float(lib().orc_rel_error(ptr(a), ptr(r), a.size))


def make_layer(*, D, F, E, K, Fs, routed_bits, shared_bits, meta, act, out_dtype, router_kind,
               shared_gate_kind, experts: np.ndarray, stride: int, off, router, eff_scale=None,
               per_expert_scale=None, shared=None, sgate=None) -> tuple[Layer, list]:
    """Fill an orc_layer.  Returns (struct, keepalive list of arrays)."""
    L = Layer()
    keep = [experts]
    L.D, L.F, L.E, L.K, L.Fs = D, F, E, K, Fs
    L.routed_bits, L.shared_bits, L.meta, L.act, L.out_dtype = routed_bits, shared_bits, meta, act, out_dtype
    L.router_kind, L.shared_gate_kind = router_kind, shared_gate_kind
    L.experts = experts.ctypes.data
    L.stride = stride
    for i in range(9):
        L.off[i] = int(off[i])
    rw, rs, rb = router
    keep += [rw, rs, rb, eff_scale, per_expert_scale]
    L.router_W = rw.ctypes.data
    L.router_S = rs.ctypes.data if rs is not None else None
    L.router_B = rb.ctypes.data if rb is not None else None
    L.eff_scale = eff_scale.ctypes.data if eff_scale is not None else None
    L.per_expert_scale = per_expert_scale.ctypes.data if per_expert_scale is not None else None
    if shared is not None:
        for i, a in enumerate(shared):
            keep.append(a)
            L.shared[i] = a.ctypes.data
    if sgate is not None:
        gw, gs, gb = sgate
        keep += [gw, gs, gb]
        L.sgate_W = gw.ctypes.data
        L.sgate_S = gs.ctypes.data if gs is not None else None
        L.sgate_B = gb.ctypes.data if gb is not None else None
    return L, keep
