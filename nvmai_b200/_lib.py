"""Loads libnvmai_cuda_moe.so and declares its C ABI for ctypes.

There is no fallback: if the shared object is missing (or was built without the
CUDA toolkit) importing the bindings raises.  Build it with
`python -m nvmai_b200.build`.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libnvmai_cuda_moe.so"

OK, EINVAL, ERANGE, ENOMEM, ECUDA, ETIMEOUT, ENCCL, EIO = 0, 22, 34, 12, 1001, 1002, 1003, 5


class Config(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in (
        "d", "f", "shared_f", "num_experts", "top_k", "routed_bits", "shared_bits", "router_kind",
        "shared_gate_kind", "meta_dtype", "activation", "out_dtype", "max_tokens", "num_layers")]


class ExpertOffsets(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in (
        "gate_w", "gate_s", "gate_b", "up_w", "up_s", "up_b", "down_w", "down_s", "down_b")]


class AffineTensor(C.Structure):
    _fields_ = [("w", C.c_void_p), ("scales", C.c_void_p), ("biases", C.c_void_p)]


class Layer(C.Structure):
    _fields_ = [
        ("experts", C.c_void_p), ("expert_stride", C.c_uint64), ("offsets", ExpertOffsets),
        ("router", AffineTensor), ("effective_scale", C.c_void_p), ("per_expert_scale", C.c_void_p),
        ("shared_gate_proj", AffineTensor), ("shared_up_proj", AffineTensor),
        ("shared_down_proj", AffineTensor), ("shared_gate", AffineTensor),
    ]


_lib = None

# name -> (restype, argtypes); the list the ABI test checks against include/nvmai_cuda_moe.h
vp, u32, u64 = C.c_void_p, C.c_uint32, C.c_uint64
PROTOTYPES = {
    "nvmai_cuda_moe_expert_offsets": (u64, [u32, u32, u32, C.POINTER(ExpertOffsets)]),
    "nvmai_cuda_moe_create": (vp, [C.POINTER(Config), C.POINTER(C.c_int)]),
    "nvmai_cuda_moe_destroy": (None, [vp]),
    "nvmai_cuda_moe_register_layer": (C.c_int, [vp, u32, C.POINTER(Layer)]),
    "nvmai_cuda_moe_router": (C.c_int, [vp, u32, vp, u32, u32, vp, vp, vp]),
    "nvmai_cuda_moe_router_noalloc": (C.c_int, [C.POINTER(Config), C.POINTER(AffineTensor), vp, vp, vp, u32, u32, vp, vp, vp]),
    "nvmai_cuda_moe_router_noalloc_status": (C.c_int, [vp]),
    "nvmai_cuda_moe_shared_expert": (C.c_int, [vp, u32, vp, u32, u32, vp, vp]),
    "nvmai_cuda_moe_routed_phase1": (C.c_int, [vp, C.POINTER(vp), C.POINTER(ExpertOffsets), vp, vp,
                                                C.POINTER(u32), u32, vp]),
    "nvmai_cuda_moe_routed_phase2": (C.c_int, [vp, C.POINTER(vp), C.POINTER(ExpertOffsets), vp, vp, vp, vp, vp]),
    "nvmai_cuda_moe_layer_decode": (C.c_int, [vp, u32, vp, u32, vp, vp, vp, vp, vp]),
    "nvmai_cuda_moe_layer_verify_pair": (C.c_int, [vp, u32, vp, vp, vp, vp, vp, vp]),
    "nvmai_cuda_moe_layer_decode_prenorm": (C.c_int, [vp, u32, vp, vp, vp, C.c_float, u32, vp, vp, vp, vp, vp]),
    "nvmai_cuda_moe_layer_decode_fused_norms": (C.c_int, [vp, u32, vp, vp, vp, C.c_float, u32, vp, C.c_float, vp, vp, vp, vp,
                                                          vp, vp]),
    "nvmai_cuda_moe_group_pairs": (C.c_int, [vp, vp, vp, u32, vp, vp, vp, vp]),
    "nvmai_cuda_moe_set_expert_map": (C.c_int, [vp, vp, u32]),
    "nvmai_cuda_moe_routed_partial": (C.c_int, [vp, u32, vp, u32, vp, vp, vp, vp]),
    "nvmai_cuda_moe_ep_finalize": (C.c_int, [vp, vp, u32, vp, u32, vp, vp, vp]),
    "nvmai_cuda_moe_rms_renorm": (C.c_int, [vp, vp, u32, vp, vp]),
    "nvmai_cuda_moe_layer_prefill": (C.c_int, [vp, u32, vp, u32, vp, vp, vp, vp, vp]),
    "nvmai_cuda_moe_ep_unique_id": (C.c_int, [vp]),
    "nvmai_cuda_moe_ep_init": (C.c_int, [vp, vp, u32, u32, u32]),
    "nvmai_cuda_moe_ep_shutdown": (C.c_int, [vp]),
    "nvmai_cuda_moe_ep_synchronize": (C.c_int, [vp, vp, u32]),
    "nvmai_cuda_moe_debug_host_delay": (C.c_int, [vp, vp, u32]),
    "nvmai_cuda_moe_debug_drop_prefill_copy": (C.c_int, [vp]),
    "nvmai_cuda_moe_ep_peer_export": (C.c_int, [vp, vp]),
    "nvmai_cuda_moe_ep_peer_attach": (C.c_int, [vp, vp]),
    "nvmai_cuda_moe_ep_stack_decode": (C.c_int, [vp, vp, u32, vp, vp]),
    "nvmai_cuda_moe_stack_decode": (C.c_int, [vp, vp, u32, vp, vp]),
    "nvmai_cuda_moe_stack_decode_host": (C.c_int, [vp, vp, u32, vp, vp]),
    "nvmai_cuda_moe_dequant": (C.c_int, [u32, u32, vp, vp, vp, u32, u32, vp, vp]),
    "nvmai_cuda_moe_affine_gemv": (C.c_int, [u32, u32, vp, vp, vp, vp, vp, u32, u32, vp]),
    "nvmai_cuda_moe_silu_mul_f16": (C.c_int, [vp, vp, vp, u32, vp]),
    "nvmai_cuda_moe_sigmoid_scalar_mul_f16": (C.c_int, [vp, vp, u32, vp]),
    "nvmai_cuda_moe_residual_add_f16": (C.c_int, [vp, vp, u32, vp]),
    "nvmai_cuda_moe_set_trace": (C.c_int, [vp, C.c_int]),
    "nvmai_cuda_moe_read_trace": (C.c_int, [vp, vp, u32]),
    "nvmai_cuda_moe_read_block_trace": (C.c_int, [vp, vp, u32, C.POINTER(u32)]),
    "nvmai_cuda_moe_synchronize": (C.c_int, [vp, vp]),
    "nvmai_cuda_moe_last_cuda_error": (C.c_int, [vp]),
    "nvmai_cuda_moe_error_string": (C.c_char_p, [C.c_int]),
    "nvmai_cuda_moe_read_file_to_device": (C.c_int, [C.c_char_p, C.c_uint64, C.c_uint64, vp, vp]),
    "nvmai_cuda_moe_launch_count": (u64, []),
    "nvmai_cuda_moe_set_decode_mode": (C.c_int, [vp, C.c_int]),
    "nvmai_cuda_moe_read_route_log": (C.c_int, [vp, vp, u32]),
    "nvmai_cuda_moe_read_route_log_rows": (C.c_int, [vp, vp, u32, u32]),
    "nvmai_cuda_moe_debug_set_wait_limit": (C.c_int, [u64]),
    "nvmai_cuda_moe_debug_mute_block": (C.c_int, [vp, u32]),
}


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: the CUDA library was not built "
                "(run `python -m nvmai_b200.build`); there is no CPU fallback")
        _lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(_lib, name)
            fn.restype = res
            fn.argtypes = args
    return _lib


class NvmaiError(RuntimeError):
    def __init__(self, code: int, where: str):
        self.code = code
        msg = lib().nvmai_cuda_moe_error_string(code).decode()
        super().__init__(f"{where}: {msg} (code {code})")


def check(code: int, where: str) -> None:
    if code != OK:
        raise NvmaiError(code, where)
