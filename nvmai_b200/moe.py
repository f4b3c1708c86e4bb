"""Thin ctypes wrapper over the C ABI, shaped like the reference's Swift kernel
wrappers (`MoE`, `SharedExpertRuntime`, `Elementwise`; sources/NVMAI/Kernels).

Device buffers are passed as anything with a `data_ptr()` (e.g. a CUDA torch
tensor) or as a raw integer address; this module allocates nothing on the device
itself.  Errors surface as `NvmaiError` carrying the library's error code.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

from . import _lib
from . import format as fmt
from ._lib import NvmaiError, check  # noqa: F401  (re-exported)


def _ptr(buf) -> int | None:
    if buf is None:
        return None
    if isinstance(buf, int):
        return buf
    return buf.data_ptr()


def _stream(stream) -> int | None:
    if stream is None:
        return None
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream        # torch.cuda.Stream


@dataclass
class MoEConfig:
    d: int = 2048
    f: int = 512
    shared_f: int = 512
    num_experts: int = 256
    top_k: int = 8
    routed_bits: int = 4
    shared_bits: int = 4
    router_kind: int = fmt.ROUTER_DENSE_F16
    shared_gate_kind: int = fmt.ROUTER_DENSE_F16
    meta_dtype: int = fmt.META_BF16
    activation: int = fmt.ACT_SILU
    out_dtype: int = fmt.OUT_FP16
    max_tokens: int = 1
    num_layers: int = 1

    def to_c(self) -> _lib.Config:
        return _lib.Config(self.d, self.f, self.shared_f, self.num_experts, self.top_k, self.routed_bits,
                           self.shared_bits, self.router_kind, self.shared_gate_kind, self.meta_dtype,
                           self.activation, self.out_dtype, self.max_tokens, self.num_layers)


def offsets_struct(off: dict[str, int]) -> _lib.ExpertOffsets:
    return _lib.ExpertOffsets(*[off[n] for n in fmt.OFFSET_NAMES])


def _tensor(t) -> _lib.AffineTensor:
    if t is None:
        return _lib.AffineTensor(None, None, None)
    w, s, b = t
    return _lib.AffineTensor(_ptr(w), _ptr(s), _ptr(b))


class MoE:
    """Counterpart of the reference's `MoE` + `SharedExpertRuntime` pair for one model."""

    def __init__(self, config: MoEConfig):
        self.config = config
        self._lib = _lib.lib()
        err = C.c_int(0)
        cfg = config.to_c()
        self._h = self._lib.nvmai_cuda_moe_create(C.byref(cfg), C.byref(err))
        if not self._h:
            raise NvmaiError(err.value, "nvmai_cuda_moe_create")
        self._keep = {}

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.nvmai_cuda_moe_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- weights ---------------------------------------------------------------
    def register_layer(self, layer: int, *, experts, expert_stride: int, offsets: dict[str, int], router,
                       effective_scale=None, per_expert_scale=None, shared=None, shared_gate=None) -> None:
        """router / shared[i] / shared_gate are (w, scales, biases) device buffers."""
        L = _lib.Layer()
        L.experts = _ptr(experts)
        L.expert_stride = expert_stride
        L.offsets = offsets_struct(offsets)
        L.router = _tensor(router)
        L.effective_scale = _ptr(effective_scale)
        L.per_expert_scale = _ptr(per_expert_scale)
        if shared is not None:
            L.shared_gate_proj, L.shared_up_proj, L.shared_down_proj = (_tensor(t) for t in shared)
        L.shared_gate = _tensor(shared_gate)
        self._keep[layer] = (experts, router, effective_scale, per_expert_scale, shared, shared_gate)
        check(self._lib.nvmai_cuda_moe_register_layer(self._h, layer, C.byref(L)), "register_layer")

    # -- reference-shaped entry points -------------------------------------------
    def encode_router(self, layer: int, x, out_idx, out_w, *, tokens: int = 1, x_stride: int | None = None,
                      stream=None) -> None:
        """`MoE.encodeRouter` (MoE.swift:151-213) / `PrefillRouter.encodeBlock`."""
        check(self._lib.nvmai_cuda_moe_router(self._h, layer, _ptr(x), x_stride or self.config.d, tokens,
                                              _ptr(out_idx), _ptr(out_w), _stream(stream)), "router")

    def encode_shared_expert(self, layer: int, x, h1, *, tokens: int = 1, x_stride: int | None = None,
                             stream=None) -> None:
        """`SharedExpertRuntime.encode` + scalar gate + sigmoid mul (RealForwardRunner.swift:3866-3905)."""
        check(self._lib.nvmai_cuda_moe_shared_expert(self._h, layer, _ptr(x), x_stride or self.config.d, tokens,
                                                     _ptr(h1), _stream(stream)), "shared_expert")

    def encode_routed_phase1(self, blobs, offsets: dict[str, int], x, acts, *, active_slots=None,
                             stream=None) -> None:
        """`encodeRoutedPersistentPhase1U16Load` / `…SubsetU16Load` (MoE.swift:295-392)."""
        arr = (C.c_void_p * len(blobs))(*[_ptr(b) for b in blobs])
        off = offsets_struct(offsets)
        slots, n = None, 0
        if active_slots is not None:
            n = len(active_slots)
            slots = (C.c_uint32 * max(n, 1))(*active_slots)
        check(self._lib.nvmai_cuda_moe_routed_phase1(self._h, arr, C.byref(off), _ptr(x), _ptr(acts), slots, n,
                                                     _stream(stream)), "routed_phase1")

    def encode_routed_phase2(self, blobs, offsets: dict[str, int], acts, routing_w, residual, y, *,
                             stream=None) -> None:
        """`encodeRoutedPersistentPhase2Reduce` (MoE.swift:394-440)."""
        arr = (C.c_void_p * len(blobs))(*[_ptr(b) for b in blobs])
        off = offsets_struct(offsets)
        check(self._lib.nvmai_cuda_moe_routed_phase2(self._h, arr, C.byref(off), _ptr(acts), _ptr(routing_w),
                                                     _ptr(residual), _ptr(y), _stream(stream)), "routed_phase2")

    def group_pairs(self, idx, w, tokens: int, sorted_pairs, expert_offsets, expert_counts, *, stream=None) -> None:
        """`makeTokenExpertPairs` + `groupTokenExpertPairs` (PrefillMoEGrouping.swift:90-192) on the device."""
        check(self._lib.nvmai_cuda_moe_group_pairs(self._h, _ptr(idx), _ptr(w), tokens, _ptr(sorted_pairs),
                                                   _ptr(expert_offsets), _ptr(expert_counts), _stream(stream)),
              "group_pairs")

    # -- expert parallelism --------------------------------------------------------------
    def set_expert_map(self, expert_map) -> None:
        """expert_map[e] = index of global expert e among this rank's blobs, or 0xFFFFFFFF."""
        if expert_map is None:
            check(self._lib.nvmai_cuda_moe_set_expert_map(self._h, None, 0), "set_expert_map")
            return
        arr = (C.c_uint32 * len(expert_map))(*[int(v) for v in expert_map])
        n_local = sum(1 for v in expert_map if int(v) != 0xFFFFFFFF)
        check(self._lib.nvmai_cuda_moe_set_expert_map(self._h, arr, n_local), "set_expert_map")

    def routed_partial(self, layer: int, x, tokens: int, idx, w, share, *, stream=None) -> None:
        check(self._lib.nvmai_cuda_moe_routed_partial(self._h, layer, _ptr(x), tokens, _ptr(idx), _ptr(w), _ptr(share),
                                                      _stream(stream)), "routed_partial")

    def ep_finalize(self, shares, ranks: int, h1, tokens: int, *, y=None, hidden=None, stream=None) -> None:
        check(self._lib.nvmai_cuda_moe_ep_finalize(self._h, _ptr(shares), ranks, _ptr(h1), tokens, _ptr(y), _ptr(hidden),
                                                   _stream(stream)), "ep_finalize")

    def layer_prefill(self, layer: int, x, tokens: int, *, hidden=None, y_out=None, out_idx=None, out_w=None,
                      stream=None) -> None:
        """The block for a prefill chunk (encodeRoutedMoEPrefill, RealForwardRunner.swift:3244-3591):
        x fp16 [tokens][d]; hidden updated in place with the prefill path's two-step residual;
        y_out = out(h1 + h2)."""
        check(self._lib.nvmai_cuda_moe_layer_prefill(self._h, layer, _ptr(x), tokens, _ptr(hidden), _ptr(y_out),
                                                     _ptr(out_idx), _ptr(out_w), _stream(stream)), "layer_prefill")

    def ep_unique_id(self) -> bytes:
        """The 128-byte id one rank makes and the launcher hands to every rank."""
        import ctypes
        buf = ctypes.create_string_buffer(128)
        check(self._lib.nvmai_cuda_moe_ep_unique_id(buf), "ep_unique_id")
        return buf.raw

    def ep_init(self, unique_id: bytes, rank: int, world: int, rows_own: int) -> None:
        """Collective over the ranks: opens the library's own communicator."""
        import ctypes
        if len(unique_id) != 128:
            raise ValueError("the communicator id is 128 bytes")
        buf = ctypes.create_string_buffer(unique_id, 128)
        check(self._lib.nvmai_cuda_moe_ep_init(self._h, buf, rank, world, rows_own), "ep_init")

    def ep_peer_export(self) -> bytes:
        """The 64-byte handle of this rank's receive area for the peer-memory exchange."""
        import ctypes
        buf = ctypes.create_string_buffer(64)
        check(self._lib.nvmai_cuda_moe_ep_peer_export(self._h, buf), "ep_peer_export")
        return buf.raw

    def ep_peer_attach(self, handles: list[bytes]) -> None:
        """handles: every rank's exported handle, in rank order."""
        import ctypes
        blob = b"".join(handles)
        buf = ctypes.create_string_buffer(blob, len(blob))
        check(self._lib.nvmai_cuda_moe_ep_peer_attach(self._h, buf), "ep_peer_attach")

    def ep_shutdown(self) -> None:
        check(self._lib.nvmai_cuda_moe_ep_shutdown(self._h), "ep_shutdown")

    def ep_synchronize(self, stream=None, timeout_ms: int = 0) -> None:
        """Host-polled wait of an expert-parallel rank: raises (and aborts the communicator) when NCCL reports an
        asynchronous error or the stream has not finished after `timeout_ms`."""
        check(self._lib.nvmai_cuda_moe_ep_synchronize(self._h, _stream(stream), int(timeout_ms)), "ep_synchronize")

    def debug_drop_prefill_copy(self) -> None:
        check(self._lib.nvmai_cuda_moe_debug_drop_prefill_copy(self._h), "debug_drop_prefill_copy")

    def debug_host_delay(self, ms: int, stream=None) -> None:
        check(self._lib.nvmai_cuda_moe_debug_host_delay(self._h, _stream(stream), int(ms)), "debug_host_delay")

    def ep_stack_decode(self, x_own, rows_own: int, y_own, *, stream=None) -> None:
        check(self._lib.nvmai_cuda_moe_ep_stack_decode(self._h, _ptr(x_own), rows_own, _ptr(y_own), _stream(stream)),
              "ep_stack_decode")

    def rms_renorm(self, y, tokens: int, x_out, *, stream=None) -> None:
        check(self._lib.nvmai_cuda_moe_rms_renorm(self._h, _ptr(y), tokens, _ptr(x_out), _stream(stream)), "rms_renorm")

    # -- fused paths ----------------------------------------------------------------
    def layer_decode(self, layer: int, x, tokens: int, *, hidden=None, h2_out=None, out_idx=None, out_w=None,
                     stream=None) -> None:
        check(self._lib.nvmai_cuda_moe_layer_decode(self._h, layer, _ptr(x), tokens, _ptr(hidden), _ptr(h2_out),
                                                    _ptr(out_idx), _ptr(out_w), _stream(stream)), "layer_decode")

    def layer_verify_pair(self, layer: int, x, *, hidden=None, h2_out=None, out_idx=None, out_w=None,
                          stream=None) -> None:
        """`encodeRoutedMoEVerifyPair` (RealForwardRunner.swift:3016-3235): the decode block for two rows."""
        check(self._lib.nvmai_cuda_moe_layer_verify_pair(self._h, layer, _ptr(x), _ptr(hidden), _ptr(h2_out),
                                                         _ptr(out_idx), _ptr(out_w), _stream(stream)),
              "layer_verify_pair")

    def layer_decode_prenorm(self, layer: int, hidden, norm_weight, eps: float, tokens: int, *, attn_delta=None,
                             h2_out=None, x_out=None, out_idx=None, out_w=None, stream=None) -> None:
        """Residual add + `rmsnorm_bf16w` + the decode block (RealForwardRunner.swift:1900-1909) in three launches."""
        check(self._lib.nvmai_cuda_moe_layer_decode_prenorm(self._h, layer, _ptr(hidden), _ptr(attn_delta),
                                                            _ptr(norm_weight), float(eps), tokens, _ptr(h2_out),
                                                            _ptr(x_out), _ptr(out_idx), _ptr(out_w), _stream(stream)),
              "layer_decode_prenorm")

    def layer_decode_fused_norms(self, layer: int, hidden, norm_weight, eps: float, tokens: int, next_norm_weight,
                                 next_eps: float, x_next, *, attn_delta=None, h2_out=None, x_out=None, out_idx=None,
                                 out_w=None, stream=None) -> None:
        """`layer_decode_prenorm` plus the next block's input norm of the hidden state it writes."""
        check(self._lib.nvmai_cuda_moe_layer_decode_fused_norms(self._h, layer, _ptr(hidden), _ptr(attn_delta),
                                                                _ptr(norm_weight), float(eps), tokens,
                                                                _ptr(next_norm_weight), float(next_eps), _ptr(x_next),
                                                                _ptr(h2_out), _ptr(x_out), _ptr(out_idx), _ptr(out_w),
                                                                _stream(stream)), "layer_decode_fused_norms")

    def stack_decode(self, x0, tokens: int, y_last, *, stream=None) -> None:
        check(self._lib.nvmai_cuda_moe_stack_decode(self._h, _ptr(x0), tokens, _ptr(y_last), _stream(stream)),
              "stack_decode")

    def stack_decode_host(self, x0_host: int, tokens: int, y_last_host: int, *, stream=None) -> None:
        """x0_host / y_last_host are HOST addresses (e.g. pinned numpy / torch CPU buffers)."""
        check(self._lib.nvmai_cuda_moe_stack_decode_host(self._h, _ptr(x0_host), tokens, _ptr(y_last_host),
                                                         _stream(stream)), "stack_decode_host")

    DECODE_AUTO, DECODE_STAGED, DECODE_RESIDENT = 0, 1, 2

    def set_decode_mode(self, mode: int) -> None:
        """How a single-token stack step runs: one resident kernel (auto / forced) or the staged launches."""
        check(self._lib.nvmai_cuda_moe_set_decode_mode(self._h, int(mode)), "set_decode_mode")

    def debug_mute_block(self, block: int = 0xFFFFFFFF) -> None:
        """Test hook: one block of the resident kernel withholds its phase-1 results (bounded waits then expire)."""
        check(self._lib.nvmai_cuda_moe_debug_mute_block(self._h, block & 0xFFFFFFFF), "debug_mute_block")

    def read_route_log(self, layers: int | None = None):
        """-> uint32 [layers, top_k]: the experts each layer of the last resident-kernel step selected."""
        import numpy as np
        n = self.config.num_layers if layers is None else layers
        out = np.zeros((n, self.config.top_k), dtype=np.uint32)
        check(self._lib.nvmai_cuda_moe_read_route_log(self._h, out.ctypes.data, n), "read_route_log")
        return out

    def read_route_log_rows(self, rows: int, layers: int | None = None):
        """-> uint32 [layers, rows, top_k] after a resident-kernel step of `rows` rows (2..8, or all ranks' rows)."""
        import numpy as np
        n = self.config.num_layers if layers is None else layers
        out = np.zeros((n, rows, self.config.top_k), dtype=np.uint32)
        check(self._lib.nvmai_cuda_moe_read_route_log_rows(self._h, out.ctypes.data, n, rows), "read_route_log_rows")
        return out

    def set_trace(self, enable: bool) -> None:
        check(self._lib.nvmai_cuda_moe_set_trace(self._h, int(enable)), "set_trace")

    # what the three staged launches of a layer do, in the reference's role names (recordKernelGPU(role:),
    # RealForwardRunner.swift:3839-3844)
    TRACE_STAGE_ROLES = ("attn_tail_router + shared_expert (router logits, shared gate/up, gate row)",
                         "moe_phase1_hit (routed gate/up + activation)",
                         "moe_phase1_2_routed tail (routed down, weighted sum, shared down, gate)")

    def read_trace(self, layers: int | None = None):
        """-> uint64 array [layers, 3, 8]: {start, end, six phase marks of block 0} GPU-timer ns per stage launch
        (the stages are TRACE_STAGE_ROLES)."""
        import numpy as np
        n = self.config.num_layers if layers is None else layers
        out = np.zeros((n, 3, 8), dtype=np.uint64)
        check(self._lib.nvmai_cuda_moe_read_trace(self._h, out.ctypes.data, n), "read_trace")
        return out

    def read_block_trace(self, layers: int | None = None):
        """-> uint64 [layers, blocks, 16]: the resident kernel's per-block phase marks (GPU-timer ns, 0 = none)."""
        import numpy as np
        n = self.config.num_layers if layers is None else layers
        blocks = C.c_uint32(0)
        check(self._lib.nvmai_cuda_moe_read_block_trace(self._h, None, n, C.byref(blocks)), "read_block_trace")
        out = np.zeros((n, blocks.value, 16), dtype=np.uint64)
        check(self._lib.nvmai_cuda_moe_read_block_trace(self._h, out.ctypes.data, n, C.byref(blocks)), "read_block_trace")
        return out

    def synchronize(self, stream=None) -> None:
        check(self._lib.nvmai_cuda_moe_synchronize(self._h, _stream(stream)), "synchronize")


# -- handle-free helpers ---------------------------------------------------------------

def dequant(bits: int, meta: int, w, scales, biases, rows: int, n: int, out_f32, stream=None) -> None:
    check(_lib.lib().nvmai_cuda_moe_dequant(bits, meta, _ptr(w), _ptr(scales), _ptr(biases), rows, n,
                                            _ptr(out_f32), _stream(stream)), "dequant")


def affine_gemv(bits: int, meta: int, w, scales, biases, x, y, m: int, n: int, stream=None) -> None:
    """`DequantInt4GEMV.encode` / `DequantInt8GEMV.encode`."""
    check(_lib.lib().nvmai_cuda_moe_affine_gemv(bits, meta, _ptr(w), _ptr(scales), _ptr(biases), _ptr(x), _ptr(y),
                                                m, n, _stream(stream)), "affine_gemv")


NOALLOC_MAX_TOKENS = 64


def router_noalloc(config: MoEConfig, router, x, out_idx, out_w, *, tokens: int = 1, x_stride: int | None = None,
                   effective_scale=None, per_expert_scale=None, stream=None) -> None:
    """Router for callers that must not allocate device memory (no handle; the
    scratch is a fixed array inside the library, at most NOALLOC_MAX_TOKENS rows).
    Calls that overlap on the GPU race on that array: keep them ordered."""
    cfg = config.to_c()
    t = _tensor(router)
    check(_lib.lib().nvmai_cuda_moe_router_noalloc(C.byref(cfg), C.byref(t), _ptr(effective_scale),
                                                   _ptr(per_expert_scale), _ptr(x), x_stride or config.d, tokens,
                                                   _ptr(out_idx), _ptr(out_w), _stream(stream)), "router_noalloc")


def router_noalloc_status(stream=None) -> None:
    """Waits for `stream`; raises NvmaiError(ETIMEOUT) if the last allocation-free router call gave up a wait."""
    check(_lib.lib().nvmai_cuda_moe_router_noalloc_status(_stream(stream)), "router_noalloc_status")


class Elementwise:
    """`Elementwise` (sources/NVMAI/Kernels/Primitives/Elementwise.swift), the three MoE-side kernels."""

    @staticmethod
    def encode_silu_mul(gate, up, out, count: int, stream=None) -> None:
        check(_lib.lib().nvmai_cuda_moe_silu_mul_f16(_ptr(gate), _ptr(up), _ptr(out), count, _stream(stream)),
              "silu_mul")

    @staticmethod
    def encode_sigmoid_scalar_mul(y, gate, count: int, stream=None) -> None:
        check(_lib.lib().nvmai_cuda_moe_sigmoid_scalar_mul_f16(_ptr(y), _ptr(gate), count, _stream(stream)),
              "sigmoid_scalar_mul")

    @staticmethod
    def encode_residual_add(hidden, delta, count: int, stream=None) -> None:
        check(_lib.lib().nvmai_cuda_moe_residual_add_f16(_ptr(hidden), _ptr(delta), count, _stream(stream)),
              "residual_add")


def debug_set_wait_limit(nanoseconds: int) -> None:
    """Test hook: the longest any device-side wait lasts (0 = the default of one second)."""
    check(_lib.lib().nvmai_cuda_moe_debug_set_wait_limit(int(nanoseconds)), "debug_set_wait_limit")


def launch_count() -> int:
    return int(_lib.lib().nvmai_cuda_moe_launch_count())
