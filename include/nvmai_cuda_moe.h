/*
 * libnvmai_cuda_moe — CUDA (sm_100a) implementation of NVMAI's routed-expert
 * MoE FFN on NVMAIRepack quantized weights, behind a C ABI in the style of the
 * reference's NVMAIKernelsC target (sources/NVMAIKernelsC/include/nvmai_kernels.h,
 * nvmai_expert_io.h): C99 types only, `nvmai_` prefix, opaque handle with
 * create/destroy, work functions return 0 or an error code and leave outputs
 * undefined on failure.
 *
 * Every work function ENQUEUES on the caller's CUDA stream (`stream` is a
 * cudaStream_t passed as void*, NULL = the legacy default stream) and returns;
 * this is the CUDA counterpart of the reference's `encode…(commandBuffer:)`
 * methods.  All data pointers are DEVICE pointers unless the parameter name ends
 * in `_host`.  A handle is single-owner and not thread-safe, like the
 * reference's runner (sources/NVMAI/Runtime/Inference/RealForwardRunner.swift:128-134).
 *
 * Weight bytes are consumed exactly as NVMAIRepack wrote them: U32-packed
 * codes, LSB first (code i of a row at bit i*bits), one 16-bit scale and one
 * 16-bit bias per group of 64 inputs, w = q*scale + bias.  The library never
 * copies or re-lays-out weights.  Tensor base addresses must be 16-byte aligned
 * (routed expert blobs are 16 KiB aligned by construction,
 * sources/NVMAIRepack/Core/Planning/RepackPlanner.swift:428).
 */
#ifndef NVMAI_CUDA_MOE_H
#define NVMAI_CUDA_MOE_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define NVMAI_API __attribute__((visibility("default")))
#else
#define NVMAI_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- error codes (0 = success; errno-style like nvmai_expert_io.h:46-55) ---- */
#define NVMAI_CUDA_OK 0
#define NVMAI_CUDA_EINVAL 22    /* bad shape, null pointer, misaligned tensor */
#define NVMAI_CUDA_ERANGE 34    /* index / size outside the configured limits */
#define NVMAI_CUDA_ENOMEM 12    /* device allocation failed */
#define NVMAI_CUDA_ECUDA 1001   /* CUDA runtime error; see nvmai_cuda_moe_last_cuda_error */
#define NVMAI_CUDA_ETIMEOUT 1002 /* a bounded device-side wait expired */
#define NVMAI_CUDA_ENCCL 1003
#define NVMAI_CUDA_EIO 5        /* a weight file could not be opened or is shorter than the requested range */

/* ---- enums ---- */
#define NVMAI_META_BF16 0u   /* the reference's format (RepackPlanner.swift:302-305) */
#define NVMAI_META_FP16 1u
#define NVMAI_ACT_SILU 0u        /* moe.metal:134-139, FC_MOE_ACT_SILU = true (Qwen SwiGLU) */
#define NVMAI_ACT_GELU_TANH 1u   /* moe.metal:82-89, the `MoE(context:)` default */
#define NVMAI_OUT_FP16 0u    /* reference rounding points (moe.metal:808, utility.metal:102) */
#define NVMAI_OUT_FP32 1u    /* h1 / h2 / hidden kept in fp32 (no fp16 overflow on wide-range weights) */
#define NVMAI_ROUTER_DENSE_F16 0u  /* [E][D] fp16 gate matrix */
#define NVMAI_ROUTER_AFFINE4 4u    /* affine codes + 16-bit scale/bias per 64 (moe.metal:157-214) */
#define NVMAI_ROUTER_AFFINE8 8u
#define NVMAI_GATE_NONE 0xFFFFFFFFu /* shared expert without a sigmoid gate */

typedef struct nvmai_cuda_moe nvmai_cuda_moe;

/* Mirrors the arguments of `MoE.init` (sources/NVMAI/Kernels/MoE/MoE.swift:60-149)
 * plus the scratch the runner allocates around it (RealForwardRunner.swift:503-511). */
typedef struct {
    uint32_t d;              /* hidden size, multiple of 64 */
    uint32_t f;              /* routed expert intermediate size, multiple of 64 */
    uint32_t shared_f;       /* shared expert intermediate size (0 = no shared expert) */
    uint32_t num_experts;    /* <= 256 (MoE.swift:164) */
    uint32_t top_k;          /* decode entry points need 8 (MoE.swift:165); prefill router <= 64 */
    uint32_t routed_bits;    /* 4 or 8 */
    uint32_t shared_bits;    /* 4 or 8 */
    uint32_t router_kind;    /* NVMAI_ROUTER_* */
    uint32_t shared_gate_kind; /* NVMAI_ROUTER_* encoding of the [1][D] gate row, or NVMAI_GATE_NONE */
    uint32_t meta_dtype;     /* NVMAI_META_* */
    uint32_t activation;     /* NVMAI_ACT_* */
    uint32_t out_dtype;      /* NVMAI_OUT_* : element type of h1, y and hidden */
    uint32_t max_tokens;     /* largest token count of one call (decode batch or prefill chunk) */
    uint32_t num_layers;     /* layers that may be registered */
} nvmai_cuda_moe_config;

/* Mirrors `MoEExpertOffsets` (MoE.swift:4-29) == `ExpertOffsets` (moe.metal:141-151): 9 x u32. */
typedef struct {
    uint32_t gate_w, gate_s, gate_b, up_w, up_s, up_b, down_w, down_s, down_b;
} nvmai_expert_offsets;

/* One affine (or dense) matrix: W | scales | biases as three device pointers,
 * like `SharedExpertProjection` (SharedExpertInt4.swift:125-152). */
typedef struct {
    const void *w;
    const void *scales;  /* NULL for a dense fp16 matrix */
    const void *biases;
} nvmai_affine_tensor;

/* Per-layer weight views: `Model.routedExpertOffsets` + the runner's per-layer
 * shared-expert projections (ModelExpertIO.swift:67-82, RealForwardRunner.swift:587-610).
 * `experts` and `expert_stride` must be 16-byte aligned (the blobs are never copied).  The
 * other tensors may start at any even address, as they do in the reference's weight file
 * (RepackPlanner.swift:310-316; DequantInt4GEMVTests.swift:114-121 tests a base off by two
 * bytes): register_layer copies a tensor whose base is not 16-byte aligned into an aligned
 * buffer of its own, once, and uses that. */
typedef struct {
    const void *experts;         /* num_experts blobs, expert_stride bytes apart */
    uint64_t expert_stride;
    nvmai_expert_offsets offsets;
    nvmai_affine_tensor router;  /* [E][D] */
    const void *effective_scale;   /* bf16[D] or NULL (= 1.0, RealForwardRunner.swift:612-632) */
    const void *per_expert_scale;  /* bf16[E] or NULL (= 1.0) */
    nvmai_affine_tensor shared_gate_proj, shared_up_proj, shared_down_proj; /* [Fs][D],[Fs][D],[D][Fs] */
    nvmai_affine_tensor shared_gate;  /* [1][D] scalar-gate row (RealForwardRunner.swift:3884-3896) */
} nvmai_cuda_moe_layer;

/* Expert-blob byte offsets for (d, f, bits): `CPUExpertFFN.Offsets.init`
 * (sources/NVMAI/Kernels/CPU/CPUExpertFFN.swift:42-59) generalised to 8-bit.
 * Returns the expert stride in bytes (1,769,472 for 2048/512/4-bit). */
NVMAI_API uint64_t nvmai_cuda_moe_expert_offsets(uint32_t d, uint32_t f, uint32_t bits, nvmai_expert_offsets *out);

/* `MoE.init` (MoE.swift:60-149): validates the shape, allocates device scratch.
 * NULL on failure with *out_err set (nvmai_expert_reader_create convention,
 * nvmai_expert_io.h:20-44). */
NVMAI_API nvmai_cuda_moe *nvmai_cuda_moe_create(const nvmai_cuda_moe_config *config, int *out_err);
NVMAI_API void nvmai_cuda_moe_destroy(nvmai_cuda_moe *h);

/* Records the layer's device views (ModelExpertIO.swift:67-82). */
NVMAI_API int nvmai_cuda_moe_register_layer(nvmai_cuda_moe *h, uint32_t layer, const nvmai_cuda_moe_layer *weights);

/* `MoE.encodeRouter` (MoE.swift:151-213) = router_gemv_r4 + router_topk_select_k8
 * (moe.metal:174-285) for `tokens` rows of x (row stride x_stride elements;
 * tokens = 1 is the reference's decode call, tokens > 1 is
 * `PrefillRouter.encodeBlock`, PrefillRouter.swift:41-95).
 * out_idx u32[tokens][top_k], out_w fp16[tokens][top_k]. */
NVMAI_API int nvmai_cuda_moe_router(nvmai_cuda_moe *h, uint32_t layer, const void *x_f16, uint32_t x_stride,
                          uint32_t tokens, uint32_t *out_idx, void *out_w_f16, void *stream);

/* The same router for callers that cannot allocate device memory.  It has no
 * counterpart in the reference.  Meant for hosts that gave all of HBM to their own
 * arena before the first token (resident experts, KV state), where a cudaMalloc at
 * this point can fail, and for decode loops that cannot afford the device-wide
 * serialisation of cudaMalloc / cudaFree.  No handle: the logits and block
 * counters live in a fixed 64.5 KiB array inside the library image (every GPU that
 * loads the library holds it until the process exits), so the batch is limited to
 * NVMAI_CUDA_NOALLOC_MAX_TOKENS rows; more returns NVMAI_CUDA_ERANGE.  `config`
 * supplies d, num_experts, top_k, router_kind, meta_dtype; `router`,
 * `effective_scale`, `per_expert_scale` as in nvmai_cuda_moe_layer.  The call
 * makes no cudaMalloc / cudaFree and calls no allocating routine; it clears the
 * counters with a memset on `stream` and launches one kernel.  The first call on
 * a device looks up the array's device address (cudaGetSymbolAddress with that
 * device current) and should therefore happen before any stream capture.  All
 * calls share the one array: two calls that overlap on the GPU (different
 * streams, no ordering) race on it; order them.  Results are bit-identical to
 * nvmai_cuda_moe_router. */
#define NVMAI_CUDA_NOALLOC_MAX_TOKENS 64u
NVMAI_API int nvmai_cuda_moe_router_noalloc(const nvmai_cuda_moe_config *config, const nvmai_affine_tensor *router,
                                  const void *effective_scale, const void *per_expert_scale, const void *x_f16,
                                  uint32_t x_stride, uint32_t tokens, uint32_t *out_idx, void *out_w_f16,
                                  void *stream);

/* Completion check for nvmai_cuda_moe_router_noalloc (there is no handle whose synchronize
 * could report it; no counterpart in the reference): waits for `stream`, then returns
 * NVMAI_CUDA_ETIMEOUT if the last allocation-free router call on the current device gave
 * up a bounded device-side wait (its out_idx / out_w are then unwritten), else 0.  Copies
 * four bytes back; allocates nothing. */
NVMAI_API int nvmai_cuda_moe_router_noalloc_status(void *stream);

/* `SharedExpertRuntime.encode` + scalar gate GEMV + `sigmoid_scalar_mul_fp16`
 * (RealForwardRunner.swift:3866-3905): h1 = sigmoid(g.x) * down(act(gate.x)*up.x).
 * h1 is out_dtype[tokens][d]. */
NVMAI_API int nvmai_cuda_moe_shared_expert(nvmai_cuda_moe *h, uint32_t layer, const void *x_f16, uint32_t x_stride,
                                 uint32_t tokens, void *h1, void *stream);

/* `MoE.encodeRoutedPersistentPhase1U16Load` / `…Phase1SubsetU16Load`
 * (MoE.swift:295-392; moe.metal:642-727, 812-861):
 * acts[slot*f + j] = half(act(gate_slot[j].x) * (up_slot[j].x)) for the 8 blobs
 * in `blobs_host` (host array of 8 device pointers, the argument-buffer of
 * MoE.swift:215-227).  active_slots_host NULL = all slots.  The acts buffer holds
 * fp16 values with out_dtype = NVMAI_OUT_FP16 and fp32 values rounded to 11
 * significant bits with NVMAI_OUT_FP32 (top_k * f elements either way); phase 2
 * reads the same type. */
NVMAI_API int nvmai_cuda_moe_routed_phase1(nvmai_cuda_moe *h, const void *const *blobs_host,
                                 const nvmai_expert_offsets *offsets, const void *x_f16, void *acts_f16,
                                 const uint32_t *active_slots_host, uint32_t active_count, void *stream);

/* `MoE.encodeRoutedPersistentPhase2Reduce` (MoE.swift:394-440; moe.metal:769-810, 863-892):
 * y[i] = out(residual[i] + sum_{k=0..7} float(w[k]) * (down_k[i,:].acts_k)), partials added in slot order. */
NVMAI_API int nvmai_cuda_moe_routed_phase2(nvmai_cuda_moe *h, const void *const *blobs_host,
                                 const nvmai_expert_offsets *offsets, const void *acts_f16,
                                 const void *routing_w_f16, const void *residual, void *y, void *stream);

/* The whole MoE block of a decode step for `tokens` independent rows
 * (RealForwardRunner.swift:1911-1995, 3866-3905, 3914-4312):
 * router -> shared expert -> phase 1 -> phase 2 (h1 as residual) -> hidden += h2.
 * x is the normalised input fp16[tokens][d]; hidden_inout out_dtype[tokens][d] may be
 * NULL; h2_out (optional) receives the block output before the residual add.
 * out_idx / out_w optional.  Experts stay on the device: no host read-back. */
NVMAI_API int nvmai_cuda_moe_layer_decode(nvmai_cuda_moe *h, uint32_t layer, const void *x_f16, uint32_t tokens,
                                void *hidden_inout, void *h2_out, uint32_t *out_idx, void *out_w_f16,
                                void *stream);

/* Width-2 verification of a speculated token (`encodeRoutedMoEVerifyPair`,
 * RealForwardRunner.swift:3016-3235): the decode block, in the decode rounding order,
 * for exactly two rows x fp16[2][d]; hidden_inout / h2_out / out_idx / out_w as in
 * _layer_decode with tokens = 2.  The reference encodes phase 1 and phase 2 once per
 * row and fetches the union of the two rows' experts; here both rows share one launch
 * of each stage and a blob that both rows selected crosses HBM once. */
NVMAI_API int nvmai_cuda_moe_layer_verify_pair(nvmai_cuda_moe *h, uint32_t layer, const void *x_f16, void *hidden_inout,
                                               void *h2_out, uint32_t *out_idx, void *out_w_f16, void *stream);

/* The decode block with the two steps the runner encodes in front of it folded in
 * (RealForwardRunner.swift:1900-1909; residual_add_fp16, utility.metal:94-103;
 * rmsnorm_bf16w, rmsnorm.metal:69-99):
 *   hidden' = out(hidden + attn_delta)              (attn_delta fp16[tokens][d], NULL = no add)
 *   x       = half(hidden' * rsqrt(mean(hidden'^2) + eps) * w)   (w bf16[d])
 *   hidden  = out(hidden' + h2(x))
 * hidden_inout is out_dtype[tokens][d] and is written once, by the last stage.
 * x_out_f16 (optional, fp16[tokens][d]) receives the normalised rows (`routedX`);
 * h2_out / out_idx / out_w as in _layer_decode.  Saves the two elementwise launches and
 * their 4 KB round trips per row. */
NVMAI_API int nvmai_cuda_moe_layer_decode_prenorm(nvmai_cuda_moe *h, uint32_t layer, void *hidden_inout,
                                                  const void *attn_delta_f16, const void *norm_weight_bf16, float eps,
                                                  uint32_t tokens, void *h2_out, void *x_out_f16, uint32_t *out_idx,
                                                  void *out_w_f16, void *stream);

/* The same block with the step AFTER it folded in too: the layer that follows starts with
 * rmsnorm_bf16w of the hidden state this block has just written (RealForwardRunner.swift:1886-1899,
 * rmsnorm.metal:69-99), so the stage that writes hidden also writes
 *   x_next = half(hidden * rsqrt(mean(hidden^2) + next_eps) * next_w)      (next_w bf16[d])
 * to x_next_out_f16 (fp16[tokens][d]).  Single rows: the down-stage block that completes a row
 * normalises it; batched rows: the combine block of the row.  Everything else as in
 * _layer_decode_prenorm, with bit-identical results. */
NVMAI_API int nvmai_cuda_moe_layer_decode_fused_norms(nvmai_cuda_moe *h, uint32_t layer, void *hidden_inout,
                                                      const void *attn_delta_f16, const void *norm_weight_bf16, float eps,
                                                      uint32_t tokens, const void *next_norm_weight_bf16, float next_eps,
                                                      void *x_next_out_f16, void *h2_out, void *x_out_f16,
                                                      uint32_t *out_idx, void *out_w_f16, void *stream);

/* `PrefillRouter.makeTokenExpertPairs` + `PrefillMoEGrouping.groupTokenExpertPairs`
 * (PrefillRouter.swift:97-117, PrefillMoEGrouping.swift:90-192) on the device: the
 * tokens*top_k (token, expert, rank, weight) records sorted by (expert, token,
 * rank), 16 bytes each with fields at 0/4/8/12 like `PrefillTokenExpertPair`;
 * expert_offsets[e] = first sorted position (0xFFFFFFFF when e has no pair),
 * expert_counts[e] = its number of pairs.  idx / w as written by the router. */
NVMAI_API int nvmai_cuda_moe_group_pairs(nvmai_cuda_moe *h, const uint32_t *idx, const void *w_f16, uint32_t tokens,
                               void *sorted_pairs, uint32_t *expert_offsets, uint32_t *expert_counts, void *stream);

/* Reads `bytes` bytes at `file_offset` of a weight file (a `packed_experts/layer_NN.bin`
 * of a .gturbo artifact, GTurboPackedExpertsLayoutV1.swift:185-196) into device memory:
 * positioned reads into two pinned staging buffers that alternate with asynchronous
 * copies on `stream`, so the file read of one piece overlaps the copy of the one before.
 * Replaces the slot-cache reader of the reference (expert_io.c, ExpertStreamer) for a
 * host that keeps every expert resident.  Returns after the last copy is enqueued and
 * the staging buffers are released (the call synchronises the stream once at its end).
 * NVMAI_CUDA_EIO: cannot open, or the file ends before file_offset + bytes. */
NVMAI_API int nvmai_cuda_moe_read_file_to_device(const char *path, uint64_t file_offset, uint64_t bytes,
                                                 void *device_dst, void *stream);

/* ---- expert parallelism (no counterpart in the reference, which runs on one GPU) ----
 * A rank holds n_local of the layer's expert blobs, contiguous at `experts` in
 * local-index order; map_host[e] = local index of global expert e or 0xFFFFFFFF.
 * The map is validated: every local index below n_local is named by exactly one expert
 * (NVMAI_CUDA_EINVAL for a duplicate or a gap, NVMAI_CUDA_ERANGE for an index >= n_local).
 * NULL resets. */
NVMAI_API int nvmai_cuda_moe_set_expert_map(nvmai_cuda_moe *h, const uint32_t *map_host, uint32_t n_local);

/* This rank's share of the routed experts for `tokens` rows that every rank holds:
 * share[t] = sum over the token's (expert, weight) pairs whose expert is local of
 * float(w) * down_e(act(gate_e.x) * up_e.x), fp32 rows [tokens][d]; idx / w as the
 * router wrote them (global expert ids).  Rows of a token with no local expert are
 * zero.  The shared expert and the residual are the token owner's business. */
NVMAI_API int nvmai_cuda_moe_routed_partial(nvmai_cuda_moe *h, uint32_t layer, const void *x_f16, uint32_t tokens,
                                  const uint32_t *idx, const void *w_f16, float *share_f32, void *stream);

/* Owner side: y = out(h1 + sum_r shares[r]) with the ranks' shares added in rank
 * order (bitwise reproducible), hidden += y.  shares fp32 [ranks][tokens][d]. */
NVMAI_API int nvmai_cuda_moe_ep_finalize(nvmai_cuda_moe *h, const float *shares_f32, uint32_t ranks, const void *h1,
                               uint32_t tokens, void *y, void *hidden_inout, void *stream);

/* x = half(y * rsqrt(mean(y^2) + 1e-6)) per row: the stand-in for the attention +
 * rmsnorm between two MoE blocks that the stack benchmark uses. */
NVMAI_API int nvmai_cuda_moe_rms_renorm(nvmai_cuda_moe *h, const void *y, uint32_t tokens, void *x_f16_out, void *stream);

/* The whole MoE block for a prefill chunk (RealForwardRunner.swift:3244-3591:
 * PrefillRouter.encodeBlock, pair grouping, prefill_grouped_routed_moe_batched_phase1 /
 * _down, prefill_moe_reduce_token_major, PrefillSharedExpert.encodeBlock, the tail at
 * :3560-3569) as grouped GEMMs on the tensor cores: x fp16 [tokens][d] (dense rows),
 * hidden_inout = out(out(hidden + h1) + h2) in place, y_out (optional) = out(h1 + h2),
 * out_idx / out_w (optional) the routing.  The tensor cores multiply the centred weight
 * s*(q - 8) in fp16 (exact for bf16 scales; an 8-bit code goes through as its two nibbles,
 * 16 s*(hq - 8) and s*(lq - 8), in two passes over the same token rows) and the per-group
 * constant b + c*s enters through correction columns, so results stay within 1e-3 of the
 * CPU path for both bit widths.  Shapes the tiles do not cover (f % 128, d % 256 or
 * shared_f % 128 non-zero: the reference's own prefill test runs d = f = 64) and
 * NVMAI_CUDA_PREFILL_TC=0 in the environment run the exact grouped kernels of the batched
 * decode path with the same rounding points. */
NVMAI_API int nvmai_cuda_moe_layer_prefill(nvmai_cuda_moe *h, uint32_t layer, const void *x_f16, uint32_t tokens,
                                           void *hidden_inout, void *y_out, uint32_t *out_idx, void *out_w_f16,
                                           void *stream);

/* Expert parallelism with the exchange inside the library (no counterpart in the
 * reference, which runs on one GPU): the library opens its own NCCL communicator
 * (libnccl.so.2, resolved at run time; NVMAI_CUDA_ENCCL when it is missing or a call
 * fails).  One rank obtains an id, the host's launcher hands the 128 bytes to every
 * rank, and every rank calls ep_init (collective, blocking) after set_expert_map and
 * before ep_stack_decode.  world * rows_own must fit max_tokens. */
#define NVMAI_CUDA_EP_ID_BYTES 128
NVMAI_API int nvmai_cuda_moe_ep_unique_id(void *id_out_host);
NVMAI_API int nvmai_cuda_moe_ep_init(nvmai_cuda_moe *h, const void *id_host, uint32_t rank, uint32_t world,
                                     uint32_t rows_own);
NVMAI_API int nvmai_cuda_moe_ep_shutdown(nvmai_cuda_moe *h);

/* Waits for `stream` as a rank of an expert-parallel job has to: a collective whose peer is
 * gone never ends, so this polls the stream and the communicator's asynchronous error state
 * (ncclCommGetAsyncError) from the host instead of blocking in the driver.  When NCCL
 * reports an error (NVMAI_CUDA_ENCCL), or `timeout_ms` (0 = no limit) passes without the
 * stream finishing (NVMAI_CUDA_ETIMEOUT), the communicator is aborted (ncclCommAbort ends
 * its kernels in flight), the handle's expert-parallel state is dropped as by ep_shutdown,
 * and the step's outputs are undefined; ep_init opens a new communicator.  Otherwise the
 * result is that of nvmai_cuda_moe_synchronize.  NVMAI_CUDA_NCCL_LIB in the environment
 * names the NCCL library to load instead of libnccl.so.2. */
NVMAI_API int nvmai_cuda_moe_ep_synchronize(nvmai_cuda_moe *h, void *stream, uint32_t timeout_ms);

/* Optional, after ep_init: exchange the ranks' shares through peer memory instead of NCCL
 * (small batches, where every rank keeps all rows).  Every rank exports the handle of its
 * receive area (a CUDA IPC handle, 64 bytes), the launcher collects the handles of all
 * ranks in rank order and gives the array to every rank's attach.  Afterwards the down
 * stage stores its share rows straight into every rank's receive area over NVLink (plain
 * peer stores, no multicast) and the sum waits, with a bounded wait, for the per-layer
 * arrival counter; one process per GPU on one node.  Every rank must attach (or none). */
#define NVMAI_CUDA_EP_PEER_HANDLE_BYTES 64
NVMAI_API int nvmai_cuda_moe_ep_peer_export(nvmai_cuda_moe *h, void *handle_out_host);
NVMAI_API int nvmai_cuda_moe_ep_peer_attach(nvmai_cuda_moe *h, const void *handles_host);

/* The FFN-only stack of the benchmark, sharded by experts: this rank's rows in
 * (fp16 [rows_own][d]), the last layer's block output for them out (out_dtype).
 * Per layer: shared expert on the own rows, all-gather of the rows, router on all
 * rows, local experts' shares, all-to-all of the shares to the rows' owners, rank-
 * ordered sum + shared expert, RMS renormalisation.  Every rank must call it with the
 * same rows_own, the same number of times.  The first call per (x, y, rows, stream)
 * issues plain launches, the second captures a CUDA graph, later ones replay it.
 * With the peers attached (ep_peer_attach) and at most 8 rows in total, a step is ONE
 * launch of the resident kernel per rank and nothing else: the rows are gathered and the
 * shares exchanged by tagged peer stores over NVLink from inside that kernel (no
 * collective call); every rank keeps all rows.  A peer that stops makes the kernel's
 * bounded wait run out (NVMAI_CUDA_ETIMEOUT from the synchronize calls); the ranks then
 * call ep_init again before the next step, since their step counters may differ. */
NVMAI_API int nvmai_cuda_moe_ep_stack_decode(nvmai_cuda_moe *h, const void *x_own_f16, uint32_t rows_own, void *y_own,
                                             void *stream);

/* Benchmark driver for an FFN-only stack: runs layers 0..num_layers-1 on one
 * token batch; between layers the block output is renormalised to unit RMS in
 * fp32 and rounded to fp16 (a stand-in for the attention + rmsnorm the real model
 * runs there, RealForwardRunner.swift:1900-1909).  x0 fp16[tokens][d];
 * y_last out_dtype[tokens][d] = last layer's block output. */
NVMAI_API int nvmai_cuda_moe_stack_decode(nvmai_cuda_moe *h, const void *x0_f16, uint32_t tokens, void *y_last,
                                void *stream);

/* How a single-token nvmai_cuda_moe_stack_decode step runs (no counterpart in the
 * reference, whose command buffers are its only launch unit):
 *   0  (default) one resident kernel for the whole step when the shape allows it
 *      (top_k <= 8, shared_bits == routed_bits, d <= 16 * SM count, f and shared_f <= 1024,
 *      no expert map, stream not under capture), the staged kernels otherwise;
 *   1  always the staged kernels (three launches per layer, replayed as a CUDA graph);
 *   2  the resident kernel, or NVMAI_CUDA_EINVAL when the shape does not allow it.
 * Both paths give bit-identical results.  NVMAI_CUDA_DECODE_MODE in the environment sets
 * the initial value. */
NVMAI_API int nvmai_cuda_moe_set_decode_mode(nvmai_cuda_moe *h, int mode);

/* The experts every layer of the last resident-kernel step selected, u32 [layers][top_k] in
 * rank order: the data of the reference's NVMAI_ROUTE_TRACE lines
 * (RealForwardRunner.swift:1208-1237).  Synchronises the device. */
NVMAI_API int nvmai_cuda_moe_read_route_log(nvmai_cuda_moe *h, uint32_t *out_host, uint32_t layers);

/* The same after a step of several rows (2..8 rows through the resident kernel, or an
 * expert-parallel step, where the rows are those of all ranks): u32 [layers][rows][top_k].
 * `rows` must be the row count of that step. */
NVMAI_API int nvmai_cuda_moe_read_route_log_rows(nvmai_cuda_moe *h, uint32_t *out_host, uint32_t layers, uint32_t rows);

/* Test hook: the longest any device-side wait of this library lasts, in nanoseconds
 * (0 restores the default of one second).  Process-wide, per device. */
NVMAI_API int nvmai_cuda_moe_debug_set_wait_limit(uint64_t nanoseconds);

/* Test hook for the failure path of the prefill GEMM: in the next gate/up launch one block
 * leaves out the copy of one K block of its activation rows, so its bounded waits run out:
 * the block sets the status word, frees its tensor memory and returns, blocks that start
 * later return at once, nvmai_cuda_moe_synchronize reports NVMAI_CUDA_ETIMEOUT, and the next
 * call runs normally.  Nothing faults or hangs. */
NVMAI_API int nvmai_cuda_moe_debug_drop_prefill_copy(nvmai_cuda_moe *h);

/* Test hook: holds `stream` for `ms` milliseconds with a host function (no kernel runs, the
 * device stays idle), so that a test can watch a host-side wait run out. */
NVMAI_API int nvmai_cuda_moe_debug_host_delay(nvmai_cuda_moe *h, void *stream, uint32_t ms);

/* Test hook for the failure path of the resident kernel: block `block` keeps its phase-1
 * results (router logits, shared-expert activations or the gate value) to itself, so that
 * every other block's bounded wait for them runs out and the step ends with
 * NVMAI_CUDA_ETIMEOUT at the next synchronize.  Nothing faults; 0xFFFFFFFF switches it off. */
NVMAI_API int nvmai_cuda_moe_debug_mute_block(nvmai_cuda_moe *h, uint32_t block);

/* Host-buffer convenience of the same call (copies x in, y out on `stream`, and
 * synchronises): the end-to-end path a host runtime without device buffers uses. */
NVMAI_API int nvmai_cuda_moe_stack_decode_host(nvmai_cuda_moe *h, const void *x0_f16_host, uint32_t tokens,
                                     void *y_last_host, void *stream);

/* out[r][i] = float(q)*scale + bias (Quantization.swift:104-119, 179-191) for a
 * [rows][n] affine tensor: the dequantisation every kernel here applies,
 * exposed so that it can be compared bit for bit. */
NVMAI_API int nvmai_cuda_moe_dequant(uint32_t bits, uint32_t meta_dtype, const void *w, const void *scales,
                           const void *biases, uint32_t rows, uint32_t n, float *out_f32, void *stream);

/* y[m] = half(W[m,:].x): `DequantInt4GEMV.encode` / `DequantInt8GEMV.encode`
 * (dequant_int4.metal:101-199, dequant_int8.metal:66-107). */
NVMAI_API int nvmai_cuda_moe_affine_gemv(uint32_t bits, uint32_t meta_dtype, const void *w, const void *scales,
                               const void *biases, const void *x_f16, void *y_f16, uint32_t m, uint32_t n,
                               void *stream);

/* `Elementwise` (sources/NVMAI/Kernels/Primitives/Elementwise.swift;
 * utility.metal:32-44, 60-70, 94-103). */
NVMAI_API int nvmai_cuda_moe_silu_mul_f16(const void *gate, const void *up, void *out, uint32_t count, void *stream);
NVMAI_API int nvmai_cuda_moe_sigmoid_scalar_mul_f16(void *y, const void *gate, uint32_t count, void *stream);
NVMAI_API int nvmai_cuda_moe_residual_add_f16(void *hidden, const void *delta, uint32_t count, void *stream);

/* Optional per-kernel timeline of the single-token decode stages, the counterpart
 * of the reference's NVMAI_KERNEL_STATS command-buffer times
 * (RealForwardRunner.swift:1086-1133): with tracing on, every stage launch of
 * layer_decode / stack_decode stores GPU-timer nanoseconds at
 * [layer][stage 0..2][8]: {start of block 0, latest block end, six phase marks of
 * block 0}.  read_trace synchronises the device. */
NVMAI_API int nvmai_cuda_moe_set_trace(nvmai_cuda_moe *h, int enable);
NVMAI_API int nvmai_cuda_moe_read_trace(nvmai_cuda_moe *h, uint64_t *out_host, uint32_t layers);

/* The same timeline for the resident kernel of a single-token stack step: with tracing on,
 * every block stores GPU-timer nanoseconds at [layer][block][16]: {0 input row ready, 1 phase-1
 * results stored, 2 all logits in, 3 expert tiles requested, 4 first gate/up tile landed,
 * 5 activations stored, 6 shared-expert down done, 7 routed activations staged, 8 down done,
 * 9 block output stored, 10 top-k done, 11 last gate/up tile landed, rest unused}; 0 = the block has no
 * share of that phase.
 * out_host NULL: only *out_blocks (the number of blocks) is returned. */
NVMAI_API int nvmai_cuda_moe_read_block_trace(nvmai_cuda_moe *h, uint64_t *out_host, uint32_t layers, uint32_t *out_blocks);

/* waitUntilCompleted + `.error` (RealForwardRunner.swift:3805-3837). */
NVMAI_API int nvmai_cuda_moe_synchronize(nvmai_cuda_moe *h, void *stream);
NVMAI_API int nvmai_cuda_moe_last_cuda_error(const nvmai_cuda_moe *h);
NVMAI_API const char *nvmai_cuda_moe_error_string(int code);

/* Kernel launches issued through this library since load (bench accounting). */
NVMAI_API uint64_t nvmai_cuda_moe_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* NVMAI_CUDA_MOE_H */
