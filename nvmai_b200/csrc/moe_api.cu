// C ABI of libnvmai_cuda_moe: handle, validation, launches.  The host-side
// counterpart of the reference's Swift wrappers (sources/NVMAI/Kernels/MoE/MoE.swift,
// SharedExpertInt4.swift, SharedExpertInt8.swift, Kernels/Primitives/Elementwise.swift):
// the same shape checks, turned into error codes instead of preconditions.
#include "../../include/nvmai_cuda_moe.h"

#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>
#include <fcntl.h>
#include <unistd.h>
#include <cerrno>
#include <chrono>

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <new>
#include <thread>
#include <tuple>
#include <vector>

#include "ep_comm.cuh"
#include "grouped_decode.cuh"
#include "misc_kernels.cuh"
#include "persistent_batch.cuh"
#include "persistent_decode.cuh"
#include "prefill_gemm.cuh"

using namespace nvmai;

static std::atomic<uint64_t> g_launches{0};

struct LayerViews {
    bool registered = false;
    nvmai_cuda_moe_layer w{};
    std::vector<void *> owned;      // aligned copies of resident tensors whose base was not 16-byte aligned
};

struct StackGraphKey {
    const void *x0; void *y; uint32_t tokens; cudaStream_t stream;
    bool operator<(const StackGraphKey &o) const {
        return std::tie(x0, y, tokens, stream) < std::tie(o.x0, o.y, o.tokens, o.stream);
    }
};

struct nvmai_cuda_moe {
    nvmai_cuda_moe_config cfg{};
    std::vector<LayerViews> layers;
    int last_cuda_error = 0;
    // device scratch (sized for max_tokens)
    float *logits = nullptr;        // [T][E]
    uint32_t *idx = nullptr;        // [T][K]
    __half *w = nullptr;            // [T][K]
    void *acts = nullptr;           // [T][K][F]   fp16 or fp32 by out_dtype
    void *shared_act = nullptr;     // [T][Fs]     fp16 or fp32 by out_dtype
    float *gate_val = nullptr;      // [T]
    void *y = nullptr;              // [T][D] out_dtype
    __half *xnorm = nullptr;        // [T][D]
    unsigned int *counter = nullptr;
    unsigned int *status = nullptr;  // set by a kernel whose bounded wait expired
    // batched decode: pair grouping and per-pair partial results
    uint32_t *sorted_pair = nullptr, *inv = nullptr, *expert_offsets = nullptr, *expert_counts = nullptr;
    WorkItem *work = nullptr;
    uint32_t *n_work = nullptr;
    float *partial = nullptr;        // [T*K][D]
    float *shared_partial = nullptr; // [T][D]
    uint32_t max_work = 0;
    uint32_t *group_hist = nullptr;  // [ceil(T*K / 1024)][256]: per-block expert histograms of the large grouping path
    uint32_t *expert_map = nullptr;  // expert parallelism: global id -> local blob index (device), or null
    uint32_t n_local = 0;
    // optional kernel timeline (the counterpart of the reference's NVMAI_KERNEL_STATS)
    unsigned long long *trace = nullptr;   // [num_layers][3 stages][start, end]
    bool trace_on = false;
    unsigned long long *cur_trace = nullptr;   // slot handed to the next stage launch
    const void **blob_table = nullptr;   // unused on device; kept for symmetry
    void *stage_x = nullptr;        // host-call staging: [T][D] fp16
    void *stage_y = nullptr;        // host-call staging: [T][D] out_dtype
    std::map<StackGraphKey, cudaGraphExec_t> stack_graphs;
    bool graphs_stale = false, ep_graphs_stale = false;
    // L2 prefetch of the next stage's weights in the fused layer chain: off unless
    // NVMAI_CUDA_L2_PREFETCH=1 (measured slower on B200: the prefetch competes with the
    // running stage's own copies); in_layer_chain: stage 3 follows this stage 2
    bool l2_prefetch = false, in_layer_chain = false;
    // Batches below this run every token's blocks separately; from here on rows are grouped by expert.  Measured on
    // B200 (8-bit layer): 4 rows 60 us separate / 102 us grouped, 16 rows 190 / 265, 64 rows 697 / 570.
    // NVMAI_CUDA_GROUPED_MIN overrides it.
    uint32_t grouped_min_tokens = 24;
    uint32_t tc_min_tokens = 32;     // batched decode calls from this many rows on run the tensor-core (prefill) kernels
    // prefill chunks on the tensor cores (default); NVMAI_CUDA_PREFILL_TC=0 sends them through the exact grouped
    // kernels of the batched decode path instead
    bool prefill_tc = true;
    // prefill GEMMs: fp16 operand copies (allocated by the first prefill call)
    __half *pf_x = nullptr;          // [T*K][D] x rows gathered into sorted pair order, in the weights' K order
    __half *pf_xn = nullptr;         // [T][D] x rows in token order (shared expert), in its weights' K order
    __half *pf_acts16 = nullptr;     // [T*K][F] routed activations as the down GEMM reads them
    __half *pf_sacts16 = nullptr;    // [T][Fs] the shared expert's
    float *pf_rowscale = nullptr, *pf_srowscale = nullptr;   // per row: power of two taken out of a wide-range row
    // expert parallelism over NCCL: communicator and exchange buffers
    NcclComm ep_comm = nullptr;
    uint32_t ep_rank = 0, ep_world = 0, ep_rows_own = 0;
    __half *ep_x_all = nullptr;      // [world * rows_own][D]: every rank's rows, in rank order
    float *ep_share = nullptr;       // [world * rows_own][D]: this rank's share of every row
    float *ep_recv = nullptr;        // [world][rows_own][D]: every rank's share of this rank's rows
    void *ep_h1 = nullptr;           // [rows_own][D] out_dtype: shared expert of this rank's rows
    // the shared expert runs beside the exchange + routed experts on a second stream (forked and joined per layer,
    // also inside the captured graph)
    cudaStream_t ep_side = nullptr;
    cudaEvent_t ep_fork = nullptr, ep_join = nullptr;
    // peer-memory exchange of the shares (replicated mode): own area = [counters, 4 KB][receive buffers 2 x world*rows*D fp32],
    // exported to the other ranks as a CUDA IPC handle; ep_peer_base[r] = rank r's area as mapped here
    unsigned char *ep_xchg = nullptr;
    unsigned char *ep_peer_base[kEpMaxRanks] = {};
    bool ep_peers_attached = false;
    unsigned long long *ep_step = nullptr;      // device: [0] number of steps enqueued (incremented by the step's first kernel),
                                                // [2 ..] this rank's block counters per layer
    size_t ep_buf_elems = 0;
    struct EpGraph { cudaGraphExec_t exec = nullptr; uint32_t calls = 0; };
    std::map<StackGraphKey, EpGraph> ep_graphs;
    // one-launch decode step (persistent_decode.cuh): per-layer views on the device, the tagged exchange words,
    // the epoch word and the experts each layer selected
    PdLayer *pd_layers = nullptr;
    bool pd_layers_stale = true, pd_unavailable = false;
    unsigned long long *pd_xchg = nullptr;
    unsigned long long *pb_xchg = nullptr;    // the batch kernel's exchange words (up to kPbMaxRows rows)
    unsigned int *pd_epoch = nullptr;
    uint32_t *pd_route_log = nullptr;     // [num_layers][rows of the step <= 8][top_k]
    uint32_t pd_route_rows = 1;           // rows of the last resident-kernel step
    size_t ep_xin_off = 0;                // byte offset of the fused dispatch's row area inside ep_xchg
    bool pf_debug_drop = false;           // test hook: the next gate/up GEMM launch leaves out one copy (its waits run out)
    int sm_count = 0;
    // 0: a single-token stack step takes the one-launch kernel when the shape allows it; 1: always the staged
    // kernels; 2: the one-launch kernel or NVMAI_CUDA_EINVAL
    int decode_mode = 0;
    unsigned long long *pd_trace = nullptr;   // [num_layers][sm_count][16] marks of the resident kernel (allocated by set_trace)
    uint32_t pd_mute_block = 0xFFFFFFFFu;     // test hook, see nvmai_cuda_moe_debug_mute_block
    // the next block's input norm, handed from the entry point to the launch of the block's last stage
    NextNorm next_norm{};
    unsigned int *row_counter = nullptr;      // [max_tokens]
};

namespace {

// NVTX ranges around the entry points, named after the roles the reference's runner gives its command buffers
// (recordKernelGPU(role:), RealForwardRunner.swift:3839-3844, :3224-3225, :3393-3418, :3574), so that a timeline of the
// host reads like the reference's NVMAI_KERNEL_STATS.  On when NVMAI_CUDA_NVTX=1 is in the environment at the first
// call; without a profiler attached a range costs a function-pointer check.
inline bool nvtx_on() {
    static const bool on = [] { const char *v = std::getenv("NVMAI_CUDA_NVTX"); return v && std::atoi(v) != 0; }();
    return on;
}
struct NvtxRange {
    bool on;
    explicit NvtxRange(const char *role) : on(nvtx_on()) { if (on) nvtxRangePushA(role); }
    ~NvtxRange() { if (on) nvtxRangePop(); }
    NvtxRange(const NvtxRange &) = delete;
    NvtxRange &operator=(const NvtxRange &) = delete;
};


inline size_t out_size(uint32_t out_dtype) { return out_dtype == NVMAI_OUT_FP16 ? 2 : 4; }
inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool valid_bits(uint32_t b) { return b == 4 || b == 8; }

int record(nvmai_cuda_moe *h, cudaError_t e) {
    if (e == cudaSuccess) return NVMAI_CUDA_OK;
    if (h) h->last_cuda_error = (int)e;
    return NVMAI_CUDA_ECUDA;
}

int check_launch(nvmai_cuda_moe *h) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return record(h, cudaGetLastError());
}

RoutedSource source_from_blobs(const void *const *blobs, uint32_t top_k) {
    RoutedSource s{};
    for (uint32_t k = 0; k < kMaxTopK; ++k) s.blob[k] = k < top_k ? static_cast<const uint8_t *>(blobs[k]) : nullptr;
    return s;
}

RoutedSource source_from_layer(const nvmai_cuda_moe *h, const LayerViews &lv, const uint32_t *idx) {
    RoutedSource s{};
    s.idx = idx;
    s.base = static_cast<const uint8_t *>(lv.w.experts);
    s.stride = lv.w.expert_stride;
    s.num_experts = h->cfg.num_experts;
    return s;
}

ExpertOffsets to_offsets(const nvmai_expert_offsets &o) {
    ExpertOffsets r;
    r.o[0] = o.gate_w; r.o[1] = o.gate_s; r.o[2] = o.gate_b;
    r.o[3] = o.up_w; r.o[4] = o.up_s; r.o[5] = o.up_b;
    r.o[6] = o.down_w; r.o[7] = o.down_s; r.o[8] = o.down_b;
    return r;
}

AffineMat to_mat(const nvmai_affine_tensor &t) {
    return AffineMat{static_cast<const uint8_t *>(t.w), static_cast<const uint16_t *>(t.scales),
                     static_cast<const uint16_t *>(t.biases)};
}

// Offsets must keep every sub-tensor 16-byte aligned inside a 16-byte aligned blob
// and stay inside the blob; the reference checks `offset + bytes <= length`
// (SharedExpertInt4.swift:47-59).
int check_offsets(const nvmai_cuda_moe_config &c, const nvmai_expert_offsets &o, uint64_t stride) {
    const uint64_t gate_w = (uint64_t)c.f * c.d * c.routed_bits / 8, gate_m = (uint64_t)c.f * (c.d / 64) * 2;
    const uint64_t down_w = (uint64_t)c.d * c.f * c.routed_bits / 8, down_m = (uint64_t)c.d * (c.f / 64) * 2;
    const uint32_t offs[9] = {o.gate_w, o.gate_s, o.gate_b, o.up_w, o.up_s, o.up_b, o.down_w, o.down_s, o.down_b};
    const uint64_t lens[9] = {gate_w, gate_m, gate_m, gate_w, gate_m, gate_m, down_w, down_m, down_m};
    for (int i = 0; i < 9; ++i) {
        if (offs[i] & 15u) return NVMAI_CUDA_EINVAL;
        if (stride != 0 && (uint64_t)offs[i] + lens[i] > stride) return NVMAI_CUDA_ERANGE;
    }
    return NVMAI_CUDA_OK;
}

template <typename F>
int dispatch_out(uint32_t out_dtype, F &&f) {
    if (out_dtype == NVMAI_OUT_FP16) return f(std::integral_constant<int, OUT_F16>{});
    return f(std::integral_constant<int, OUT_F32>{});
}

template <typename F>
int dispatch_bits_meta(uint32_t bits, uint32_t meta, F &&f) {
    if (bits == 4 && meta == NVMAI_META_BF16) return f(std::integral_constant<int, 4>{}, std::integral_constant<int, META_BF16>{});
    if (bits == 4 && meta == NVMAI_META_FP16) return f(std::integral_constant<int, 4>{}, std::integral_constant<int, META_FP16>{});
    if (bits == 8 && meta == NVMAI_META_BF16) return f(std::integral_constant<int, 8>{}, std::integral_constant<int, META_BF16>{});
    if (bits == 8 && meta == NVMAI_META_FP16) return f(std::integral_constant<int, 8>{}, std::integral_constant<int, META_FP16>{});
    return NVMAI_CUDA_EINVAL;
}

// ---- stage launchers ---------------------------------------------------------

// Kernels here use more than the default 48 KB of dynamic shared memory; the
// opt-in is per function and sticky, so it is raised once per (function, size).
template <typename Kern>
cudaError_t ensure_smem(Kern kern, size_t bytes) {
    // the attribute is per device and handles may be driven from several host threads
    static std::map<std::pair<int, const void *>, size_t> granted;
    static std::mutex guard;
    int dev = 0;
    cudaError_t de = cudaGetDevice(&dev);
    if (de != cudaSuccess) return de;
    std::lock_guard<std::mutex> lock(guard);
    const auto key = std::make_pair(dev, reinterpret_cast<const void *>(kern));
    auto it = granted.find(key);
    if (it != granted.end() && it->second >= bytes) return cudaSuccess;
    if (bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) return e;
    }
    granted[key] = bytes;
    return cudaSuccess;
}

// pdl: launch with programmatic stream serialization, so that the kernel's
// prologue (its weight copies) may overlap the previous kernel's tail.
template <typename Kern, typename... Params>
int launch_kernel(nvmai_cuda_moe *h, Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl,
                  const Params &...p) {
    cudaError_t e = ensure_smem(kern, smem);
    if (e != cudaSuccess) return record(h, e);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    e = cudaLaunchKernelEx(&cfg, kern, p...);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return record(h, e);
}

constexpr size_t kMaxSmem = 227 * 1024;

// with_shared: the shared expert's gate/up tiles run here (one block per token and
// tile); with_gate: the scalar gate row.  The batched path runs the tiles in its
// grouped stage instead and asks for the gate only.
int launch_stage1(nvmai_cuda_moe *h, const LayerViews &lv, const XSource &xsrc, uint32_t tokens,
                  uint32_t *out_idx, __half *out_w, bool with_router, bool with_shared, bool with_gate, bool pdl,
                  cudaStream_t st, bool defer_topk = false) {
    const auto &c = h->cfg;
    Stage1Params p{};
    p.rW = static_cast<const uint8_t *>(lv.w.router.w);
    p.rS = static_cast<const uint16_t *>(lv.w.router.scales);
    p.rB = static_cast<const uint16_t *>(lv.w.router.biases);
    p.eff = static_cast<const uint16_t *>(lv.w.effective_scale);
    p.pes = static_cast<const uint16_t *>(lv.w.per_expert_scale);
    p.router_kind = c.router_kind;
    p.logits = h->logits;
    p.out_idx = out_idx;
    p.out_w = out_w;
    p.counter = h->counter;
    p.defer_topk = defer_topk ? 1u : 0u;
    p.sgate = to_mat(lv.w.shared_gate_proj);
    p.sup = to_mat(lv.w.shared_up_proj);
    p.shared_f = with_shared ? c.shared_f : 0;
    p.shared_act = h->shared_act;
    p.gW = static_cast<const uint8_t *>(lv.w.shared_gate.w);
    p.gS = static_cast<const uint16_t *>(lv.w.shared_gate.scales);
    p.gB = static_cast<const uint16_t *>(lv.w.shared_gate.biases);
    p.gate_kind = c.shared_gate_kind;
    p.gate_val = h->gate_val;
    p.xsrc = xsrc; p.tokens = tokens;
    p.trace = h->cur_trace;
    p.D = c.d; p.E = c.num_experts; p.K = c.top_k; p.act = c.activation;
    p.status = h->status;
    p.tokens_per_chunk = tokens <= 8 ? tokens : 8;
    const uint32_t chunks = (tokens + p.tokens_per_chunk - 1) / p.tokens_per_chunk;
    p.router_row_blocks = (c.num_experts + kRowsPerRouterBlock - 1) / kRowsPerRouterBlock;
    p.n_router_blocks = with_router ? p.router_row_blocks * chunks : 0;
    p.n_shared_blocks = with_shared ? ((c.shared_f + kBlockFeatures - 1) / kBlockFeatures) * tokens : 0;
    const bool gated = with_gate && c.shared_f != 0 && c.shared_gate_kind != NVMAI_GATE_NONE;
    p.n_gate_blocks = gated ? chunks : 0;
    const uint32_t grid = p.n_router_blocks + p.n_shared_blocks + p.n_gate_blocks;
    if (grid == 0) return NVMAI_CUDA_OK;
    size_t smem = 0;
    if (with_router) smem = std::max(smem, RowsLayout(c.d, c.router_kind).total);
    if (with_router && !defer_topk) smem = std::max(smem, kTopkSmemBytes);      // the last router block selects in place
    if (gated) smem = std::max(smem, RowsLayout(c.d, c.shared_gate_kind).total);
    if (with_shared) smem = std::max(smem, GateUpLayout(c.d, c.shared_bits).total);
    return dispatch_bits_meta(c.shared_f ? c.shared_bits : 4, c.meta_dtype, [&](auto B, auto M) {
        return dispatch_out(c.out_dtype, [&](auto O) {
            return launch_kernel(h, stage1_kernel<decltype(B)::value, decltype(M)::value, decltype(O)::value>,
                                 dim3(grid), dim3(kDecodeThreads), smem, st, pdl, p);
        });
    });
}

int launch_stage2(nvmai_cuda_moe *h, const RoutedSource &src, const ExpertOffsets &off, const __half *x,
                  uint32_t x_stride, uint32_t tokens, void *acts, const uint32_t *active_slots_dev,
                  uint32_t n_slots, bool pdl, cudaStream_t st) {
    const auto &c = h->cfg;
    Stage2Params p{};
    p.src = src; p.off = off; p.x = x; p.x_stride = x_stride; p.acts = acts;
    p.active_slots = active_slots_dev;
    p.D = c.d; p.F = c.f; p.top_k = c.top_k; p.act = c.activation;
    p.prefetch_down = (h->l2_prefetch && h->in_layer_chain) ? 1u : 0u;
    p.status = h->status;
    p.trace = h->cur_trace;
    dim3 grid((c.f + kBlockFeatures - 1) / kBlockFeatures, n_slots, tokens);
    const size_t smem = GateUpLayout(c.d, c.routed_bits).total;
    return dispatch_bits_meta(c.routed_bits, c.meta_dtype, [&](auto B, auto M) {
        return dispatch_out(c.out_dtype, [&](auto O) {
            return launch_kernel(h, stage2_kernel<decltype(B)::value, decltype(M)::value, decltype(O)::value>, grid,
                                 dim3(kDecodeThreads), smem, st, pdl, p);
        });
    });
}

int launch_stage3(nvmai_cuda_moe *h, Stage3Params p, uint32_t tokens, bool pdl, cudaStream_t st) {
    const auto &c = h->cfg;
    p.D = c.d; p.F = c.f;
    p.status = h->status;
    p.trace = h->cur_trace;
    dim3 grid(c.d / kTileRows, tokens);
    const uint32_t units = p.top_k + (p.shared_f ? 1 : 0);
    const uint32_t threads = (units < 1 ? 1 : units) * kDownSplit * 32;
    const size_t smem = DownLayout(c.f, p.shared_f, c.routed_bits, p.shared_bits, units).total;
    return dispatch_bits_meta(c.routed_bits, c.meta_dtype, [&](auto B, auto M) {
        return dispatch_out(c.out_dtype, [&](auto O) {
            return launch_kernel(h, stage3_kernel<decltype(B)::value, decltype(M)::value, decltype(O)::value>, grid,
                                 dim3(threads), smem, st, pdl, p);
        });
    });
}

int check_layer(const nvmai_cuda_moe *h, uint32_t layer) {
    if (!h) return NVMAI_CUDA_EINVAL;
    if (layer >= h->layers.size()) return NVMAI_CUDA_ERANGE;
    if (!h->layers[layer].registered) return NVMAI_CUDA_EINVAL;
    return NVMAI_CUDA_OK;
}

// The shared expert alone: gate/up tiles + gate row, then its down projection.
int shared_expert_impl(nvmai_cuda_moe *h, const LayerViews &lv, const XSource &xsrc, uint32_t tokens, void *h1,
                       cudaStream_t st) {
    const auto &c = h->cfg;
    int rc = launch_stage1(h, lv, xsrc, tokens, nullptr, nullptr, false, true, true, false, st);
    if (rc) return rc;
    Stage3Params p{};
    p.sdown = to_mat(lv.w.shared_down_proj);
    p.shared_f = c.shared_f;
    p.shared_bits = c.shared_bits;
    p.shared_act = h->shared_act;
    p.gate_val = c.shared_gate_kind != NVMAI_GATE_NONE ? h->gate_val : nullptr;
    p.y = h1;
    p.top_k = 0;
    return launch_stage3(h, p, tokens, false, st);
}

void ep_release(nvmai_cuda_moe *h) {
    for (auto &kv : h->ep_graphs) if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
    h->ep_graphs.clear();
    if (h->ep_comm) { nccl_api().CommDestroy(h->ep_comm); h->ep_comm = nullptr; }
    for (uint32_t r = 0; r < (uint32_t)kEpMaxRanks; ++r) {
        if (h->ep_peer_base[r] && h->ep_peer_base[r] != h->ep_xchg) cudaIpcCloseMemHandle(h->ep_peer_base[r]);
        h->ep_peer_base[r] = nullptr;
    }
    h->ep_peers_attached = false;
    cudaFree(h->ep_xchg); h->ep_xchg = nullptr;
    cudaFree(h->ep_step); h->ep_step = nullptr;
    if (h->ep_side) { cudaStreamDestroy(h->ep_side); h->ep_side = nullptr; }
    if (h->ep_fork) { cudaEventDestroy(h->ep_fork); h->ep_fork = nullptr; }
    if (h->ep_join) { cudaEventDestroy(h->ep_join); h->ep_join = nullptr; }
    cudaFree(h->ep_x_all); cudaFree(h->ep_share); cudaFree(h->ep_recv); cudaFree(h->ep_h1);
    h->ep_x_all = nullptr; h->ep_share = nullptr; h->ep_recv = nullptr; h->ep_h1 = nullptr;
    h->ep_world = h->ep_rows_own = 0;
}


int launch_group_pairs(nvmai_cuda_moe *h, const uint32_t *idx, const __half *w, uint32_t tokens,
                       TokenExpertPair *pairs_out, uint32_t *offsets_out, uint32_t *counts_out, bool with_work,
                       bool pdl, cudaStream_t st, bool with_shared = true, bool use_map = false,
                       uint32_t pairs_per_item = 0, bool even_split = false) {
    const auto &c = h->cfg;
    GroupParams g{};
    g.idx = idx; g.weights = w; g.tokens = tokens; g.K = c.top_k; g.E = c.num_experts;
    g.sorted_pair = h->sorted_pair; g.inv = h->inv;
    g.expert_offsets = offsets_out ? offsets_out : h->expert_offsets;
    g.expert_counts = counts_out ? counts_out : h->expert_counts;
    g.pairs_out = pairs_out;
    g.work = with_work ? h->work : nullptr;
    g.n_work = h->n_work;
    g.shared_chunks = (with_work && with_shared && c.shared_f) ? (tokens + kPairsPerItem - 1) / kPairsPerItem : 0;
    g.expert_map = use_map ? h->expert_map : nullptr;
    g.n_local = (use_map && h->expert_map) ? h->n_local : c.num_experts;
    g.pairs_per_item = pairs_per_item; g.even_split = even_split ? 1u : 0u;
    const uint32_t P = tokens * c.top_k;
    if (P > 4 * kGroupThreads) {          // large pair counts: histogram / scan / scatter over P / 1024 blocks
        const uint32_t n_blocks = (P + kGroupThreads - 1) / kGroupThreads;
        int rc = launch_kernel(h, group_hist_kernel, dim3(n_blocks), dim3(kGroupThreads), 0, st, pdl, g, h->group_hist);
        if (rc) return rc;
        if ((rc = launch_kernel(h, group_scan_kernel, dim3(1), dim3(kMaxExperts), 0, st, true, g, h->group_hist, n_blocks))) return rc;
        return launch_kernel(h, group_scatter_kernel, dim3(n_blocks), dim3(kGroupThreads), 0, st, true, g,
                             static_cast<const uint32_t *>(h->group_hist));
    }
    return launch_kernel(h, group_pairs_kernel, dim3(1), dim3(kGroupThreads), 0, st, pdl, g);
}

// Batched tail of a layer: group pairs by expert, gate/up and down per (tile, work
// item), then the per-token weighted sum in rank order.
// partial_y != nullptr: expert-parallel share (local experts only, no shared expert, fp32 rows out).
int grouped_tail(nvmai_cuda_moe *h, const LayerViews &lv, const __half *x_rows, uint32_t tokens, const uint32_t *idx,
                 const __half *w, void *hidden, void *y, cudaStream_t st, float *partial_y = nullptr,
                 const __half *hidden_delta = nullptr, bool prefill_rounding = false) {
    const auto &c = h->cfg;
    const bool ep = partial_y != nullptr;
    int rc = launch_group_pairs(h, idx, w, tokens, nullptr, nullptr, nullptr, true, !ep, st, !ep, ep);
    if (rc) return rc;
    const uint32_t P = tokens * c.top_k;
    const uint32_t routed_bound = std::min(P, c.num_experts + P / kPairsPerItem);
    const uint32_t shared_chunks = (c.shared_f && !ep) ? (tokens + kPairsPerItem - 1) / kPairsPerItem : 0;
    GroupedStage2Params p2{};
    p2.experts = static_cast<const uint8_t *>(lv.w.experts); p2.stride = lv.w.expert_stride; p2.num_experts = c.num_experts;
    p2.off = to_offsets(lv.w.offsets);
    p2.work = h->work; p2.n_work = h->n_work; p2.sorted_pair = h->sorted_pair;
    p2.x = x_rows; p2.x_stride = c.d; p2.acts = h->acts;
    p2.sgate = to_mat(lv.w.shared_gate_proj); p2.sup = to_mat(lv.w.shared_up_proj);
    p2.shared_f = c.shared_f; p2.shared_bits = c.shared_bits; p2.shared_act = h->shared_act;
    p2.D = c.d; p2.F = c.f; p2.K = c.top_k; p2.act = c.activation; p2.status = h->status;
    const uint32_t fmax = std::max(c.f, c.shared_f);
    size_t smem2 = GroupedGateUpLayout(c.d, c.routed_bits).total;
    if (c.shared_f) smem2 = std::max(smem2, GroupedGateUpLayout(c.d, c.shared_bits).total);
    rc = dispatch_bits_meta(c.routed_bits, c.meta_dtype, [&](auto B, auto M) {
        return dispatch_out(c.out_dtype, [&](auto O) {
            return launch_kernel(h, grouped_stage2_kernel<decltype(B)::value, decltype(M)::value, decltype(O)::value>,
                                 dim3(fmax / kTileFeatures, routed_bound + shared_chunks), dim3(kDecodeThreads), smem2,
                                 st, true, p2);
        });
    });
    if (rc) return rc;
    GroupedStage3Params p3{};
    p3.experts = p2.experts; p3.stride = p2.stride; p3.num_experts = c.num_experts; p3.off = p2.off;
    p3.work = h->work; p3.n_work = h->n_work; p3.acts = h->acts; p3.partial = h->partial;
    p3.sdown = to_mat(lv.w.shared_down_proj); p3.shared_f = c.shared_f; p3.shared_bits = c.shared_bits;
    p3.shared_act = h->shared_act; p3.shared_partial = h->shared_partial;
    p3.D = c.d; p3.F = c.f; p3.status = h->status;
    const size_t smem3 = GroupedDownLayout(c.f, c.shared_f, c.routed_bits, c.shared_bits).total;
    rc = dispatch_bits_meta(c.routed_bits, c.meta_dtype, [&](auto B, auto M) {
        return dispatch_out(c.out_dtype, [&](auto O) {
            return launch_kernel(h, grouped_stage3_kernel<decltype(B)::value, decltype(M)::value, decltype(O)::value>,
                                 dim3(c.d / kTileRows, routed_bound + shared_chunks), dim3(kDecodeThreads), smem3, st,
                                 true, p3);
        });
    });
    if (rc) return rc;
    CombineParams pc{};
    pc.partial = h->partial; pc.shared_partial = (c.shared_f && !ep) ? h->shared_partial : nullptr;
    pc.inv = h->inv; pc.routing_w = w;
    pc.gate_val = (c.shared_f && c.shared_gate_kind != NVMAI_GATE_NONE) ? h->gate_val : nullptr;
    pc.residual = nullptr; pc.y = y; pc.hidden = hidden; pc.D = c.d; pc.K = c.top_k;
    pc.partial_y = partial_y;
    pc.hidden_delta = hidden_delta;
    pc.prefill = prefill_rounding ? 1 : 0;
    if (!prefill_rounding && !ep) pc.next = h->next_norm;
    return dispatch_out(c.out_dtype, [&](auto O) {
        return launch_kernel(h, combine_kernel<decltype(O)::value>, dim3(tokens), dim3(256), 0, st, true, pc);
    });
}

// xsrc: where stage 1 gets its rows; x_rows: the fp16 rows stages 2 reads (the
// same buffer, or the buffer stage 1 writes its normalised rows to).
int layer_decode_impl(nvmai_cuda_moe *h, uint32_t layer, const XSource &xsrc, const __half *x_rows, uint32_t tokens,
                      void *hidden, void *h2_out, uint32_t *out_idx, __half *out_w, cudaStream_t st,
                      const LayerViews *next_layer = nullptr, const __half *hidden_delta = nullptr) {
    const auto &c = h->cfg;
    const LayerViews &lv = h->layers[layer];
    uint32_t *idx = out_idx ? out_idx : h->idx;
    __half *w = out_w ? out_w : h->w;
    const bool grouped = tokens >= h->grouped_min_tokens;
    auto slot = [&](int stage) { return (h->trace_on && !grouped) ? h->trace + ((size_t)layer * 3 + stage) * kTraceWords : nullptr; };
    h->cur_trace = slot(0);
    // single-token path: the expert stages select the experts themselves from the logits
    // (the block-wide selection wants one thread per expert in the down stage's block too)
    const bool defer = !grouped && (c.top_k + (c.shared_f ? 1 : 0)) * kDownSplit * 32 >= (uint32_t)kMaxExperts;
    int rc = launch_stage1(h, lv, xsrc, tokens, idx, w, true, c.shared_f != 0 && !grouped, c.shared_f != 0, true, st,
                           defer);
    if (rc) return rc;
    h->cur_trace = nullptr;
    if (grouped) return grouped_tail(h, lv, x_rows, tokens, idx, w, hidden, h2_out ? h2_out : h->y, st, nullptr, hidden_delta);
    h->cur_trace = slot(1);
    RoutedSource src = source_from_layer(h, lv, idx);
    if (defer) {
        src.logits = h->logits;
        src.pes = static_cast<const uint16_t *>(lv.w.per_expert_scale);
        src.publish_idx = idx;
        src.publish_w = w;
    }
    h->in_layer_chain = true;
    rc = launch_stage2(h, src, to_offsets(lv.w.offsets), x_rows, c.d, tokens, h->acts, nullptr, c.top_k, true, st);
    h->in_layer_chain = false;
    h->cur_trace = nullptr;
    if (rc) return rc;
    h->cur_trace = slot(2);
    Stage3Params p{};
    p.src = src;
    p.off = to_offsets(lv.w.offsets);
    p.acts = h->acts;
    p.routing_w = w;
    p.residual = nullptr;
    p.sdown = to_mat(lv.w.shared_down_proj);
    p.shared_f = c.shared_f;
    p.shared_bits = c.shared_bits;
    p.shared_act = h->shared_act;
    p.gate_val = c.shared_gate_kind != NVMAI_GATE_NONE ? h->gate_val : nullptr;
    p.h1_out = nullptr;
    p.y = h2_out ? h2_out : h->y;
    p.hidden = hidden;
    p.hidden_delta = hidden_delta;
    p.top_k = c.top_k;
    p.next = h->next_norm;
    if (next_layer != nullptr && h->l2_prefetch) {    // stack driver: warm the L2 with what the next layer's first stage reads
        const auto &nw = next_layer->w;
        const size_t router_bytes = c.router_kind == 0 ? (size_t)c.num_experts * c.d * 2
                                                       : (size_t)c.num_experts * c.d * c.router_kind / 8;
        const size_t router_meta = c.router_kind == 0 ? 0 : (size_t)c.num_experts * (c.d / 64) * 2;
        const size_t sw = (size_t)c.shared_f * c.d * c.shared_bits / 8, sm = (size_t)c.shared_f * (c.d / 64) * 2;
        int n = 0;
        auto add = [&](const void *ptr, size_t bytes) { if (ptr && bytes && n < 6) { p.next_ptr[n] = ptr; p.next_bytes[n] = bytes; ++n; } };
        add(nw.router.w, router_bytes);
        add(nw.router.scales, router_meta);
        add(nw.router.biases, router_meta);
        if (c.shared_f) {
            add(nw.shared_gate_proj.w, sw);
            add(nw.shared_up_proj.w, sw);
            add(nw.shared_gate_proj.scales, sm);   // the remaining meta arrays are small; the copies fetch them
        }
    }
    rc = launch_stage3(h, p, tokens, true, st);
    h->cur_trace = nullptr;
    return rc;
}

// ---- prefill: grouped GEMMs on the tensor cores ----------------------------------
int ensure_prefill_scratch(nvmai_cuda_moe *h, cudaStream_t st) {
    if (h->pf_acts16) return NVMAI_CUDA_OK;
    // the first prefill call allocates; a stream under capture forbids that: make one eager call first
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (st != nullptr && (cudaStreamIsCapturing(st, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone)) {
        cudaGetLastError();
        return NVMAI_CUDA_EINVAL;
    }
    const auto &c = h->cfg;
    const size_t T = c.max_tokens, P = T * c.top_k;
    auto alloc = [&](auto **ptr, size_t bytes) { return cudaMalloc(reinterpret_cast<void **>(ptr), bytes ? bytes : 16) == cudaSuccess; };
    const size_t dx = c.d + pf_extra_cols(c.d), fx = c.f + pf_extra_cols(c.f), sfx = c.shared_f + pf_extra_cols(c.shared_f);
    if (alloc(&h->pf_x, P * dx * 2) && alloc(&h->pf_xn, T * dx * 2) && alloc(&h->pf_acts16, P * fx * 2) &&
        alloc(&h->pf_sacts16, T * sfx * 2) && alloc(&h->pf_rowscale, P * 4) && alloc(&h->pf_srowscale, T * 4))
        return NVMAI_CUDA_OK;
    cudaGetLastError();
    cudaFree(h->pf_x); cudaFree(h->pf_xn); cudaFree(h->pf_acts16); cudaFree(h->pf_sacts16); cudaFree(h->pf_rowscale);
    cudaFree(h->pf_srowscale);
    h->pf_x = h->pf_xn = h->pf_acts16 = h->pf_sacts16 = nullptr; h->pf_rowscale = h->pf_srowscale = nullptr;
    return NVMAI_CUDA_ENOMEM;
}

// cuTensorMapEncodeTiled, looked up through the runtime (the library does not link libcuda)
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                   const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Tensor map over fp16 rows [rows][cols] (row stride in elements), box = 64 values x box_rows rows, 128-byte
// swizzle, zero fill outside.  Base and row stride must be 16-byte multiples.
int make_rows_tmap(nvmai_cuda_moe *h, CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, uint64_t stride_elems,
                   uint32_t box_rows) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return NVMAI_CUDA_ECUDA;
    if (!aligned16(base) || (stride_elems * 2) % 16 != 0 || cols % kPfKBlock != 0) return NVMAI_CUDA_EINVAL;
    const cuuint64_t gdim[2] = {cols, rows};
    const cuuint64_t gstride[1] = {stride_elems * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kPfKBlock, box_rows};
    const cuuint32_t estride[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(base), gdim, gstride, box, estride,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { h->last_cuda_error = (int)r; return NVMAI_CUDA_ECUDA; }
    return NVMAI_CUDA_OK;
}

// b_rows: fp16 [b_count][kdim] in work-item order; b2_rows: the direct items' rows (token order), or nullptr
template <int PHASE>
int launch_prefill_gemm(nvmai_cuda_moe *h, uint32_t bits, const PrefillGemmParams &p, const void *b_rows, uint64_t b_count,
                        const void *b2_rows, uint64_t b2_count, dim3 grid, cudaStream_t st) {
    const auto &c = h->cfg;
    PrefillGemmArgs args{};
    args.p = p;
    if (PHASE == 0 && h->pf_debug_drop) { args.p.debug_drop_b = 1; h->pf_debug_drop = false; }     // one launch only
    const uint64_t cols = p.kdim + pf_extra_cols(p.kdim);        // the rows carry their correction columns
    int rc = make_rows_tmap(h, &args.tmap_b, b_rows, b_count, cols, cols, kPfBoxRows);
    if (rc) return rc;
    if (b2_rows != nullptr) {
        if ((rc = make_rows_tmap(h, &args.tmap_a, b2_rows, b2_count, cols, cols, kPfBoxRows))) return rc;
    } else {
        args.tmap_a = args.tmap_b;
    }
    return dispatch_bits_meta(bits, c.meta_dtype, [&](auto B, auto M) {
        return dispatch_out(c.out_dtype, [&](auto O) {
            return launch_kernel(h, prefill_gemm_kernel<decltype(B)::value, decltype(M)::value, decltype(O)::value, PHASE>,
                                 grid, dim3(kPfThreads), kPfSmemBytes, st, true, args);
        });
    });
}

// rows of src (out_dtype for intermediates, fp16 for x) -> fp16 rows in the K order the weights of `bits` unpack
// in; gather != nullptr: output row r comes from source row gather[r] / gather_div
int launch_pack_rows(nvmai_cuda_moe *h, const void *src, bool src_f32, __half *dst, float *row_scale, uint32_t rows,
                     uint32_t n, uint32_t bits, cudaStream_t st, const uint32_t *gather = nullptr, uint32_t gather_div = 1,
                     uint32_t src_rows = 1) {
    PackRowsParams p{src, dst, src_f32 ? row_scale : nullptr, rows, n, bits == 4 ? 1u : 0u, gather, gather_div, src_rows, pf_extra_cols(n)};
    const dim3 grid((rows + 7) / 8), block(256);
    if (src_f32) return launch_kernel(h, pack_rows_kernel<1>, grid, block, 0, st, true, p);
    return launch_kernel(h, pack_rows_kernel<0>, grid, block, 0, st, true, p);
}

// The whole block for `tokens` rows: router, grouping, gate/up GEMMs + activation,
// down GEMMs, rank-ordered weighted sum with the shared expert and the two-step
// residual of the prefill path (RealForwardRunner.swift:3244-3591).
// The same launches serve the batched decode entry points from a few dozen rows on, where the tensor-core tiles
// beat the per-row tiles of the decode kernels:
//   decode_order  the block's result takes the decode path's rounding (one rounding of h1 + sum, one residual add)
//   routed_only   routing given by the caller (out_idx / out_w are inputs), no router, no shared expert
//   partial_y     fp32 rows that receive sum_r w_r * down_r instead of y / hidden (expert-parallel share, replay)
struct PrefillMode {
    bool decode_order = false;
    bool routed_only = false;
    float *partial_y = nullptr;
    const __half *hidden_delta = nullptr;
};

int layer_prefill_impl(nvmai_cuda_moe *h, uint32_t layer, const __half *x, uint32_t tokens, void *hidden, void *y,
                       uint32_t *out_idx, __half *out_w, cudaStream_t st, const PrefillMode mode = PrefillMode{}) {
    const LayerViews &lv = h->layers[layer];
    int rc = ensure_prefill_scratch(h, st);
    if (rc) return rc;
    nvmai_cuda_moe_config c = h->cfg;
    if (mode.routed_only) c.shared_f = 0;
    uint32_t *idx = out_idx ? out_idx : h->idx;
    __half *w = out_w ? out_w : h->w;
    const bool wide = c.out_dtype == NVMAI_OUT_FP32;
    const XSource xsrc{x, c.d, nullptr, nullptr};
    // A dense fp16 router without an input scale is a plain GEMM (products of two fp16 values are
    // exact in fp32, so only the order of the fp32 additions differs from the decode router's);
    // affine routers keep the exact code-times-activation kernel.
    const bool gemm_router = c.router_kind == NVMAI_ROUTER_DENSE_F16 && lv.w.effective_scale == nullptr &&
                             c.num_experts % (2 * kPfTileM) == 0;
    if (mode.routed_only) {
        // nothing to route
    } else if (gemm_router) {
        PrefillGemmArgs ra{};
        PrefillGemmParams &r = ra.p;
        r.shared_from = 0;
        r.tokens = tokens; r.top_k = c.top_k; r.kdim = c.d;
        r.out2 = h->logits; r.out_stride2 = c.num_experts; r.status = h->status;
        if ((rc = make_rows_tmap(h, &ra.tmap_b, x, tokens, c.d, c.d, kPfBoxRows))) return rc;
        if ((rc = make_rows_tmap(h, &ra.tmap_a, lv.w.router.w, c.num_experts, c.d, c.d, kPfTileM))) return rc;
        const dim3 grid(c.num_experts / (2 * kPfTileM), (tokens + kPfTileN - 1) / kPfTileN);
        if ((rc = launch_kernel(h, prefill_gemm_kernel<16, 0, 0, 2>, grid, dim3(kPfThreads), kPfSmemBytes, st, false, ra)))
            return rc;
        TopkRowsParams tk{h->logits, static_cast<const uint16_t *>(lv.w.per_expert_scale), idx, w, c.num_experts, c.top_k, tokens};
        if ((rc = launch_kernel(h, topk_rows_kernel, dim3((tokens + 7) / 8), dim3(256), 0, st, true, tk))) return rc;
        if (c.shared_f && (rc = launch_stage1(h, lv, xsrc, tokens, nullptr, nullptr, false, false, true, false, st))) return rc;
    } else if ((rc = launch_stage1(h, lv, xsrc, tokens, idx, w, true, false, c.shared_f != 0, false, st))) {
        return rc;
    }
    // with an expert map (this rank holds a part of the experts) the pairs of the other ranks' experts are left out
    // of the grouping: the items, the packed rows and the partial rows then cover this rank's pairs only
    const bool use_map = h->expert_map != nullptr;
    if ((rc = launch_group_pairs(h, idx, w, tokens, nullptr, nullptr, nullptr, true, true, st, false, use_map, kPfTileN, true)))
        return rc;
    const uint32_t P = tokens * c.top_k;
    const uint32_t max_items = std::min(P, c.num_experts + P / kPfTileN);
    const uint32_t shared_items = (tokens + kPfTileN - 1) / kPfTileN;
    // x rows as the GEMMs read them: gathered into sorted pair order for the routed items (an item's rows are then
    // one row range of the tensor map), token order for the shared expert; each in its weights' K order
    if ((rc = launch_pack_rows(h, x, false, h->pf_x, nullptr, P, c.d, c.routed_bits, st, h->sorted_pair, c.top_k, tokens))) return rc;
    if (c.shared_f && (rc = launch_pack_rows(h, x, false, h->pf_xn, nullptr, tokens, c.d, c.shared_bits, st))) return rc;

    PrefillGemmParams g{};
    g.experts = static_cast<const uint8_t *>(lv.w.experts); g.stride = lv.w.expert_stride;
    g.num_experts = use_map ? h->n_local : c.num_experts;
    g.off = to_offsets(lv.w.offsets);
    g.work = h->work; g.n_work = h->n_work; g.sorted_pair = h->sorted_pair;
    g.tokens = tokens; g.top_k = c.top_k; g.act = c.activation; g.status = h->status;
    // The shared expert rides in the routed launches (its token tiles after the routed items) when bit width and
    // shapes agree; otherwise it gets launches of its own.
    const bool merged = c.shared_f != 0 && c.shared_bits == c.routed_bits && c.shared_f == c.f;
    const uint32_t none = 0xFFFFFFFFu;
    // gate/up
    g.kdim = c.d;
    g.out = h->acts; g.out_stride = c.f; g.round_gate_up = 0;
    g.s0 = to_mat(lv.w.shared_gate_proj); g.s1 = to_mat(lv.w.shared_up_proj);
    g.out2 = h->shared_act; g.out_stride2 = c.shared_f; g.round_gate_up2 = 1; g.row_scale2 = nullptr;
    g.trace = h->trace_on ? h->trace + ((size_t)layer * 3 + 0) * kTraceWords : nullptr;
    g.shared_from = merged ? max_items : none;
    if ((rc = launch_prefill_gemm<0>(h, c.routed_bits, g, h->pf_x, P, merged ? h->pf_xn : nullptr, tokens,
                                     dim3(c.f / kPfTileM, max_items + (merged ? shared_items : 0)), st)))
        return rc;
    if (c.shared_f && !merged) {
        PrefillGemmParams s = g;
        s.shared_from = 0; s.trace = nullptr;
        if ((rc = launch_prefill_gemm<0>(h, c.shared_bits, s, h->pf_xn, tokens, h->pf_xn, tokens,
                                         dim3(c.shared_f / kPfTileM, shared_items), st)))
            return rc;
    }
    // activation rows as the down GEMMs read them
    const __half *acts16 = h->pf_acts16, *sacts16 = h->pf_sacts16;
    if ((rc = launch_pack_rows(h, h->acts, wide, h->pf_acts16, h->pf_rowscale, P, c.f, c.routed_bits, st))) return rc;
    if (c.shared_f &&
        (rc = launch_pack_rows(h, h->shared_act, wide, h->pf_sacts16, h->pf_srowscale, tokens, c.shared_f, c.shared_bits, st)))
        return rc;
    // down
    g.kdim = c.f; g.row_scale = wide ? h->pf_rowscale : nullptr;
    g.out = h->partial; g.out_stride = c.d;
    g.s0 = to_mat(lv.w.shared_down_proj); g.s1 = g.s0;
    g.out2 = h->shared_partial; g.out_stride2 = c.d; g.row_scale2 = wide ? h->pf_srowscale : nullptr;
    g.trace = h->trace_on ? h->trace + ((size_t)layer * 3 + 1) * kTraceWords : nullptr;
    if ((rc = launch_prefill_gemm<1>(h, c.routed_bits, g, acts16, P, merged ? sacts16 : nullptr, tokens,
                                     dim3(c.d / (2 * kPfTileM), max_items + (merged ? shared_items : 0)), st)))
        return rc;
    if (c.shared_f && !merged) {
        PrefillGemmParams s = g;
        s.shared_from = 0; s.kdim = c.shared_f; s.trace = nullptr;
        if ((rc = launch_prefill_gemm<1>(h, c.shared_bits, s, sacts16, tokens, sacts16, tokens,
                                         dim3(c.d / (2 * kPfTileM), shared_items), st)))
            return rc;
    }
    CombineParams pc{};
    pc.partial = h->partial; pc.shared_partial = c.shared_f ? h->shared_partial : nullptr;
    pc.inv = h->inv; pc.routing_w = w;
    pc.gate_val = (c.shared_f && c.shared_gate_kind != NVMAI_GATE_NONE) ? h->gate_val : nullptr;
    pc.residual = nullptr; pc.y = y; pc.hidden = hidden; pc.D = c.d; pc.K = c.top_k;
    pc.partial_y = mode.partial_y; pc.prefill = mode.decode_order ? 0 : 1;
    pc.hidden_delta = mode.hidden_delta;
    if (mode.decode_order && mode.partial_y == nullptr) pc.next = h->next_norm;
    return dispatch_out(c.out_dtype, [&](auto O) {
        return launch_kernel(h, combine_kernel<decltype(O)::value>, dim3(tokens), dim3(256), 0, st, true, pc);
    });
}

// A batched decode call can take the tensor-core kernels when the fp16 operand holds the centred weight exactly
// (bf16 scales; 8-bit codes go through as two nibbles) and the tile shapes divide the layer.
bool tc_batch_ok(const nvmai_cuda_moe *h, uint32_t tokens, bool with_shared, cudaStream_t st) {
    const auto &c = h->cfg;
    if (tokens < h->tc_min_tokens) return false;
    // with an expert map only the routed-only form is taken (a rank's share of the routed sum); the whole block on
    // a part of the experts is the per-row kernels' business
    if (h->expert_map != nullptr && with_shared) return false;
    if (h->pf_acts16 == nullptr && st != nullptr) {
        // the first such call allocates the packed-row scratch, which a stream under capture does not allow:
        // a call that is being captured before any eager one stays on the per-row kernels
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(st, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) return false;
    }
    if (c.meta_dtype != NVMAI_META_BF16 || c.top_k > (uint32_t)kMaxTopK) return false;
    if (c.f % kPfTileM != 0 || c.d % (2 * kPfTileM) != 0) return false;
    if (with_shared && c.shared_f != 0 && c.shared_f % kPfTileM != 0) return false;
    return true;
}


// ---- one-launch decode step ----------------------------------------------------------
struct PdPlan { uint32_t router_rows = 0, slots = 0, max_tiles = 0; size_t smem = 0; };

// exchange words: logits [E] | shared activations [Fs] | gate [2] | routed activations [K][F] | block output [D]
struct PdXchg {
    size_t logits, sact, gate, acts, y, words;
    explicit PdXchg(const nvmai_cuda_moe_config &c) {
        auto up = [](size_t v) { return (v + 15) & ~(size_t)15; };      // keep every area 128-byte aligned
        size_t o = 0;
        logits = o; o += up(c.num_experts);
        sact = o; o += up(c.shared_f ? c.shared_f : 1);
        gate = o; o += 16;
        acts = o; o += up((size_t)c.top_k * c.f);
        y = o; o += up(c.d);
        words = o;
    }
};

// Can a single-token step of this handle run as one resident kernel?  (Shapes outside these limits take the
// staged kernels.)
bool pd_plan(const nvmai_cuda_moe *h, PdPlan &plan) {
    const auto &c = h->cfg;
    const uint32_t G = (uint32_t)h->sm_count;
    if (G == 0 || h->pd_xchg == nullptr || h->expert_map != nullptr) return false;
    if (c.top_k > (uint32_t)kMaxTopK || c.num_experts > (uint32_t)kPdThreads) return false;
    if (c.shared_f != 0 && c.shared_bits != c.routed_bits) return false;
    if (c.d > (uint32_t)(kPdKeep * kPdNormThreads) || c.d / kTileRows > G) return false;
    if (c.f > 1024 || c.shared_f > 1024) return false;
    // weight tiles come by tiled TMA in 128-byte lines: whole lines per row, and boxes of at most 256 values
    const uint32_t b = c.routed_bits;
    if ((c.d * b / 8) % 128 != 0 || (c.f * b / 8) % 128 != 0 || (c.shared_f * b / 8) % 128 != 0) return false;
    if (kTileFeatures * (c.d / 64) > 256 || kTileRows * (std::max(c.f, c.shared_f) / 64) > 256) return false;
    if (encode_tiled_fn() == nullptr) return false;
    const bool gated = c.shared_f != 0 && c.shared_gate_kind != NVMAI_GATE_NONE;
    // router rows spread over the blocks, one block left without any for the gate row; a shared tile per block
    const uint32_t router_blocks_max = G - (gated ? 1 : 0);
    if (router_blocks_max == 0 || c.shared_f / kTileFeatures > G) return false;
    const uint32_t rows = (c.num_experts + router_blocks_max - 1) / router_blocks_max;
    if (rows > (uint32_t)kPdWarps) return false;
    const uint32_t tiles_total = c.top_k * (c.f / kTileFeatures);
    const uint32_t max_tiles = (tiles_total + G - 1) / G;
    if (max_tiles == 0 || max_tiles > (uint32_t)kPdMaxTiles) return false;
    uint32_t slots = std::min<uint32_t>(max_tiles, kPdMaxSlots);
    const uint32_t min_slots = std::min<uint32_t>(max_tiles, kPdGroups);      // tiles that are worked on side by side
    for (; slots >= min_slots; --slots) {
        const size_t smem = PdLayout(c.d, c.f, c.shared_f, c.routed_bits, c.top_k, c.router_kind,
                                     gated ? c.shared_gate_kind : NVMAI_GATE_NONE, rows, slots, max_tiles).total;
        if (smem <= kMaxSmem) { plan.smem = smem; break; }
    }
    if (slots < min_slots) return false;
    plan.router_rows = rows; plan.slots = slots; plan.max_tiles = max_tiles;
    return true;
}

// One tensor map: `rank` dimensions, dim 0 contiguous; strides in bytes for dims 1.. .
int pd_encode(nvmai_cuda_moe *h, CUtensorMap *map, CUtensorMapDataType dt, uint32_t rank, const void *base,
              const cuuint64_t *gdim, const cuuint64_t *gstride, const cuuint32_t *box, bool swizzle) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return NVMAI_CUDA_ECUDA;
    const cuuint32_t estride[5] = {1, 1, 1, 1, 1};
    const CUresult r = enc(map, dt, rank, const_cast<void *>(base), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { h->last_cuda_error = (int)r; return NVMAI_CUDA_ECUDA; }
    return NVMAI_CUDA_OK;
}

// The per-layer table of the resident kernel: tensor maps over the layer's expert array (the expert is a coordinate)
// and the plain pointers.  NVMAI_CUDA_EINVAL when a layer's blob layout is not the regular one the maps describe.
int pd_build_layers(nvmai_cuda_moe *h, std::vector<PdLayer> &host) {
    const auto &c = h->cfg;
    const uint64_t bits = c.routed_bits;
    const uint64_t rbd = (uint64_t)c.d * bits / 8, rbf = (uint64_t)c.f * bits / 8, rbs = (uint64_t)c.shared_f * bits / 8;
    const uint64_t gd = c.d / 64, gf = c.f / 64;
    host.assign(c.num_layers, PdLayer{});
    const uint64_t n_blobs = h->expert_map ? h->n_local : c.num_experts;      // blobs this rank holds, in local-index order
    for (uint32_t l = 0; l < c.num_layers; ++l) {
        const auto &w = h->layers[l].w;
        const auto &o = w.offsets;
        PdLayer &d = host[l];
        const uint8_t *base = static_cast<const uint8_t *>(w.experts);
        // gate and up must be laid out alike, scales before biases (the repacker's order, RepackPlanner.swift:365-426)
        if (w.expert_stride == 0 || o.up_w <= o.gate_w || o.up_s <= o.gate_s || o.gate_b <= o.gate_s || o.down_b <= o.down_s ||
            o.up_s - o.gate_s != o.up_b - o.gate_b)
            return NVMAI_CUDA_EINVAL;
        int rc;
        {   // routed gate + up codes: {128 B, row, chunk, gate|up, expert}
            const cuuint64_t gdim[5] = {128, c.f, rbd / 128, 2, n_blobs};
            const cuuint64_t gstr[4] = {rbd, 128, (cuuint64_t)(o.up_w - o.gate_w), w.expert_stride};
            const cuuint32_t box[5] = {128, (cuuint32_t)kTileFeatures, (cuuint32_t)(rbd / 128), 2, 1};
            if ((rc = pd_encode(h, &d.gu_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 5, base + o.gate_w, gdim, gstr, box, true))) return rc;
        }
        {   // their scales and biases: {value, gate|up, scale|bias, expert}
            const cuuint64_t gdim[4] = {(cuuint64_t)c.f * gd, 2, 2, n_blobs};
            const cuuint64_t gstr[3] = {(cuuint64_t)(o.up_s - o.gate_s), (cuuint64_t)(o.gate_b - o.gate_s), w.expert_stride};
            const cuuint32_t box[4] = {(cuuint32_t)(kTileFeatures * gd), 2, 2, 1};
            if ((rc = pd_encode(h, &d.gu_meta, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, base + o.gate_s, gdim, gstr, box, false))) return rc;
        }
        {   // routed down codes: {128 B, row, chunk, expert}
            const cuuint64_t gdim[4] = {128, c.d, rbf / 128, n_blobs};
            const cuuint64_t gstr[3] = {rbf, 128, w.expert_stride};
            const cuuint32_t box[4] = {128, (cuuint32_t)kTileRows, (cuuint32_t)(rbf / 128), 1};
            if ((rc = pd_encode(h, &d.dn_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, base + o.down_w, gdim, gstr, box, true))) return rc;
        }
        {   // and meta: {value, scale|bias, expert}
            const cuuint64_t gdim[3] = {(cuuint64_t)c.d * gf, 2, n_blobs};
            const cuuint64_t gstr[2] = {(cuuint64_t)(o.down_b - o.down_s), w.expert_stride};
            const cuuint32_t box[3] = {(cuuint32_t)(kTileRows * gf), 2, 1};
            if ((rc = pd_encode(h, &d.dn_meta, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, base + o.down_s, gdim, gstr, box, false))) return rc;
        }
        if (c.shared_f) {   // the shared expert's three code matrices: {128 B, row, chunk}
            const cuuint64_t gdim[3] = {128, c.shared_f, rbd / 128};
            const cuuint64_t gstr[2] = {rbd, 128};
            const cuuint32_t box[3] = {128, (cuuint32_t)kTileFeatures, (cuuint32_t)(rbd / 128)};
            if ((rc = pd_encode(h, &d.sg_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, w.shared_gate_proj.w, gdim, gstr, box, true))) return rc;
            if ((rc = pd_encode(h, &d.su_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, w.shared_up_proj.w, gdim, gstr, box, true))) return rc;
            const cuuint64_t ddim[3] = {128, c.d, rbs / 128};
            const cuuint64_t dstr[2] = {rbs, 128};
            const cuuint32_t dbox[3] = {128, (cuuint32_t)kTileRows, (cuuint32_t)(rbs / 128)};
            if ((rc = pd_encode(h, &d.sd_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, w.shared_down_proj.w, ddim, dstr, dbox, true))) return rc;
        }
        d.experts_stride = w.expert_stride;
        d.rW = static_cast<const uint8_t *>(w.router.w);
        d.rS = static_cast<const uint16_t *>(w.router.scales);
        d.rB = static_cast<const uint16_t *>(w.router.biases);
        d.eff = static_cast<const uint16_t *>(w.effective_scale);
        d.pes = static_cast<const uint16_t *>(w.per_expert_scale);
        d.sgS = static_cast<const uint16_t *>(w.shared_gate_proj.scales); d.sgB = static_cast<const uint16_t *>(w.shared_gate_proj.biases);
        d.suS = static_cast<const uint16_t *>(w.shared_up_proj.scales); d.suB = static_cast<const uint16_t *>(w.shared_up_proj.biases);
        d.sdS = static_cast<const uint16_t *>(w.shared_down_proj.scales); d.sdB = static_cast<const uint16_t *>(w.shared_down_proj.biases);
        d.gW = static_cast<const uint8_t *>(w.shared_gate.w);
        d.gS = static_cast<const uint16_t *>(w.shared_gate.scales);
        d.gB = static_cast<const uint16_t *>(w.shared_gate.biases);
    }
    return NVMAI_CUDA_OK;
}

// Uploads the layer table when a layer was (re)registered.  pd_unavailable: the layout does not fit the maps.
int pd_prepare(nvmai_cuda_moe *h, cudaStream_t st) {
    if (!h->pd_layers_stale) return h->pd_unavailable ? NVMAI_CUDA_EINVAL : NVMAI_CUDA_OK;
    std::vector<PdLayer> host;
    int rc = pd_build_layers(h, host);
    h->pd_layers_stale = false;
    h->pd_unavailable = rc != NVMAI_CUDA_OK;
    if (rc) return rc;
    if ((rc = record(h, cudaMemcpyAsync(h->pd_layers, host.data(), host.size() * sizeof(PdLayer), cudaMemcpyHostToDevice, st)))) return rc;
    return record(h, cudaStreamSynchronize(st));     // `host` goes out of scope
}

int pd_launch(nvmai_cuda_moe *h, const PdPlan &plan, const __half *x0, void *y_last, cudaStream_t st) {
    const auto &c = h->cfg;
    const PdXchg X(c);
    const bool gated = c.shared_f != 0 && c.shared_gate_kind != NVMAI_GATE_NONE;
    PdParams p{};
    p.layers = h->pd_layers; p.num_layers = c.num_layers;
    p.x0 = x0; p.y_last = y_last;
    p.xlogits = h->pd_xchg + X.logits; p.xsact = h->pd_xchg + X.sact; p.xgate = h->pd_xchg + X.gate;
    p.xacts = h->pd_xchg + X.acts; p.xy = h->pd_xchg + X.y;
    p.epoch = h->pd_epoch; p.status = h->status; p.route_log = h->pd_route_log;
    h->pd_route_rows = 1;
    p.D = c.d; p.F = c.f; p.E = c.num_experts; p.K = c.top_k; p.act = c.activation; p.shared_f = c.shared_f;
    p.router_kind = c.router_kind; p.gate_kind = gated ? c.shared_gate_kind : NVMAI_GATE_NONE;
    p.router_rows = plan.router_rows; p.slots = plan.slots; p.max_tiles = plan.max_tiles;
    p.debug_mute_block = h->pd_mute_block;
    p.trace = h->trace_on ? h->pd_trace : nullptr;
    return dispatch_bits_meta(c.routed_bits, c.meta_dtype, [&](auto B, auto M) {
        return dispatch_out(c.out_dtype, [&](auto O) {
            auto kern = persistent_decode_kernel<decltype(B)::value, decltype(M)::value, decltype(O)::value>;
            cudaError_t e = ensure_smem(kern, plan.smem);
            if (e != cudaSuccess) return record(h, e);
            cudaLaunchConfig_t cfg{};
            cfg.gridDim = dim3((unsigned)h->sm_count);
            cfg.blockDim = dim3(kPdThreads);
            cfg.dynamicSmemBytes = plan.smem;
            cfg.stream = st;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeCooperative;      // every block resident: they wait on one another
            attr[0].val.cooperative = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            e = cudaLaunchKernelEx(&cfg, kern, p);
            g_launches.fetch_add(1, std::memory_order_relaxed);
            return record(h, e);
        });
    });
}


// ---- the resident kernel for 2..8 rows and for experts spread over ranks -----------------
// exchange words: logits [T][E] | shared activations [T][Fs] | gate [16] | routed activations [64][F] | block
// output [T][D] | one word per block
struct PbXchg {
    size_t logits, sact, gate, acts, y, beat, words;
    PbXchg(const nvmai_cuda_moe_config &c, uint32_t T, uint32_t blocks) {
        auto up = [](size_t v) { return (v + 15) & ~(size_t)15; };
        size_t o = 0;
        logits = o; o += up((size_t)T * c.num_experts);
        sact = o; o += up((size_t)T * (c.shared_f ? c.shared_f : 1));
        gate = o; o += 16;
        acts = o; o += up((size_t)kPbMaxPairs * c.f);
        y = o; o += up((size_t)T * c.d);
        beat = o; o += up(blocks);
        words = o;
    }
};

struct PbPlan { uint32_t router_rows = 0, slots = 0; size_t smem = 0; };

bool pb_plan(const nvmai_cuda_moe *h, uint32_t T, PbPlan &plan) {
    const auto &c = h->cfg;
    const uint32_t G = (uint32_t)h->sm_count;
    if (G == 0 || h->pb_xchg == nullptr || T == 0 || T > (uint32_t)kPbMaxRows || T > c.max_tokens) return false;
    if (c.top_k > (uint32_t)kMaxTopK || c.num_experts > (uint32_t)kMaxExperts) return false;
    if (c.shared_f != 0 && c.shared_bits != c.routed_bits) return false;
    if (c.d / kTileRows > G || c.d > (uint32_t)(kPdKeep * kPbThreads)) return false;
    if (c.f > 1024 || c.shared_f > 1024) return false;
    const uint32_t b = c.routed_bits;
    if ((c.d * b / 8) % 128 != 0 || (c.f * b / 8) % 128 != 0 || (c.shared_f * b / 8) % 128 != 0) return false;
    if (kTileFeatures * (c.d / 64) > 256 || kTileRows * (std::max(c.f, c.shared_f) / 64) > 256) return false;
    if (T * kTileRows > (uint32_t)kPbThreads / 2 || encode_tiled_fn() == nullptr) return false;
    const bool gated = c.shared_f != 0 && c.shared_gate_kind != NVMAI_GATE_NONE;
    const uint32_t router_blocks_max = G - (gated ? 1 : 0);
    if (router_blocks_max == 0 || c.shared_f / kTileFeatures > G) return false;
    const uint32_t rows = (c.num_experts + router_blocks_max - 1) / router_blocks_max;
    if (rows > (uint32_t)kPbWarps) return false;
    for (uint32_t slots = kPdMaxSlots; slots >= 1; --slots) {
        const size_t smem = PbLayout(c.d, c.f, c.shared_f, c.routed_bits, T, c.router_kind,
                                     gated ? c.shared_gate_kind : NVMAI_GATE_NONE, rows, slots).total;
        if (smem <= kMaxSmem) { plan.router_rows = rows; plan.slots = slots; plan.smem = smem; return true; }
    }
    return false;
}

// world == 1: every expert is local (or the handle's map says which are, for tests); world > 1: recv[r] = rank r's
// receive area as mapped in this process.
int pb_launch(nvmai_cuda_moe *h, const PbPlan &plan, const __half *x_all, uint32_t T, void *y_all, uint32_t rank, uint32_t world,
              unsigned long long *const *recv, cudaStream_t st, unsigned long long *const *xin = nullptr,
              const __half *x_own = nullptr, void *y_own = nullptr, uint32_t rows_own = 1) {
    const auto &c = h->cfg;
    const PbXchg X(c, kPbMaxRows, (uint32_t)h->sm_count);
    const bool gated = c.shared_f != 0 && c.shared_gate_kind != NVMAI_GATE_NONE;
    PbParams p{};
    p.layers = h->pd_layers; p.num_layers = c.num_layers; p.T = T;
    p.x0 = x_all; p.y_last = y_all;
    p.xlogits = h->pb_xchg + X.logits; p.xsact = h->pb_xchg + X.sact; p.xgate = h->pb_xchg + X.gate;
    p.xacts = h->pb_xchg + X.acts; p.xy = h->pb_xchg + X.y; p.xbeat = h->pb_xchg + X.beat;
    p.expert_map = h->expert_map;
    p.rank = rank; p.world = world;
    for (uint32_t r = 0; r < world && r < (uint32_t)kEpMaxRanks; ++r) {
        p.recv[r] = recv ? recv[r] : nullptr;
        p.xin[r] = xin ? xin[r] : nullptr;
    }
    p.x_own = x_own; p.y_own = y_own; p.rows_own = rows_own ? rows_own : 1;
    p.epoch = h->pd_epoch; p.status = h->status; p.route_log = h->pd_route_log;
    h->pd_route_rows = T;
    p.trace = h->trace_on ? h->pd_trace : nullptr;
    p.D = c.d; p.F = c.f; p.E = c.num_experts; p.K = c.top_k; p.act = c.activation; p.shared_f = c.shared_f;
    p.router_kind = c.router_kind; p.gate_kind = gated ? c.shared_gate_kind : NVMAI_GATE_NONE;
    p.router_rows = plan.router_rows; p.slots = plan.slots;
    return dispatch_bits_meta(c.routed_bits, c.meta_dtype, [&](auto B, auto M) {
        return dispatch_out(c.out_dtype, [&](auto O) {
            auto kern = persistent_batch_kernel<decltype(B)::value, decltype(M)::value, decltype(O)::value>;
            cudaError_t e = ensure_smem(kern, plan.smem);
            if (e != cudaSuccess) return record(h, e);
            cudaLaunchConfig_t cfg{};
            cfg.gridDim = dim3((unsigned)h->sm_count);
            cfg.blockDim = dim3(kPbThreads);
            cfg.dynamicSmemBytes = plan.smem;
            cfg.stream = st;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeCooperative;
            attr[0].val.cooperative = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            e = cudaLaunchKernelEx(&cfg, kern, p);
            g_launches.fetch_add(1, std::memory_order_relaxed);
            return record(h, e);
        });
    });
}

}  // namespace

// ------------------------------------------------------------------------------
// exported functions
// ------------------------------------------------------------------------------

extern "C" {

uint64_t nvmai_cuda_moe_expert_offsets(uint32_t d, uint32_t f, uint32_t bits, nvmai_expert_offsets *out) {
    const uint64_t gate_w = (uint64_t)f * d * bits / 8, gate_m = (uint64_t)f * (d / 64) * 2;
    const uint64_t down_w = (uint64_t)d * f * bits / 8, down_m = (uint64_t)d * (f / 64) * 2;
    uint64_t o = 0;
    nvmai_expert_offsets r;
    r.gate_w = (uint32_t)o; o += gate_w;
    r.gate_s = (uint32_t)o; o += gate_m;
    r.gate_b = (uint32_t)o; o += gate_m;
    r.up_w = (uint32_t)o; o += gate_w;
    r.up_s = (uint32_t)o; o += gate_m;
    r.up_b = (uint32_t)o; o += gate_m;
    r.down_w = (uint32_t)o; o += down_w;
    r.down_s = (uint32_t)o; o += down_m;
    r.down_b = (uint32_t)o; o += down_m;
    if (out) *out = r;
    return o;
}

nvmai_cuda_moe *nvmai_cuda_moe_create(const nvmai_cuda_moe_config *config, int *out_err) {
    auto fail = [&](int code) -> nvmai_cuda_moe * { if (out_err) *out_err = code; return nullptr; };
    if (!config) return fail(NVMAI_CUDA_EINVAL);
    const nvmai_cuda_moe_config &c = *config;
    // MoE.swift:163-165 and SharedExpertInt4.swift:40-45, as error codes
    if (c.d == 0 || c.d % 64 != 0 || c.f == 0 || c.f % 64 != 0 || c.shared_f % 64 != 0) return fail(NVMAI_CUDA_EINVAL);
    if (c.num_experts == 0 || c.num_experts > (uint32_t)kMaxExperts) return fail(NVMAI_CUDA_ERANGE);
    if (c.top_k == 0 || c.top_k > 32 || c.top_k > c.num_experts) return fail(NVMAI_CUDA_ERANGE);
    if (!valid_bits(c.routed_bits) || (c.shared_f && !valid_bits(c.shared_bits))) return fail(NVMAI_CUDA_EINVAL);
    if (c.router_kind != NVMAI_ROUTER_DENSE_F16 && c.router_kind != NVMAI_ROUTER_AFFINE4 &&
        c.router_kind != NVMAI_ROUTER_AFFINE8) return fail(NVMAI_CUDA_EINVAL);
    if (c.shared_gate_kind != NVMAI_GATE_NONE && c.shared_gate_kind != NVMAI_ROUTER_DENSE_F16 &&
        c.shared_gate_kind != NVMAI_ROUTER_AFFINE4 && c.shared_gate_kind != NVMAI_ROUTER_AFFINE8)
        return fail(NVMAI_CUDA_EINVAL);
    if (c.meta_dtype > NVMAI_META_FP16 || c.activation > NVMAI_ACT_GELU_TANH || c.out_dtype > NVMAI_OUT_FP32)
        return fail(NVMAI_CUDA_EINVAL);
    if (c.max_tokens == 0 || c.num_layers == 0) return fail(NVMAI_CUDA_EINVAL);
    // every block stages its weight tile in shared memory: the tile must fit
    {
        size_t need = GateUpLayout(c.d, c.routed_bits).total;
        need = std::max(need, std::max(RowsLayout(c.d, c.router_kind).total, kTopkSmemBytes));
        if (c.shared_f) need = std::max(need, GateUpLayout(c.d, c.shared_bits).total);
        const uint32_t warps = (c.top_k < (uint32_t)kMaxTopK ? c.top_k : (uint32_t)kMaxTopK) + (c.shared_f ? 1 : 0);
        need = std::max(need, DownLayout(c.f, c.shared_f, c.routed_bits, c.shared_bits, warps).total);
        {
            need = std::max(need, GroupedGateUpLayout(c.d, c.routed_bits).total);
            if (c.shared_f) need = std::max(need, GroupedGateUpLayout(c.d, c.shared_bits).total);
            need = std::max(need, GroupedDownLayout(c.f, c.shared_f, c.routed_bits, c.shared_bits).total);
        }
        if (need > kMaxSmem) return fail(NVMAI_CUDA_ERANGE);
    }

    nvmai_cuda_moe *h = new (std::nothrow) nvmai_cuda_moe();
    if (!h) return fail(NVMAI_CUDA_ENOMEM);
    h->cfg = c;
    h->layers.resize(c.num_layers);
    if (const char *env = std::getenv("NVMAI_CUDA_L2_PREFETCH")) h->l2_prefetch = env[0] == '1';
    if (const char *env = std::getenv("NVMAI_CUDA_PREFILL_TC")) h->prefill_tc = env[0] != '0';
    if (const char *env = std::getenv("NVMAI_CUDA_GROUPED_MIN")) h->grouped_min_tokens = (uint32_t)std::max(1, std::atoi(env));
    if (const char *env = std::getenv("NVMAI_CUDA_TC_MIN")) h->tc_min_tokens = (uint32_t)std::max(1, std::atoi(env));
    const size_t T = c.max_tokens;
    auto alloc = [&](auto **ptr, size_t bytes) -> bool {
        cudaError_t e = cudaMalloc(reinterpret_cast<void **>(ptr), bytes ? bytes : 16);
        if (e != cudaSuccess) { h->last_cuda_error = (int)e; return false; }
        return true;
    };
    bool ok = alloc(&h->logits, T * c.num_experts * sizeof(float)) && alloc(&h->idx, T * c.top_k * 4) &&
              alloc(&h->w, T * c.top_k * 2) && alloc(&h->acts, T * c.top_k * c.f * out_size(c.out_dtype)) &&
              alloc(&h->shared_act, T * (c.shared_f ? c.shared_f : 8) * out_size(c.out_dtype)) &&
              alloc(&h->gate_val, T * 4) &&
              alloc(&h->y, T * c.d * out_size(c.out_dtype)) && alloc(&h->xnorm, T * c.d * 2) &&
              alloc(&h->counter, (T / 8 + 2) * 4) && alloc(&h->row_counter, T * 4) && alloc(&h->status, 64) && alloc(&h->stage_x, T * c.d * 2) &&
              alloc(&h->stage_y, T * c.d * out_size(c.out_dtype));
    if (ok) ok = cudaMemset(h->counter, 0, (T / 8 + 2) * 4) == cudaSuccess && cudaMemset(h->status, 0, 64) == cudaSuccess &&
                 cudaMemset(h->row_counter, 0, T * 4) == cudaSuccess;
    {
        const size_t P = T * c.top_k;
        h->max_work = (uint32_t)(std::min(P, c.num_experts + P / kPairsPerItem) + (T + kPairsPerItem - 1) / kPairsPerItem);
        if (ok) ok = alloc(&h->sorted_pair, P * 4) && alloc(&h->inv, P * 4) && alloc(&h->expert_offsets, kMaxExperts * 4) &&
                     alloc(&h->expert_counts, kMaxExperts * 4) && alloc(&h->work, (size_t)h->max_work * sizeof(WorkItem)) &&
                     alloc(&h->n_work, 16) && alloc(&h->group_hist, ((P + kGroupThreads - 1) / kGroupThreads) * kMaxExperts * 4) && alloc(&h->trace, (size_t)c.num_layers * 3 * kTraceWords * sizeof(unsigned long long));
        // per-pair partial rows are only needed by the batched path
        if (ok)
            ok = alloc(&h->partial, P * c.d * sizeof(float)) && alloc(&h->shared_partial, T * c.d * sizeof(float));
    }
    if (ok) {     // the one-launch decode step: exchange words (zeroed: tag 0 is never used), epoch word, layer table
        int dev = 0;
        const size_t xbytes = PdXchg(c).words * sizeof(unsigned long long);
        const unsigned int first_epoch = 1;
        ok = cudaGetDevice(&dev) == cudaSuccess &&
             cudaDeviceGetAttribute(&h->sm_count, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess &&
             alloc(&h->pd_xchg, xbytes) && alloc(&h->pd_epoch, 5 * 128) &&
             alloc(&h->pb_xchg, PbXchg(c, kPbMaxRows, (uint32_t)std::max(h->sm_count, 1)).words * sizeof(unsigned long long)) &&
             cudaMemset(h->pb_xchg, 0, PbXchg(c, kPbMaxRows, (uint32_t)std::max(h->sm_count, 1)).words * sizeof(unsigned long long)) == cudaSuccess && alloc(&h->pd_layers, (size_t)c.num_layers * sizeof(PdLayer)) &&
             alloc(&h->pd_route_log, (size_t)c.num_layers * kPbMaxRows * c.top_k * 4) &&
             cudaMemset(h->pd_xchg, 0, xbytes) == cudaSuccess && cudaMemset(h->pd_epoch, 0, 5 * 128) == cudaSuccess &&
             cudaMemset(h->pd_route_log, 0, (size_t)c.num_layers * kPbMaxRows * c.top_k * 4) == cudaSuccess &&
             cudaMemcpy(h->pd_epoch, &first_epoch, sizeof(first_epoch), cudaMemcpyHostToDevice) == cudaSuccess;
    }
    if (const char *env = std::getenv("NVMAI_CUDA_DECODE_MODE")) h->decode_mode = std::atoi(env);
    if (!ok) {
        const bool oom = h->last_cuda_error == (int)cudaErrorMemoryAllocation;
        nvmai_cuda_moe_destroy(h);
        cudaGetLastError();
        return fail(oom ? NVMAI_CUDA_ENOMEM : NVMAI_CUDA_ECUDA);
    }
    if (out_err) *out_err = NVMAI_CUDA_OK;
    return h;
}

void nvmai_cuda_moe_destroy(nvmai_cuda_moe *h) {
    if (!h) return;
    for (auto &kv : h->stack_graphs) cudaGraphExecDestroy(kv.second);
    ep_release(h);
    cudaFree(h->pd_trace);
    cudaFree(h->pb_xchg);
    cudaFree(h->pd_layers); cudaFree(h->pd_xchg); cudaFree(h->pd_epoch); cudaFree(h->pd_route_log);
    cudaFree(h->pf_x); cudaFree(h->pf_xn); cudaFree(h->pf_acts16); cudaFree(h->pf_sacts16); cudaFree(h->pf_rowscale); cudaFree(h->pf_srowscale);
    for (auto &lv : h->layers)
        for (void *p : lv.owned) cudaFree(p);
    cudaFree(h->logits); cudaFree(h->idx); cudaFree(h->w); cudaFree(h->acts); cudaFree(h->shared_act);
    cudaFree(h->gate_val); cudaFree(h->y); cudaFree(h->xnorm); cudaFree(h->counter); cudaFree(h->status);
    cudaFree(h->stage_x); cudaFree(h->stage_y); cudaFree(h->row_counter);
    cudaFree(h->sorted_pair); cudaFree(h->inv); cudaFree(h->expert_offsets); cudaFree(h->expert_counts);
    cudaFree(h->work); cudaFree(h->n_work); cudaFree(h->group_hist); cudaFree(h->trace); cudaFree(h->expert_map); cudaFree(h->partial); cudaFree(h->shared_partial);
    delete h;
}

int nvmai_cuda_moe_register_layer(nvmai_cuda_moe *h, uint32_t layer, const nvmai_cuda_moe_layer *wts_in) {
    if (!h || !wts_in) return NVMAI_CUDA_EINVAL;
    if (layer >= h->layers.size()) return NVMAI_CUDA_ERANGE;
    const auto &c = h->cfg;
    nvmai_cuda_moe_layer copy = *wts_in;
    nvmai_cuda_moe_layer *wts = &copy;
    if (!wts->experts || !aligned16(wts->experts) || (wts->expert_stride & 15u)) return NVMAI_CUDA_EINVAL;
    int rc = check_offsets(c, wts->offsets, wts->expert_stride);
    if (rc) return rc;
    // The resident tensors (router, shared expert, gate row, input scale) sit back to back in the reference's weight
    // file with no alignment (RepackPlanner.swift:310-316; its kernels are tested on a base that is off by two bytes,
    // DequantInt4GEMVTests.swift:114-121), while the bulk copies here want 16-byte aligned sources: a tensor whose base
    // is not aligned is copied once, at registration, into an aligned buffer the handle owns (a few MB per layer).
    // The expert blobs are never copied: their base and stride must be aligned.
    std::vector<void *> owned;
    auto fail = [&](int code) {
        for (void *p : owned) cudaFree(p);
        return code;
    };
    auto realign = [&](const void *&ptr, size_t bytes) -> int {
        if (ptr == nullptr || aligned16(ptr)) return NVMAI_CUDA_OK;
        if (reinterpret_cast<uintptr_t>(ptr) & 1u) return NVMAI_CUDA_EINVAL;       // 16-bit elements at an odd address
        void *buf = nullptr;
        if (cudaMalloc(&buf, (bytes + 15) & ~(size_t)15) != cudaSuccess) { cudaGetLastError(); return NVMAI_CUDA_ENOMEM; }
        owned.push_back(buf);
        int r = record(h, cudaMemcpy(buf, ptr, bytes, cudaMemcpyDeviceToDevice));
        ptr = buf;
        return r;
    };
    // kind_or_bits: 0 = dense fp16 rows, else the code width of an affine tensor [rows][n]
    auto tensor = [&](nvmai_affine_tensor &t, uint32_t kind_or_bits, size_t rows, size_t n) -> int {
        if (!t.w) return NVMAI_CUDA_EINVAL;
        int r = realign(t.w, kind_or_bits == 0 ? rows * n * 2 : rows * n * kind_or_bits / 8);
        if (r || kind_or_bits == 0) return r;
        if (!t.scales || !t.biases) return NVMAI_CUDA_EINVAL;
        if ((r = realign(t.scales, rows * (n / kGroup) * 2))) return r;
        return realign(t.biases, rows * (n / kGroup) * 2);
    };
    if ((rc = tensor(wts->router, c.router_kind, c.num_experts, c.d))) return fail(rc);
    if (c.shared_f) {
        if ((rc = tensor(wts->shared_gate_proj, c.shared_bits, c.shared_f, c.d)) ||
            (rc = tensor(wts->shared_up_proj, c.shared_bits, c.shared_f, c.d)) ||
            (rc = tensor(wts->shared_down_proj, c.shared_bits, c.d, c.shared_f)))
            return fail(rc);
        if (c.shared_gate_kind != NVMAI_GATE_NONE && (rc = tensor(wts->shared_gate, c.shared_gate_kind, 1, c.d))) return fail(rc);
    }
    if ((rc = realign(wts->effective_scale, (size_t)c.d * 2))) return fail(rc);
    for (void *p : h->layers[layer].owned) cudaFree(p);       // copies made for an earlier registration of this layer
    h->layers[layer].owned = std::move(owned);
    h->layers[layer].w = *wts;
    h->layers[layer].registered = true;
    h->graphs_stale = h->ep_graphs_stale = true;
    h->pd_layers_stale = true;
    return NVMAI_CUDA_OK;
}

int nvmai_cuda_moe_router(nvmai_cuda_moe *h, uint32_t layer, const void *x_f16, uint32_t x_stride, uint32_t tokens,
                          uint32_t *out_idx, void *out_w_f16, void *stream) {
    NvtxRange nvtx_range("attn_tail_router");
    int rc = check_layer(h, layer);
    if (rc) return rc;
    if (!x_f16 || !out_idx || !out_w_f16 || !aligned16(x_f16)) return NVMAI_CUDA_EINVAL;
    if (tokens == 0 || tokens > h->cfg.max_tokens) return NVMAI_CUDA_ERANGE;
    if (x_stride < h->cfg.d || (x_stride % 8) != 0) return NVMAI_CUDA_EINVAL;   // PrefillRouter.swift:68
    const XSource xsrc{static_cast<const __half *>(x_f16), x_stride, nullptr, nullptr};
    return launch_stage1(h, h->layers[layer], xsrc, tokens, out_idx, static_cast<__half *>(out_w_f16), true, false,
                         false, false, static_cast<cudaStream_t>(stream));
}

int nvmai_cuda_moe_shared_expert(nvmai_cuda_moe *h, uint32_t layer, const void *x_f16, uint32_t x_stride,
                                 uint32_t tokens, void *h1, void *stream) {
    NvtxRange nvtx_range("shared_expert");
    int rc = check_layer(h, layer);
    if (rc) return rc;
    const auto &c = h->cfg;
    if (c.shared_f == 0 || !x_f16 || !h1 || !aligned16(x_f16)) return NVMAI_CUDA_EINVAL;
    if (tokens == 0 || tokens > c.max_tokens) return NVMAI_CUDA_ERANGE;
    if (x_stride < c.d || (x_stride % 8) != 0) return NVMAI_CUDA_EINVAL;
    const XSource xsrc{static_cast<const __half *>(x_f16), x_stride, nullptr, nullptr};
    return shared_expert_impl(h, h->layers[layer], xsrc, tokens, h1, static_cast<cudaStream_t>(stream));
}

int nvmai_cuda_moe_routed_phase1(nvmai_cuda_moe *h, const void *const *blobs_host,
                                 const nvmai_expert_offsets *offsets, const void *x_f16, void *acts_f16,
                                 const uint32_t *active_slots_host, uint32_t active_count, void *stream) {
    NvtxRange nvtx_range("moe_phase1_hit");
    if (!h || !blobs_host || !offsets || !x_f16 || !acts_f16 || !aligned16(x_f16)) return NVMAI_CUDA_EINVAL;
    const auto &c = h->cfg;
    if (c.top_k != (uint32_t)kMaxTopK) return NVMAI_CUDA_EINVAL;     // MoE.swift:442-445
    int rc = check_offsets(c, *offsets, 0);
    if (rc) return rc;
    for (uint32_t k = 0; k < c.top_k; ++k)
        if (!blobs_host[k] || !aligned16(blobs_host[k])) return NVMAI_CUDA_EINVAL;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint32_t *slots_dev = nullptr;
    uint32_t n_slots = c.top_k;
    if (active_slots_host != nullptr) {
        if (active_count == 0) return NVMAI_CUDA_OK;                 // MoE.swift:356
        if (active_count > c.top_k) return NVMAI_CUDA_ERANGE;
        // the slot list rides in the idx scratch (8 x u32), like the runner's moeMissActiveSlots buffer
        rc = record(h, cudaMemcpyAsync(h->idx, active_slots_host, active_count * 4, cudaMemcpyHostToDevice, st));
        if (rc) return rc;
        slots_dev = h->idx;
        n_slots = active_count;
    }
    return launch_stage2(h, source_from_blobs(blobs_host, c.top_k), to_offsets(*offsets),
                         static_cast<const __half *>(x_f16), c.d, 1, acts_f16, slots_dev, n_slots, false, st);
}

int nvmai_cuda_moe_routed_phase2(nvmai_cuda_moe *h, const void *const *blobs_host,
                                 const nvmai_expert_offsets *offsets, const void *acts_f16,
                                 const void *routing_w_f16, const void *residual, void *y, void *stream) {
    NvtxRange nvtx_range("moe_phase2_reduce");
    if (!h || !blobs_host || !offsets || !acts_f16 || !routing_w_f16 || !residual || !y) return NVMAI_CUDA_EINVAL;
    if (!aligned16(acts_f16)) return NVMAI_CUDA_EINVAL;
    const auto &c = h->cfg;
    if (c.top_k != (uint32_t)kMaxTopK) return NVMAI_CUDA_EINVAL;
    int rc = check_offsets(c, *offsets, 0);
    if (rc) return rc;
    for (uint32_t k = 0; k < c.top_k; ++k)
        if (!blobs_host[k] || !aligned16(blobs_host[k])) return NVMAI_CUDA_EINVAL;
    Stage3Params p{};
    p.src = source_from_blobs(blobs_host, c.top_k);
    p.off = to_offsets(*offsets);
    p.acts = acts_f16;
    p.routing_w = static_cast<const __half *>(routing_w_f16);
    p.residual = residual;
    p.y = y;
    p.top_k = c.top_k;
    return launch_stage3(h, p, 1, false, static_cast<cudaStream_t>(stream));
}

int nvmai_cuda_moe_layer_decode(nvmai_cuda_moe *h, uint32_t layer, const void *x_f16, uint32_t tokens,
                                void *hidden_inout, void *h2_out, uint32_t *out_idx, void *out_w_f16, void *stream) {
    NvtxRange nvtx_range("moe_phase1_2_routed");
    int rc = check_layer(h, layer);
    if (rc) return rc;
    if (!x_f16 || !aligned16(x_f16)) return NVMAI_CUDA_EINVAL;
    if (tokens == 0 || tokens > h->cfg.max_tokens) return NVMAI_CUDA_ERANGE;
    if (h->cfg.top_k > (uint32_t)kMaxTopK) return NVMAI_CUDA_EINVAL;
    if (tc_batch_ok(h, tokens, true, static_cast<cudaStream_t>(stream))) {
        PrefillMode mode;
        mode.decode_order = true;
        return layer_prefill_impl(h, layer, static_cast<const __half *>(x_f16), tokens, hidden_inout, h2_out, out_idx,
                                  static_cast<__half *>(out_w_f16), static_cast<cudaStream_t>(stream), mode);
    }
    const XSource xsrc{static_cast<const __half *>(x_f16), h->cfg.d, nullptr, nullptr};
    return layer_decode_impl(h, layer, xsrc, static_cast<const __half *>(x_f16), tokens, hidden_inout, h2_out,
                             out_idx, static_cast<__half *>(out_w_f16), static_cast<cudaStream_t>(stream));
}

// Width-2 verification (RealForwardRunner.swift:3016-3235): the decode block's rounding order for two rows.  Here
// the two rows share one launch of each stage, and a blob that both rows selected is read from HBM once and served
// to the second row's blocks by the L2.
int nvmai_cuda_moe_layer_verify_pair(nvmai_cuda_moe *h, uint32_t layer, const void *x_f16, void *hidden_inout,
                                     void *h2_out, uint32_t *out_idx, void *out_w_f16, void *stream) {
    NvtxRange nvtx_range("verify_routed_pair");
    int rc = check_layer(h, layer);
    if (rc) return rc;
    if (h->cfg.max_tokens < 2) return NVMAI_CUDA_ERANGE;
    return nvmai_cuda_moe_layer_decode(h, layer, x_f16, 2, hidden_inout, h2_out, out_idx, out_w_f16, stream);
}

// The block together with the two steps the runner encodes in front of it (RealForwardRunner.swift:1900-1909):
// stage 1 derives x = rmsnorm_bf16w(out(hidden + delta)) in every block (block 0 stores the rows for stage 2), the
// last stage writes hidden = out(out(hidden + delta) + h2); nothing writes the hidden state before that, so no block
// can read a half-updated row.
int nvmai_cuda_moe_layer_decode_prenorm(nvmai_cuda_moe *h, uint32_t layer, void *hidden_inout, const void *attn_delta_f16,
                                        const void *norm_weight_bf16, float eps, uint32_t tokens, void *h2_out,
                                        void *x_out_f16, uint32_t *out_idx, void *out_w_f16, void *stream) {
    NvtxRange nvtx_range("moe_phase1_2_routed");
    int rc = check_layer(h, layer);
    if (rc) return rc;
    if (!hidden_inout || !norm_weight_bf16 || !(eps >= 0.0f)) return NVMAI_CUDA_EINVAL;
    if (x_out_f16 && !aligned16(x_out_f16)) return NVMAI_CUDA_EINVAL;
    if (tokens == 0 || tokens > h->cfg.max_tokens) return NVMAI_CUDA_ERANGE;
    if (h->cfg.top_k > (uint32_t)kMaxTopK) return NVMAI_CUDA_EINVAL;
    XSource xsrc{};
    xsrc.y_prev = hidden_inout;
    xsrc.x_out = x_out_f16 ? static_cast<__half *>(x_out_f16) : h->xnorm;
    xsrc.delta = static_cast<const __half *>(attn_delta_f16);
    xsrc.norm_w = static_cast<const uint16_t *>(norm_weight_bf16);
    xsrc.eps = eps;
    return layer_decode_impl(h, layer, xsrc, xsrc.x_out, tokens, hidden_inout, h2_out, out_idx,
                             static_cast<__half *>(out_w_f16), static_cast<cudaStream_t>(stream), nullptr,
                             xsrc.delta);
}

// The same with the NEXT block's input norm folded into the last stage as well: the stage that writes the hidden
// state also writes x_next = rmsnorm_bf16w(hidden, next_norm_weight) (single-token path: the down-stage block that
// finishes a row last; batched paths: the combine block of the row).
int nvmai_cuda_moe_layer_decode_fused_norms(nvmai_cuda_moe *h, uint32_t layer, void *hidden_inout, const void *attn_delta_f16,
                                            const void *norm_weight_bf16, float eps, uint32_t tokens,
                                            const void *next_norm_weight_bf16, float next_eps, void *x_next_out_f16,
                                            void *h2_out, void *x_out_f16, uint32_t *out_idx, void *out_w_f16, void *stream) {
    NvtxRange nvtx_range("moe_phase1_2_routed");
    if (!h) return NVMAI_CUDA_EINVAL;
    if (!next_norm_weight_bf16 || !x_next_out_f16 || !(next_eps >= 0.0f)) return NVMAI_CUDA_EINVAL;
    h->next_norm = NextNorm{static_cast<const uint16_t *>(next_norm_weight_bf16), next_eps, static_cast<__half *>(x_next_out_f16),
                            h->row_counter};
    const int rc = nvmai_cuda_moe_layer_decode_prenorm(h, layer, hidden_inout, attn_delta_f16, norm_weight_bf16, eps, tokens,
                                                       h2_out, x_out_f16, out_idx, out_w_f16, stream);
    h->next_norm = NextNorm{};
    return rc;
}

int nvmai_cuda_moe_layer_prefill(nvmai_cuda_moe *h, uint32_t layer, const void *x_f16, uint32_t tokens,
                                 void *hidden_inout, void *y_out, uint32_t *out_idx, void *out_w_f16, void *stream) {
    NvtxRange nvtx_range("prefill_routed_tile");
    int rc = check_layer(h, layer);
    if (rc) return rc;
    const auto &c = h->cfg;
    if (!x_f16 || !aligned16(x_f16) || (!hidden_inout && !y_out)) return NVMAI_CUDA_EINVAL;
    if (tokens == 0 || tokens > c.max_tokens) return NVMAI_CUDA_ERANGE;
    if (c.top_k > (uint32_t)kMaxTopK) return NVMAI_CUDA_EINVAL;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // The tensor-core kernels tile the weights by 128 rows per accumulator, two accumulators per block.  Shapes
    // they do not cover (the reference's own prefill test runs d = f = 64, top-2), a rank that holds a subset of
    // the experts, and NVMAI_CUDA_PREFILL_TC=0 take the exact grouped kernels of the batched decode path with the
    // prefill shaders' rounding points: router, grouping, gate/up and down per (tile, work item), ordered combine.
    const bool tiles_fit = c.f % kPfTileM == 0 && c.d % (2 * kPfTileM) == 0 && c.shared_f % kPfTileM == 0;
    if (!tiles_fit || !h->prefill_tc) {
        if (h->expert_map) return NVMAI_CUDA_EINVAL;      // prefill runs on one GPU's full expert set
        uint32_t *idx = out_idx ? out_idx : h->idx;
        __half *w = out_w_f16 ? static_cast<__half *>(out_w_f16) : h->w;
        const XSource xsrc{static_cast<const __half *>(x_f16), c.d, nullptr, nullptr};
        if ((rc = launch_stage1(h, h->layers[layer], xsrc, tokens, idx, w, true, false, c.shared_f != 0, false, st))) return rc;
        return grouped_tail(h, h->layers[layer], static_cast<const __half *>(x_f16), tokens, idx, w, hidden_inout,
                            y_out ? y_out : h->y, st, nullptr, nullptr, true);
    }
    if (h->expert_map) return NVMAI_CUDA_EINVAL;
    return layer_prefill_impl(h, layer, static_cast<const __half *>(x_f16), tokens, hidden_inout, y_out, out_idx,
                              static_cast<__half *>(out_w_f16), st);
}

int nvmai_cuda_moe_group_pairs(nvmai_cuda_moe *h, const uint32_t *idx, const void *w_f16, uint32_t tokens,
                               void *sorted_pairs, uint32_t *expert_offsets, uint32_t *expert_counts, void *stream) {
    if (!h || !idx || !sorted_pairs || !expert_offsets || !expert_counts) return NVMAI_CUDA_EINVAL;
    if (tokens == 0 || tokens > h->cfg.max_tokens) return NVMAI_CUDA_ERANGE;
    return launch_group_pairs(h, idx, static_cast<const __half *>(w_f16), tokens,
                              static_cast<TokenExpertPair *>(sorted_pairs), expert_offsets, expert_counts, false, false,
                              static_cast<cudaStream_t>(stream));
}

int nvmai_cuda_moe_set_expert_map(nvmai_cuda_moe *h, const uint32_t *map_host, uint32_t n_local) {
    if (!h) return NVMAI_CUDA_EINVAL;
    const auto &c = h->cfg;
    h->pd_layers_stale = true;              // the tensor maps span the blobs this rank holds
    if (map_host == nullptr) {              // back to "every expert is local"
        cudaFree(h->expert_map);
        h->expert_map = nullptr;
        h->n_local = 0;
        return NVMAI_CUDA_OK;
    }
    if (n_local == 0 || n_local > c.num_experts) return NVMAI_CUDA_ERANGE;
    uint32_t seen = 0;
    std::vector<bool> used(n_local, false);
    for (uint32_t e = 0; e < c.num_experts; ++e) {
        if (map_host[e] == kNotLocal) continue;
        if (map_host[e] >= n_local) return NVMAI_CUDA_ERANGE;
        if (used[map_host[e]]) return NVMAI_CUDA_EINVAL;       // two experts on one local blob
        used[map_host[e]] = true;
        ++seen;
    }
    if (seen != n_local) return NVMAI_CUDA_EINVAL;     // a bad placement map is rejected, not trusted
    if (!h->expert_map) {
        int rc = record(h, cudaMalloc(reinterpret_cast<void **>(&h->expert_map), kMaxExperts * sizeof(uint32_t)));
        if (rc) return NVMAI_CUDA_ENOMEM;
    }
    h->n_local = n_local;
    return record(h, cudaMemcpy(h->expert_map, map_host, c.num_experts * sizeof(uint32_t), cudaMemcpyHostToDevice));
}

int nvmai_cuda_moe_routed_partial(nvmai_cuda_moe *h, uint32_t layer, const void *x_f16, uint32_t tokens,
                                  const uint32_t *idx, const void *w_f16, float *share_f32, void *stream) {
    NvtxRange nvtx_range("prefill_routed_tile");
    int rc = check_layer(h, layer);
    if (rc) return rc;
    if (!x_f16 || !idx || !w_f16 || !share_f32 || !aligned16(x_f16)) return NVMAI_CUDA_EINVAL;
    if (tokens == 0 || tokens > h->cfg.max_tokens) return NVMAI_CUDA_ERANGE;
    if (tc_batch_ok(h, tokens, false, static_cast<cudaStream_t>(stream))) {
        PrefillMode mode;
        mode.decode_order = true; mode.routed_only = true; mode.partial_y = share_f32;
        return layer_prefill_impl(h, layer, static_cast<const __half *>(x_f16), tokens, nullptr, nullptr,
                                  const_cast<uint32_t *>(idx), static_cast<__half *>(const_cast<void *>(w_f16)),
                                  static_cast<cudaStream_t>(stream), mode);
    }
    return grouped_tail(h, h->layers[layer], static_cast<const __half *>(x_f16), tokens, idx,
                        static_cast<const __half *>(w_f16), nullptr, nullptr, static_cast<cudaStream_t>(stream),
                        share_f32);
}

int nvmai_cuda_moe_ep_finalize(nvmai_cuda_moe *h, const float *shares_f32, uint32_t ranks, const void *h1,
                               uint32_t tokens, void *y, void *hidden_inout, void *stream) {
    NvtxRange nvtx_range("prefill_moe_reduce");
    if (!h || !shares_f32 || ranks == 0 || tokens == 0) return NVMAI_CUDA_EINVAL;
    EpFinalizeParams p{shares_f32, ranks, h1, y, hidden_inout, tokens, h->cfg.d};
    const size_t n = (size_t)tokens * h->cfg.d;
    const unsigned blocks = (unsigned)std::min<size_t>((n + 255) / 256, 1184);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dispatch_out(h->cfg.out_dtype, [&](auto O) {
        return launch_kernel(h, ep_finalize_kernel<decltype(O)::value>, dim3(blocks), dim3(256), 0, st, false, p);
    });
}

int nvmai_cuda_moe_rms_renorm(nvmai_cuda_moe *h, const void *y, uint32_t tokens, void *x_f16_out, void *stream) {
    if (!h || !y || !x_f16_out || tokens == 0) return NVMAI_CUDA_EINVAL;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (h->cfg.out_dtype == NVMAI_OUT_FP16)
        rms_renorm_kernel<OUT_F16><<<tokens, 256, 0, st>>>(y, static_cast<__half *>(x_f16_out), h->cfg.d);
    else
        rms_renorm_kernel<OUT_F32><<<tokens, 256, 0, st>>>(y, static_cast<__half *>(x_f16_out), h->cfg.d);
    return check_launch(h);
}

// Layer l > 0 reads the previous layer's block output and renormalises it inside
// its own stage 1 (every block derives the same rows; block 0 stores them for
// stage 2), so a layer is exactly three launches.
static int stack_enqueue(nvmai_cuda_moe *h, const __half *x0, uint32_t tokens, void *y_last, cudaStream_t st) {
    const auto &c = h->cfg;
    for (uint32_t l = 0; l < c.num_layers; ++l) {
        const bool last = l + 1 == c.num_layers;
        void *y = last ? y_last : h->y;
        XSource xsrc{};
        const __half *x_rows;
        if (l == 0) { xsrc.x = x0; xsrc.x_stride = c.d; x_rows = x0; }
        else { xsrc.y_prev = h->y; xsrc.x_out = h->xnorm; x_rows = h->xnorm; }
        int rc = layer_decode_impl(h, l, xsrc, x_rows, tokens, nullptr, y, nullptr, nullptr, st,
                                   last ? nullptr : &h->layers[l + 1]);
        if (rc) return rc;
    }
    return NVMAI_CUDA_OK;
}

int nvmai_cuda_moe_stack_decode(nvmai_cuda_moe *h, const void *x0_f16, uint32_t tokens, void *y_last, void *stream) {
    NvtxRange nvtx_range("moe_stack_decode");
    if (!h || !x0_f16 || !y_last || !aligned16(x0_f16)) return NVMAI_CUDA_EINVAL;
    const auto &c = h->cfg;
    if (tokens == 0 || tokens > c.max_tokens) return NVMAI_CUDA_ERANGE;
    if (c.top_k > (uint32_t)kMaxTopK) return NVMAI_CUDA_EINVAL;
    for (uint32_t l = 0; l < c.num_layers; ++l)
        if (!h->layers[l].registered) return NVMAI_CUDA_EINVAL;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // Launch-bound chain (3 small kernels per layer): replay it as a CUDA graph.
    // The graph is captured once per (x0, y, tokens, stream); a stream that is
    // itself being captured, or the legacy default stream, gets plain launches.
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (st != nullptr) cudaStreamIsCapturing(st, &cs);
    // One token and a shape the resident kernel covers: the whole step is one launch (no graph needed).  A stream
    // under capture keeps the staged launches (the layer table may have to be uploaded, which a capture forbids).
    if (h->decode_mode != 1 && tokens == 1 && cs == cudaStreamCaptureStatusNone) {
        PdPlan plan;
        if (pd_plan(h, plan) && pd_prepare(h, st) == NVMAI_CUDA_OK)
            return pd_launch(h, plan, static_cast<const __half *>(x0_f16), y_last, st);
    }
    if (h->decode_mode != 1 && tokens >= 2 && tokens <= (uint32_t)kPbMaxRows && cs == cudaStreamCaptureStatusNone) {
        PbPlan bplan;      // a few rows: the resident kernel with the rows as the tensor-core step's columns
        if (pb_plan(h, tokens, bplan) && pd_prepare(h, st) == NVMAI_CUDA_OK)
            return pb_launch(h, bplan, static_cast<const __half *>(x0_f16), tokens, y_last, 0, 1, nullptr, st);
    }
    if (h->decode_mode == 2) return NVMAI_CUDA_EINVAL;
    if (st == nullptr || cs != cudaStreamCaptureStatusNone)
        return stack_enqueue(h, static_cast<const __half *>(x0_f16), tokens, y_last, st);
    if (h->graphs_stale) {
        for (auto &kv : h->stack_graphs) cudaGraphExecDestroy(kv.second);
        h->stack_graphs.clear();
        h->graphs_stale = false;
    }
    StackGraphKey key{x0_f16, y_last, tokens, st};
    auto it = h->stack_graphs.find(key);
    if (it == h->stack_graphs.end()) {
        int rc = record(h, cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
        if (rc) return rc;
        const uint64_t launches_before = g_launches.load();
        rc = stack_enqueue(h, static_cast<const __half *>(x0_f16), tokens, y_last, st);
        g_launches.store(launches_before);        // captured, not launched
        cudaGraph_t graph = nullptr;
        cudaError_t e = cudaStreamEndCapture(st, &graph);
        if (rc) { if (graph) cudaGraphDestroy(graph); return rc; }
        if ((rc = record(h, e))) return rc;
        cudaGraphExec_t exec = nullptr;
        e = cudaGraphInstantiate(&exec, graph, 0);
        cudaGraphDestroy(graph);
        if ((rc = record(h, e))) return rc;
        it = h->stack_graphs.emplace(key, exec).first;
    }
    int rc = record(h, cudaGraphLaunch(it->second, st));
    if (rc == NVMAI_CUDA_OK) g_launches.fetch_add((uint64_t)c.num_layers * 3, std::memory_order_relaxed);
    return rc;
}

int nvmai_cuda_moe_stack_decode_host(nvmai_cuda_moe *h, const void *x0_f16_host, uint32_t tokens, void *y_last_host,
                                     void *stream) {
    if (!h || !x0_f16_host || !y_last_host) return NVMAI_CUDA_EINVAL;
    const auto &c = h->cfg;
    if (tokens == 0 || tokens > c.max_tokens) return NVMAI_CUDA_ERANGE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc = record(h, cudaMemcpyAsync(h->stage_x, x0_f16_host, (size_t)tokens * c.d * 2, cudaMemcpyHostToDevice, st));
    if (rc) return rc;
    rc = nvmai_cuda_moe_stack_decode(h, h->stage_x, tokens, h->stage_y, stream);
    if (rc) return rc;
    rc = record(h, cudaMemcpyAsync(y_last_host, h->stage_y, (size_t)tokens * c.d * out_size(c.out_dtype),
                                   cudaMemcpyDeviceToHost, st));
    if (rc) return rc;
    return record(h, cudaStreamSynchronize(st));
}

// ---- expert parallelism: the whole step inside the library -------------------
// The exchange runs on a communicator of the library's own, so that the compute
// launches and both collectives of all layers sit in one stream and replay as one
// CUDA graph (NCCL supports stream capture of its own calls).

int nvmai_cuda_moe_ep_unique_id(void *id_out_host) {
    if (!id_out_host) return NVMAI_CUDA_EINVAL;
    const NcclApi &nccl = nccl_api();
    if (!nccl.ok) return NVMAI_CUDA_ENCCL;
    NcclUniqueId id;
    if (nccl.GetUniqueId(&id) != kNcclSuccess) return NVMAI_CUDA_ENCCL;
    std::memcpy(id_out_host, &id, sizeof(id));
    return NVMAI_CUDA_OK;
}

int nvmai_cuda_moe_ep_init(nvmai_cuda_moe *h, const void *id_host, uint32_t rank, uint32_t world, uint32_t rows_own) {
    if (!h || !id_host || world == 0 || rank >= world || rows_own == 0) return NVMAI_CUDA_EINVAL;
    const auto &c = h->cfg;
    if ((uint64_t)world * rows_own > c.max_tokens) return NVMAI_CUDA_ERANGE;
    if (c.num_experts % world != 0) return NVMAI_CUDA_EINVAL;
    const NcclApi &nccl = nccl_api();
    if (!nccl.ok) return NVMAI_CUDA_ENCCL;
    ep_release(h);
    const size_t rows = (size_t)world * rows_own;
    auto alloc = [&](auto **ptr, size_t bytes) { return cudaMalloc(reinterpret_cast<void **>(ptr), bytes) == cudaSuccess; };
    // the replicated mode gathers every rank's share of EVERY row and keeps h1 for every row
    if (!(alloc(&h->ep_x_all, rows * c.d * 2) && alloc(&h->ep_share, rows * c.d * 4) &&
          alloc(&h->ep_recv, (size_t)world * rows * c.d * 4) && alloc(&h->ep_h1, rows * c.d * out_size(c.out_dtype)))) {
        cudaGetLastError();
        ep_release(h);
        return NVMAI_CUDA_ENOMEM;
    }
    h->ep_buf_elems = (size_t)world * rows * c.d;
    {
        // counters (4 KB), then the receive area: [2][world][rows][D] 64-bit words (the resident kernel's tagged shares;
        // the staged peer exchange uses the first half of it as fp32 rows)
        // ... and the row area of the fused dispatch: [rows][D / 2] words (two halves per word)
        h->ep_xin_off = 4096 + 2 * rows * c.d * sizeof(unsigned long long) * world;
        const size_t xbytes = h->ep_xin_off + rows * (c.d / 2) * sizeof(unsigned long long);
        if (world > (uint32_t)kEpMaxRanks || c.num_layers > (uint32_t)kEpMaxLayers ||
            cudaMalloc(reinterpret_cast<void **>(&h->ep_xchg), xbytes) != cudaSuccess ||
            cudaMemset(h->ep_xchg, 0, xbytes) != cudaSuccess ||
            cudaMalloc(reinterpret_cast<void **>(&h->ep_step), (2 + kEpMaxLayers) * 8) != cudaSuccess ||
            cudaMemset(h->ep_step, 0, (2 + kEpMaxLayers) * 8) != cudaSuccess) {
            cudaGetLastError();
            cudaFree(h->ep_xchg); h->ep_xchg = nullptr;       // the exchange stays on NCCL then
            cudaFree(h->ep_step); h->ep_step = nullptr;
        }
    }
    if (cudaStreamCreateWithFlags(&h->ep_side, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&h->ep_fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&h->ep_join, cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        ep_release(h);
        return NVMAI_CUDA_ECUDA;
    }
    NcclUniqueId id;
    std::memcpy(&id, id_host, sizeof(id));
    if (nccl.CommInitRank(&h->ep_comm, (int)world, id, (int)rank) != kNcclSuccess) {
        h->ep_comm = nullptr;
        ep_release(h);
        return NVMAI_CUDA_ENCCL;
    }
    h->ep_rank = rank; h->ep_world = world; h->ep_rows_own = rows_own;
    // Every rank's resident kernels must tag a layer alike: the epoch restarts at 1 and the exchange words are
    // cleared on all ranks here (ep_init is collective).  From here to ep_shutdown every rank makes the same
    // sequence of calls on its handle.
    {
        const unsigned int first_epoch = 1;
        const size_t pd_bytes = PdXchg(c).words * sizeof(unsigned long long);
        const size_t pb_bytes = PbXchg(c, kPbMaxRows, (uint32_t)std::max(h->sm_count, 1)).words * sizeof(unsigned long long);
        if (cudaMemset(h->pd_xchg, 0, pd_bytes) != cudaSuccess || cudaMemset(h->pb_xchg, 0, pb_bytes) != cudaSuccess ||
            cudaMemcpy(h->pd_epoch, &first_epoch, sizeof(first_epoch), cudaMemcpyHostToDevice) != cudaSuccess) {
            cudaGetLastError();
            ep_release(h);
            return NVMAI_CUDA_ECUDA;
        }
    }
    return NVMAI_CUDA_OK;
}

int nvmai_cuda_moe_ep_shutdown(nvmai_cuda_moe *h) {
    if (!h) return NVMAI_CUDA_EINVAL;
    ep_release(h);
    return NVMAI_CUDA_OK;
}

int nvmai_cuda_moe_ep_peer_export(nvmai_cuda_moe *h, void *handle_out_host) {
    if (!h || !handle_out_host) return NVMAI_CUDA_EINVAL;
    if (!h->ep_xchg) return NVMAI_CUDA_EINVAL;           // ep_init comes first
    cudaIpcMemHandle_t mh;
    int rc = record(h, cudaIpcGetMemHandle(&mh, h->ep_xchg));
    if (rc) return rc;
    static_assert(sizeof(mh) == NVMAI_CUDA_EP_PEER_HANDLE_BYTES, "IPC handle size");
    std::memcpy(handle_out_host, &mh, sizeof(mh));
    return NVMAI_CUDA_OK;
}

int nvmai_cuda_moe_ep_peer_attach(nvmai_cuda_moe *h, const void *handles_host) {
    if (!h || !handles_host || !h->ep_xchg || h->ep_world == 0) return NVMAI_CUDA_EINVAL;
    for (uint32_t r = 0; r < h->ep_world; ++r) {
        if (r == h->ep_rank) { h->ep_peer_base[r] = h->ep_xchg; continue; }
        cudaIpcMemHandle_t mh;
        std::memcpy(&mh, static_cast<const unsigned char *>(handles_host) + (size_t)r * sizeof(mh), sizeof(mh));
        void *base = nullptr;
        int rc = record(h, cudaIpcOpenMemHandle(&base, mh, cudaIpcMemLazyEnablePeerAccess));
        if (rc) return rc;
        h->ep_peer_base[r] = static_cast<unsigned char *>(base);
    }
    h->ep_peers_attached = true;
    h->ep_graphs_stale = true;
    return NVMAI_CUDA_OK;
}

static int ep_stack_enqueue(nvmai_cuda_moe *h, const __half *x_own, uint32_t rows_own, void *y_own, cudaStream_t st) {
    const auto &c = h->cfg;
    const NcclApi &nccl = nccl_api();
    const uint32_t world = h->ep_world, rows = world * rows_own;
    const size_t own_elems = (size_t)rows_own * c.d;
    for (uint32_t l = 0; l < c.num_layers; ++l) {
        const LayerViews &lv = h->layers[l];
        const bool last = l + 1 == c.num_layers;
        const __half *x = l == 0 ? x_own : h->xnorm;
        int rc;
        if (c.shared_f) {      // needs this rank's rows only: runs beside the exchange and the routed experts
            const XSource own{x, c.d, nullptr, nullptr};
            if ((rc = record(h, cudaEventRecord(h->ep_fork, st)))) return rc;
            if ((rc = record(h, cudaStreamWaitEvent(h->ep_side, h->ep_fork, 0)))) return rc;
            if ((rc = shared_expert_impl(h, lv, own, rows_own, h->ep_h1, h->ep_side))) return rc;
            if ((rc = record(h, cudaEventRecord(h->ep_join, h->ep_side)))) return rc;
        }
        if (nccl.AllGather(x, h->ep_x_all, own_elems, kNcclFloat16, h->ep_comm, st) != kNcclSuccess) return NVMAI_CUDA_ENCCL;
        const XSource all{h->ep_x_all, c.d, nullptr, nullptr};
        if ((rc = launch_stage1(h, lv, all, rows, h->idx, h->w, true, false, false, false, st))) return rc;
        if (tc_batch_ok(h, rows, false, st)) {      // enough rows for the tensor-core items over this rank's experts
            PrefillMode mode;
            mode.decode_order = true; mode.routed_only = true; mode.partial_y = h->ep_share;
            if ((rc = layer_prefill_impl(h, l, h->ep_x_all, rows, nullptr, nullptr, h->idx, h->w, st, mode))) return rc;
        } else if ((rc = grouped_tail(h, lv, h->ep_x_all, rows, h->idx, h->w, nullptr, nullptr, st, h->ep_share))) {
            return rc;
        }
        bool ok = nccl.GroupStart() == kNcclSuccess;      // all-to-all: block r of my shares -> rank r
        for (uint32_t r = 0; r < world && ok; ++r) {
            ok = nccl.Send(h->ep_share + r * own_elems, own_elems, kNcclFloat32, (int)r, h->ep_comm, st) == kNcclSuccess &&
                 nccl.Recv(h->ep_recv + r * own_elems, own_elems, kNcclFloat32, (int)r, h->ep_comm, st) == kNcclSuccess;
        }
        const bool ended = nccl.GroupEnd() == kNcclSuccess;
        if (!ok || !ended) return NVMAI_CUDA_ENCCL;
        void *y = last ? y_own : h->y;
        if (c.shared_f && (rc = record(h, cudaStreamWaitEvent(st, h->ep_join, 0)))) return rc;
        if ((rc = nvmai_cuda_moe_ep_finalize(h, h->ep_recv, world, c.shared_f ? h->ep_h1 : nullptr, rows_own, y, nullptr, st)))
            return rc;
        if (!last && (rc = nvmai_cuda_moe_rms_renorm(h, y, rows_own, h->xnorm, st))) return rc;
    }
    return NVMAI_CUDA_OK;
}

// Small batches (fewer rows in total than the grouping threshold): every rank keeps ALL rows.  One all-gather of
// x per step, then per layer the three decode kernels over all rows, with the expert stages skipping the slots
// whose expert another rank holds, ONE all-gather of the fp32 shares, and the rank-ordered sum on every rank (all
// ranks stay bitwise identical, so the next layer needs no exchange of activations).  4 kernels + 1 collective per
// layer instead of 9 + 2; the router, the shared expert and the sum are computed redundantly, which is cheap at
// these sizes.
static int ep_stack_enqueue_replicated(nvmai_cuda_moe *h, const __half *x_own, uint32_t rows_own, void *y_own, cudaStream_t st) {
    const auto &c = h->cfg;
    const NcclApi &nccl = nccl_api();
    const uint32_t world = h->ep_world, rows = world * rows_own;
    const size_t own_elems = (size_t)rows_own * c.d, all_elems = (size_t)rows * c.d;
    if (nccl.AllGather(x_own, h->ep_x_all, own_elems, kNcclFloat16, h->ep_comm, st) != kNcclSuccess) return NVMAI_CUDA_ENCCL;
    // with the peers' receive areas mapped, the shares travel by peer stores from the down stage itself
    const bool p2p = h->ep_peers_attached;
    EpPeerView view{};
    if (p2p) {
        for (uint32_t r = 0; r < world; ++r) {
            view.arrive[r] = reinterpret_cast<unsigned long long *>(h->ep_peer_base[r]);
            view.recv[r] = reinterpret_cast<float *>(h->ep_peer_base[r] + 4096);
        }
        view.step = h->ep_step; view.local_count = h->ep_step + 2; view.world = world; view.rank = h->ep_rank; view.layers = c.num_layers;
        view.buf_elems = h->ep_buf_elems;
        ep_step_kernel<<<1, 128, 0, st>>>(h->ep_step, h->ep_step + 2, c.num_layers);
        int rc = check_launch(h);
        if (rc) return rc;
    }
    for (uint32_t l = 0; l < c.num_layers; ++l) {
        const LayerViews &lv = h->layers[l];
        XSource xsrc{};
        const __half *x_rows;
        if (l == 0) { xsrc.x = h->ep_x_all; xsrc.x_stride = c.d; x_rows = h->ep_x_all; }
        else { xsrc.y_prev = h->y; xsrc.x_out = h->xnorm; x_rows = h->xnorm; }
        int rc = launch_stage1(h, lv, xsrc, rows, h->idx, h->w, true, c.shared_f != 0, c.shared_f != 0, true, st, true);
        if (rc) return rc;
        RoutedSource src = source_from_layer(h, lv, h->idx);
        src.logits = h->logits;
        src.pes = static_cast<const uint16_t *>(lv.w.per_expert_scale);
        src.publish_idx = h->idx;
        src.publish_w = h->w;
        src.expert_map = h->expert_map;
        if ((rc = launch_stage2(h, src, to_offsets(lv.w.offsets), x_rows, c.d, rows, h->acts, nullptr, c.top_k, true, st))) return rc;
        Stage3Params p{};
        p.src = src;
        p.off = to_offsets(lv.w.offsets);
        p.acts = h->acts;
        p.routing_w = h->w;
        p.sdown = to_mat(lv.w.shared_down_proj);
        p.shared_f = c.shared_f;
        p.shared_bits = c.shared_bits;
        p.shared_act = h->shared_act;
        p.gate_val = c.shared_gate_kind != NVMAI_GATE_NONE ? h->gate_val : nullptr;
        p.h1_out = h->ep_h1;
        p.top_k = c.top_k;
        if (p2p) {
            view.layer = l;
            p.peers = view;
            if ((rc = launch_stage3(h, p, rows, true, st))) return rc;
            EpFinalizePeerParams f{};
            f.recv = view.recv[h->ep_rank]; f.arrive = view.arrive[h->ep_rank] + l; f.step = h->ep_step;
            f.arrivals_per_step = world;          // one announcement per source rank and step
            f.buf_elems = h->ep_buf_elems; f.ranks = world; f.layer = l; f.layers = c.num_layers;
            f.h1 = c.shared_f ? h->ep_h1 : nullptr; f.y = h->y; f.tokens = rows; f.D = c.d; f.status = h->status;
            const unsigned blocks = (unsigned)std::min<size_t>((all_elems + 255) / 256, 148);
            rc = dispatch_out(c.out_dtype, [&](auto O) {
                return launch_kernel(h, ep_finalize_peer_kernel<decltype(O)::value>, dim3(blocks), dim3(256), 0, st, false, f);
            });
            if (rc) return rc;
            continue;
        }
        p.share_out = h->ep_share;
        if ((rc = launch_stage3(h, p, rows, true, st))) return rc;
        if (nccl.AllGather(h->ep_share, h->ep_recv, all_elems, kNcclFloat32, h->ep_comm, st) != kNcclSuccess) return NVMAI_CUDA_ENCCL;
        if ((rc = nvmai_cuda_moe_ep_finalize(h, h->ep_recv, world, c.shared_f ? h->ep_h1 : nullptr, rows, h->y, nullptr, st)))
            return rc;
    }
    return record(h, cudaMemcpyAsync(y_own, static_cast<const char *>(h->y) + (size_t)h->ep_rank * own_elems * out_size(c.out_dtype),
                                     own_elems * out_size(c.out_dtype), cudaMemcpyDeviceToDevice, st));
}

static bool ep_replicated_mode(const nvmai_cuda_moe *h, uint32_t rows_own) {
    const auto &c = h->cfg;
    const uint32_t rows = h->ep_world * rows_own;
    return rows < h->grouped_min_tokens && c.top_k <= (uint32_t)kMaxTopK &&
           (c.top_k + (c.shared_f ? 1 : 0)) * kDownSplit * 32 >= (uint32_t)kMaxExperts;
}

int nvmai_cuda_moe_ep_stack_decode(nvmai_cuda_moe *h, const void *x_own_f16, uint32_t rows_own, void *y_own, void *stream) {
    NvtxRange nvtx_range("moe_ep_stack_decode");
    if (!h || !x_own_f16 || !y_own || !aligned16(x_own_f16)) return NVMAI_CUDA_EINVAL;
    if (!h->ep_comm || !h->expert_map) return NVMAI_CUDA_EINVAL;    // ep_init and set_expert_map come first
    if (rows_own == 0 || rows_own > h->ep_rows_own) return NVMAI_CUDA_ERANGE;
    const auto &c = h->cfg;
    for (uint32_t l = 0; l < c.num_layers; ++l)
        if (!h->layers[l].registered) return NVMAI_CUDA_EINVAL;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const __half *x = static_cast<const __half *>(x_own_f16);
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (st != nullptr) cudaStreamIsCapturing(st, &cs);
    // Up to eight rows in total with the peers' receive areas mapped: one all-gather of the rows, then ONE resident
    // kernel per rank for the whole step; the ranks' shares cross NVLink by peer stores from inside the down phase.
    if (h->ep_peers_attached && h->decode_mode != 1 && cs == cudaStreamCaptureStatusNone) {
        const uint32_t T = h->ep_world * rows_own;
        PbPlan plan;
        if (T <= (uint32_t)kPbMaxRows && pb_plan(h, T, plan) && pd_prepare(h, st) == NVMAI_CUDA_OK) {
            // the dispatch and the combine both live in the kernel: no collective call, no copy around the launch
            unsigned long long *recv[kEpMaxRanks] = {}, *xin[kEpMaxRanks] = {};
            for (uint32_t r = 0; r < h->ep_world; ++r) {
                recv[r] = reinterpret_cast<unsigned long long *>(h->ep_peer_base[r] + 4096);
                xin[r] = reinterpret_cast<unsigned long long *>(h->ep_peer_base[r] + h->ep_xin_off);
            }
            return pb_launch(h, plan, nullptr, T, h->y, h->ep_rank, h->ep_world, recv, st, xin, x, y_own, rows_own);
        }
    }
    if (st == nullptr || cs != cudaStreamCaptureStatusNone) return (ep_replicated_mode(h, rows_own) ? ep_stack_enqueue_replicated(h, x, rows_own, y_own, st) : ep_stack_enqueue(h, x, rows_own, y_own, st));
    if (h->ep_graphs_stale) {
        for (auto &kv : h->ep_graphs) if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
        h->ep_graphs.clear();
        h->ep_graphs_stale = false;
    }
    auto &g = h->ep_graphs[StackGraphKey{x_own_f16, y_own, rows_own, st}];
    // First call per key: plain launches (NCCL sets up its channels on first use).
    // Second call: capture.  Every rank takes the same branch, since all count alike.
    if (g.calls++ == 0) return (ep_replicated_mode(h, rows_own) ? ep_stack_enqueue_replicated(h, x, rows_own, y_own, st) : ep_stack_enqueue(h, x, rows_own, y_own, st));
    if (!g.exec) {
        int rc = record(h, cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
        if (rc) return rc;
        const uint64_t launches_before = g_launches.load();
        rc = (ep_replicated_mode(h, rows_own) ? ep_stack_enqueue_replicated(h, x, rows_own, y_own, st) : ep_stack_enqueue(h, x, rows_own, y_own, st));
        g_launches.store(launches_before);
        cudaGraph_t graph = nullptr;
        cudaError_t e = cudaStreamEndCapture(st, &graph);
        if (rc) { if (graph) cudaGraphDestroy(graph); return rc; }
        if ((rc = record(h, e))) return rc;
        e = cudaGraphInstantiate(&g.exec, graph, 0);
        cudaGraphDestroy(graph);
        if ((rc = record(h, e))) { g.exec = nullptr; return rc; }
    }
    int rc = record(h, cudaGraphLaunch(g.exec, st));
    if (rc == NVMAI_CUDA_OK) {
        if (ep_replicated_mode(h, rows_own)) {
            g_launches.fetch_add((uint64_t)c.num_layers * 4, std::memory_order_relaxed);     // 3 stages + finalize per layer
        } else {
            const uint64_t per_layer = 6 + (c.shared_f ? 2 : 0) + 1;     // router, group, 2 grouped, combine, finalize (+shared 2, +renorm)
            g_launches.fetch_add((uint64_t)c.num_layers * per_layer - 1, std::memory_order_relaxed);
        }
    }
    return rc;
}

int nvmai_cuda_moe_dequant(uint32_t bits, uint32_t meta_dtype, const void *w, const void *scales, const void *biases,
                           uint32_t rows, uint32_t n, float *out_f32, void *stream) {
    if (!w || !scales || !biases || !out_f32 || n % 64 != 0 || rows == 0 || n == 0) return NVMAI_CUDA_EINVAL;
    const size_t total = (size_t)rows * n;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dispatch_bits_meta(bits, meta_dtype, [&](auto B, auto M) {
        dequant_kernel<decltype(B)::value, decltype(M)::value><<<blocks, 256, 0, st>>>(
            static_cast<const uint8_t *>(w), static_cast<const uint16_t *>(scales),
            static_cast<const uint16_t *>(biases), rows, n, out_f32);
        return check_launch(nullptr);
    });
}

int nvmai_cuda_moe_affine_gemv(uint32_t bits, uint32_t meta_dtype, const void *w, const void *scales,
                               const void *biases, const void *x_f16, void *y_f16, uint32_t m, uint32_t n,
                               void *stream) {
    if (!w || !scales || !biases || !x_f16 || !y_f16 || m == 0 || n == 0 || n % 64 != 0) return NVMAI_CUDA_EINVAL;
    if (!aligned16(w) || !aligned16(x_f16)) return NVMAI_CUDA_EINVAL;
    if (!valid_bits(bits) || meta_dtype > NVMAI_META_FP16) return NVMAI_CUDA_EINVAL;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned blocks = (m + 7) / 8;
    if (meta_dtype == NVMAI_META_BF16)
        affine_gemv_kernel<META_BF16><<<blocks, 256, 0, st>>>(bits, static_cast<const uint8_t *>(w),
            static_cast<const uint16_t *>(scales), static_cast<const uint16_t *>(biases),
            static_cast<const __half *>(x_f16), static_cast<__half *>(y_f16), m, n);
    else
        affine_gemv_kernel<META_FP16><<<blocks, 256, 0, st>>>(bits, static_cast<const uint8_t *>(w),
            static_cast<const uint16_t *>(scales), static_cast<const uint16_t *>(biases),
            static_cast<const __half *>(x_f16), static_cast<__half *>(y_f16), m, n);
    return check_launch(nullptr);
}

int nvmai_cuda_moe_silu_mul_f16(const void *gate, const void *up, void *out, uint32_t count, void *stream) {
    if (!gate || !up || !out) return NVMAI_CUDA_EINVAL;
    if (count == 0) return NVMAI_CUDA_OK;
    silu_mul_kernel<<<(count + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half *>(gate), static_cast<const __half *>(up), static_cast<__half *>(out), count);
    return check_launch(nullptr);
}

int nvmai_cuda_moe_sigmoid_scalar_mul_f16(void *y, const void *gate, uint32_t count, void *stream) {
    if (!y || !gate) return NVMAI_CUDA_EINVAL;
    if (count == 0) return NVMAI_CUDA_OK;
    sigmoid_scalar_mul_kernel<<<(count + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__half *>(y), static_cast<const __half *>(gate), count);
    return check_launch(nullptr);
}

int nvmai_cuda_moe_residual_add_f16(void *hidden, const void *delta, uint32_t count, void *stream) {
    if (!hidden || !delta) return NVMAI_CUDA_EINVAL;
    if (count == 0) return NVMAI_CUDA_OK;
    residual_add_kernel<<<(count + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__half *>(hidden), static_cast<const __half *>(delta), count);
    return check_launch(nullptr);
}

int nvmai_cuda_moe_set_trace(nvmai_cuda_moe *h, int enable) {
    if (!h) return NVMAI_CUDA_EINVAL;
    h->trace_on = enable != 0;
    h->graphs_stale = true;     // captured launches carry (or do not carry) the trace slots
    const size_t pd_bytes = (size_t)h->cfg.num_layers * (size_t)std::max(h->sm_count, 1) * 16 * sizeof(unsigned long long);
    if (enable && !h->pd_trace && cudaMalloc(reinterpret_cast<void **>(&h->pd_trace), pd_bytes) != cudaSuccess) {
        cudaGetLastError();
        h->pd_trace = nullptr;
        return NVMAI_CUDA_ENOMEM;
    }
    if (h->pd_trace) cudaMemset(h->pd_trace, 0, pd_bytes);
    return record(h, cudaMemset(h->trace, 0, (size_t)h->cfg.num_layers * 3 * kTraceWords * sizeof(unsigned long long)));
}

int nvmai_cuda_moe_read_trace(nvmai_cuda_moe *h, uint64_t *out_host, uint32_t layers) {
    if (!h || !out_host || layers > h->cfg.num_layers) return NVMAI_CUDA_EINVAL;
    return record(h, cudaMemcpy(out_host, h->trace, (size_t)layers * 3 * kTraceWords * sizeof(unsigned long long),
                                cudaMemcpyDeviceToHost));
}

int nvmai_cuda_moe_read_block_trace(nvmai_cuda_moe *h, uint64_t *out_host, uint32_t layers, uint32_t *out_blocks) {
    if (!h || !out_blocks || layers > h->cfg.num_layers) return NVMAI_CUDA_EINVAL;
    *out_blocks = (uint32_t)h->sm_count;
    if (!out_host) return NVMAI_CUDA_OK;          // size query
    if (!h->pd_trace) return NVMAI_CUDA_EINVAL;   // set_trace(1) comes first
    return record(h, cudaMemcpy(out_host, h->pd_trace, (size_t)layers * h->sm_count * 16 * sizeof(unsigned long long),
                                cudaMemcpyDeviceToHost));
}

int nvmai_cuda_moe_synchronize(nvmai_cuda_moe *h, void *stream) {
    int rc = record(h, cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    if (rc || !h) return rc;
    unsigned int st = 0;
    rc = record(h, cudaMemcpy(&st, h->status, sizeof(st), cudaMemcpyDeviceToHost));
    if (rc) return rc;
    if (st != 0) {      // a kernel gave up a bounded wait; its outputs are undefined
        cudaMemset(h->status, 0, sizeof(st));
        // the one-launch step may have stopped half way: move its epoch past every tag it can have written
        unsigned int epoch = 0;
        if (h->pd_epoch && cudaMemcpy(&epoch, h->pd_epoch, sizeof(epoch), cudaMemcpyDeviceToHost) == cudaSuccess) {
            epoch += h->cfg.num_layers + 1;
            if (epoch == 0) epoch = 1;
            cudaMemcpy(h->pd_epoch, &epoch, sizeof(epoch), cudaMemcpyHostToDevice);
        }
        return NVMAI_CUDA_ETIMEOUT;
    }
    return NVMAI_CUDA_OK;
}

// Waits for `stream` the way a rank of an expert-parallel job has to: a collective whose peer died never ends, so the
// wait polls the stream and the communicator's asynchronous error state from the host instead of blocking in the
// driver.  An error reported by NCCL, or `timeout_ms` without the stream finishing, aborts the communicator (which
// ends its kernels in flight), drops the expert-parallel state of the handle (ep_init makes a new one) and returns
// NVMAI_CUDA_ENCCL / NVMAI_CUDA_ETIMEOUT.  Otherwise the result is that of nvmai_cuda_moe_synchronize.
int nvmai_cuda_moe_ep_synchronize(nvmai_cuda_moe *h, void *stream, uint32_t timeout_ms) {
    if (!h) return NVMAI_CUDA_EINVAL;
    if (!h->ep_comm) return nvmai_cuda_moe_synchronize(h, stream);
    const NcclApi &nccl = nccl_api();
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const auto t0 = std::chrono::steady_clock::now();
    int verdict = NVMAI_CUDA_OK;
    for (uint32_t spins = 0;; ++spins) {
        const cudaError_t q = cudaStreamQuery(st);
        if (q == cudaSuccess) break;
        if (q != cudaErrorNotReady) return record(h, q);
        int async = kNcclSuccess;
        if (nccl.CommGetAsyncError(h->ep_comm, &async) != kNcclSuccess || (async != kNcclSuccess && async != kNcclInProgress)) {
            verdict = NVMAI_CUDA_ENCCL;
            break;
        }
        const auto waited = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (timeout_ms != 0 && waited >= (long long)timeout_ms) { verdict = NVMAI_CUDA_ETIMEOUT; break; }
        if (spins > 1000) std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    if (verdict != NVMAI_CUDA_OK) {
        nccl.CommAbort(h->ep_comm);      // frees the communicator and ends what it still has on the device
        h->ep_comm = nullptr;
        cudaStreamSynchronize(st);       // the rest of the stream (kernels of this library wait bounded times only)
        cudaGetLastError();
        ep_release(h);
        unsigned int zero = 0;
        cudaMemcpy(h->status, &zero, sizeof(zero), cudaMemcpyHostToDevice);
        return verdict;
    }
    return nvmai_cuda_moe_synchronize(h, stream);
}

// Test hook: holds `stream` for `ms` milliseconds with a host function (no kernel runs, the device is idle), so that
// a test can watch a wait run out without anything being wrong on the GPU.
int nvmai_cuda_moe_debug_host_delay(nvmai_cuda_moe *h, void *stream, uint32_t ms) {
    if (!h) return NVMAI_CUDA_EINVAL;
    return record(h, cudaLaunchHostFunc(static_cast<cudaStream_t>(stream),
                                        [](void *arg) { std::this_thread::sleep_for(std::chrono::milliseconds((uintptr_t)arg)); },
                                        reinterpret_cast<void *>((uintptr_t)ms)));
}

int nvmai_cuda_moe_last_cuda_error(const nvmai_cuda_moe *h) { return h ? h->last_cuda_error : 0; }

const char *nvmai_cuda_moe_error_string(int code) {
    switch (code) {
        case NVMAI_CUDA_OK: return "ok";
        case NVMAI_CUDA_EINVAL: return "invalid argument (shape, null pointer or alignment)";
        case NVMAI_CUDA_ERANGE: return "index or size out of range";
        case NVMAI_CUDA_ENOMEM: return "device allocation failed";
        case NVMAI_CUDA_ECUDA: return "CUDA runtime error";
        case NVMAI_CUDA_ETIMEOUT: return "bounded device-side wait expired";
        case NVMAI_CUDA_ENCCL: return "NCCL error";
        case NVMAI_CUDA_EIO: return "weight file cannot be opened or is too short";
        default: return "unknown error";
    }
}

uint64_t nvmai_cuda_moe_launch_count(void) { return g_launches.load(); }

int nvmai_cuda_moe_set_decode_mode(nvmai_cuda_moe *h, int mode) {
    if (!h || mode < 0 || mode > 2) return NVMAI_CUDA_EINVAL;
    h->decode_mode = mode;
    return NVMAI_CUDA_OK;
}

int nvmai_cuda_moe_read_route_log(nvmai_cuda_moe *h, uint32_t *out_host, uint32_t layers) {
    if (!h || !out_host || layers > h->cfg.num_layers || h->pd_route_rows != 1) return NVMAI_CUDA_EINVAL;
    return record(h, cudaMemcpy(out_host, h->pd_route_log, (size_t)layers * h->cfg.top_k * 4, cudaMemcpyDeviceToHost));
}

int nvmai_cuda_moe_read_route_log_rows(nvmai_cuda_moe *h, uint32_t *out_host, uint32_t layers, uint32_t rows) {
    if (!h || !out_host || layers > h->cfg.num_layers || rows != h->pd_route_rows) return NVMAI_CUDA_EINVAL;
    return record(h, cudaMemcpy(out_host, h->pd_route_log, (size_t)layers * rows * h->cfg.top_k * 4, cudaMemcpyDeviceToHost));
}

int nvmai_cuda_moe_debug_drop_prefill_copy(nvmai_cuda_moe *h) {
    if (!h) return NVMAI_CUDA_EINVAL;
    h->pf_debug_drop = true;
    return NVMAI_CUDA_OK;
}

int nvmai_cuda_moe_debug_mute_block(nvmai_cuda_moe *h, uint32_t block) {
    if (!h) return NVMAI_CUDA_EINVAL;
    h->pd_mute_block = block;
    return NVMAI_CUDA_OK;
}

int nvmai_cuda_moe_debug_set_wait_limit(uint64_t nanoseconds) {
    const unsigned long long v = nanoseconds ? nanoseconds : 1000000000ull;
    return cudaMemcpyToSymbol(g_wait_limit_ns, &v, sizeof(v)) == cudaSuccess ? NVMAI_CUDA_OK : NVMAI_CUDA_ECUDA;
}

int nvmai_cuda_moe_read_file_to_device(const char *path, uint64_t file_offset, uint64_t bytes, void *device_dst,
                                       void *stream) {
    if (!path || (!device_dst && bytes)) return NVMAI_CUDA_EINVAL;
    if (bytes == 0) return NVMAI_CUDA_OK;
    const int fd = ::open(path, O_RDONLY);
    if (fd < 0) return NVMAI_CUDA_EIO;
    constexpr size_t kPiece = 16u << 20;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned char *stage[2] = {nullptr, nullptr};
    cudaEvent_t copied[2] = {nullptr, nullptr};
    int rc = NVMAI_CUDA_OK;
    for (int i = 0; i < 2 && rc == NVMAI_CUDA_OK; ++i) {
        if (cudaMallocHost(reinterpret_cast<void **>(&stage[i]), kPiece) != cudaSuccess) rc = NVMAI_CUDA_ENOMEM;
        else if (cudaEventCreateWithFlags(&copied[i], cudaEventDisableTiming) != cudaSuccess) rc = NVMAI_CUDA_ECUDA;
    }
    uint64_t done = 0;
    for (int piece = 0; rc == NVMAI_CUDA_OK && done < bytes; ++piece) {
        const int b = piece & 1;
        const size_t n = (size_t)std::min<uint64_t>(kPiece, bytes - done);
        if (piece >= 2 && cudaEventSynchronize(copied[b]) != cudaSuccess) { rc = NVMAI_CUDA_ECUDA; break; }
        // the piece is read by a few threads side by side: one positioned read runs at memcpy speed out of the page
        // cache, well below what the copy engine takes
        constexpr int kReaders = 4;
        const size_t share = ((n + kReaders - 1) / kReaders + 4095) & ~(size_t)4095;
        std::atomic<int> short_reads{0};
        auto read_range = [&](size_t lo, size_t hi) {
            size_t got = lo;
            while (got < hi) {      // a positioned read may return less than asked
                const ssize_t r = ::pread(fd, stage[b] + got, hi - got, (off_t)(file_offset + done + got));
                if (r < 0 && errno == EINTR) continue;
                if (r <= 0) break;
                got += (size_t)r;
            }
            if (got != hi) short_reads.fetch_add(1);
        };
        std::thread readers[kReaders - 1];
        int started = 0;
        for (int t = 1; t < kReaders; ++t) {
            const size_t lo = std::min(n, (size_t)t * share), hi = std::min(n, lo + share);
            if (lo < hi) readers[started++] = std::thread(read_range, lo, hi);
        }
        read_range(0, std::min(n, share));
        for (int t = 0; t < started; ++t) readers[t].join();
        if (short_reads.load() != 0) { rc = NVMAI_CUDA_EIO; break; }
        if (cudaMemcpyAsync(static_cast<unsigned char *>(device_dst) + done, stage[b], n, cudaMemcpyHostToDevice, st) !=
                cudaSuccess || cudaEventRecord(copied[b], st) != cudaSuccess) { rc = NVMAI_CUDA_ECUDA; break; }
        done += n;
    }
    if (cudaStreamSynchronize(st) != cudaSuccess && rc == NVMAI_CUDA_OK) rc = NVMAI_CUDA_ECUDA;
    for (int i = 0; i < 2; ++i) {
        if (copied[i]) cudaEventDestroy(copied[i]);
        if (stage[i]) cudaFreeHost(stage[i]);
    }
    ::close(fd);
    return rc;
}

}  // extern "C"
