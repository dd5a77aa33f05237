// Shared declarations of the CUDA backend: device layout of a palettized
// tensor, the context object behind the C ABI, and launch helpers.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/prism_cuda.h"

namespace prism {

// Device ordinals a context may be created on (prism_cuda_create refuses larger ones); sizes the
// per-device "kernel attributes set" caches.
constexpr int PRISM_MAX_DEVICES = 64;

// ---------------------------------------------------------------------------
// Device layout of one palettized tensor ("re-laid" form of the .cimage
// split-block payload, src/quantization/cimage.rs:98-125).
//
//   pal : [m_pad][2^bits] fp16      palette of every row, rows >= m are zero
//   idx : [n_hb][n_chunks][32][16 B]
//         half-block hb = rows hb*32 .. hb*32+31, chunk c = bytes 16c..16c+15
//         of each row's packed index string (32 weights at 4 bit, 64 at 2 bit).
//
// One warp-wide 128-bit load therefore fetches the same 16-byte chunk of 32
// consecutive rows as one contiguous 512-byte line, and a half-block's whole K
// range is one contiguous run of n_chunks*512 bytes.  m_pad is a multiple of
// 64 so a CTA can always read two half-blocks.
// ---------------------------------------------------------------------------
struct LutTensor {
    std::string name;
    uint32_t m = 0, k = 0, bits = 4;
    uint32_t m_pad = 0, n_hb = 0;
    uint32_t row_bytes = 0;  // k*bits/8
    uint32_t n_chunks = 0;   // ceil(row_bytes/16)
    uint8_t *idx = nullptr;
    uint16_t *pal = nullptr;
    size_t idx_bytes = 0, pal_bytes = 0;
    bool live = false;
    uint32_t n_ent() const { return 1u << bits; }
    // bytes a GEMV over this tensor must move: indices + palettes + x + y
    uint64_t algorithmic_bytes() const {
        return (uint64_t)m * row_bytes + (uint64_t)m * n_ent() * 2 + 2ull * k + 2ull * m;
    }
};

__host__ __device__ inline uint32_t round_up_u32(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

__host__ __device__ inline size_t lut_idx_offset(uint32_t n_chunks, uint32_t hb, uint32_t chunk,
                                                 uint32_t lane) {
    return ((size_t)hb * n_chunks + chunk) * 512 + (size_t)lane * 16;
}

}  // namespace prism

struct prism_nccl_api;

// The opaque context of the C ABI.
struct prism_cuda_ctx {
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    std::string err;
    std::vector<prism::LutTensor> tensors;
    std::unordered_map<std::string, int32_t> by_name;
    // options
    int gemv_variant = 1;
    float pending_norm_eps = -1.0f;  // >= 0: the next launch_gemv normalises its input row first (then clears this)
    int gemm_variant = 1;  // 1: tcgen05/TMEM kernel where eligible, 0: activation rows through the GEMV kernel
    int fuse = 1;
    int sk_min_chunks = 8;      // stream-K GEMV, small matrices: fewest 1 KB index chunks a CTA is given
    int sk_stream_chunks = 64;  // chunks per CTA from which the balanced contiguous partition is used
    int cl_max_units = 16384;    // cluster GEMV for matrices of at most this many (64-row block, 1 KB chunk) units; 0: never
    int batch_gemv_max = 8;   // decode batches up to this size use the batched GEMV (groups of 8), larger ones the GEMM
    int attn_cluster = 0;    // CTAs per (head, sequence) of the fused attention kernel; 0: chosen from max_seq
    int ws_whole_blocks = 1024;  // warp-specialised GEMV: one whole block per CTA when there are almost as many blocks as SMs and rows have at most this many chunks; 0: never
    int ws_whole_fill = 50;  // ... for one activation row, when the matrix has at least this many blocks per 100 SMs
    int attn_group = 0;      // most query heads of a KV group one cluster of the fused attention serves (1/2/4/8); 0: chosen from the shape
    int gemm_reuse_x = 0;    // set by a caller for the second of two GEMMs over the same activations: skip the re-lay
    int pdl = 1;  // programmatic dependent launch between the kernels of the decode chain
    int prefill_chunk = 512;  // prompt tokens generate() puts through the layers at once (tensor-core GEMMs); 0: one step per token
    int cimage_cache = 0;  // engine_load_cimage keeps / uses the cache of the re-laid image beside the file
    // Upper bound, in polls, of the device-side waits on something outside the waiting CTA (a peer
    // GPU's flag, a grid-wide arrival); a wait that runs out sets the device error word and the
    // kernel goes on.  0: the built-in limits (seconds).  Option "wait_limit_polls".  The mbarrier
    // hand-overs between the warps of one CTA keep their fixed bounds.
    uint32_t wait_limit_polls = 0;
    uint64_t option_epoch = 0;  // bumped by every set_option: a captured decode graph is valid for one epoch
    uint64_t launches = 0;
    // staging for host-pointer entry points (grown on demand)
    // (each pointer is null exactly when its element count is zero)
    uint8_t *stage_in = nullptr, *stage_out = nullptr;
    size_t stage_in_bytes = 0, stage_out_bytes = 0;
    // scratch for split-K partial sums, arrival counters, MLP activation
    float *splitk_partials = nullptr;
    size_t splitk_floats = 0;
    unsigned int *splitk_counters = nullptr;
    size_t splitk_counter_n = 0;
    uint16_t *act_scratch = nullptr;
    size_t act_halfs = 0;
    uint16_t *tmp_scratch = nullptr;  // gate/up outputs of the unfused SwiGLU path
    size_t tmp_halfs = 0;
    // device error word [0] (kernels set it instead of trapping) and probe result [1]
    unsigned int *dev_err = nullptr;
    int smem_base = -1;  // offset of dynamic shared memory in the shared window, probed at create
    // tensor parallel
    int tp_world = 1, tp_rank = 0;
    void *nccl_comm = nullptr;
    prism_nccl_api *nccl = nullptr;
    // peer-memory all-reduce (tp.cu): receive area and flags of this rank, mapped by every peer
    float *tp_recv = nullptr;          // [2 epochs][world][tp_cap] floats
    unsigned int *tp_flags = nullptr;  // [world][TP_AR_MAX_CTAS] last epoch each peer CTA has delivered
    unsigned int *tp_state = nullptr;  // {epoch, CTAs done} of the all-reduce sequence
    void **tp_peer_tab = nullptr;      // device array: world receive-area pointers, then world flag pointers
    void *tp_peer_map[32] = {nullptr};   // what cudaIpcOpenMemHandle returned: [q] receive area, [16+q] flags of peer q
    size_t tp_cap = 0;                 // floats per rank slot; 0: peer path unavailable, NCCL is used
    int tp_peer_ar = 1;                // option "tp_peer_ar": use the peer-memory all-reduce when available
    // option "tp_fused_ar" (batch-1 decode): 0 = GEMV writes fp32 partial sums, a separate kernel pushes and reduces them;
    // 1 = the GEMV epilogue stores its sums straight into every rank's receive area, a small kernel publishes flags and
    // reduces; 2 = flags, wait and reduction inside the GEMV kernel too; 3 = the GEMV epilogue stores 8-byte words
    // {sum, epoch} into every rank's flagged-word area, a small kernel polls the words themselves and reduces; 4 = the
    // flagged words are polled and reduced at the end of the GEMV kernel itself
    int tp_fused_ar = 3;
    std::string tp_peer_reason;        // why the peer path is unavailable ("" when it is set up)
    bool tp_loopback = false;          // prism_cuda_tp_init_loopback: every "peer" is this GPU's own receive area
    // rotation frequencies of the fused attention kernel (attn.cu), one table per (head size, base) ever
    // asked for; tables live until the context is destroyed, so a captured graph's pointer stays valid
    struct RopeTab { uint32_t hd; float base; float *dev; float host[128]; };
    std::vector<RopeTab *> rope_tabs;
    // backend-held KV cache of the MetalBackend-style entry points (prism_cuda_kv_init / kv_append / attention_kv)
    uint16_t *kv_k = nullptr, *kv_v = nullptr;
    uint32_t kv_layers = 0, kv_dim = 0, kv_max_seq = 0;
    // execution plan of the last .cimage that was loaded (src/lut/graph.rs:552-589); version 0: none / unparseable
    struct PlanInfo {
        uint32_t version = 0, num_layers = 0, n_nodes = 0, n_gemm_nodes = 0;
        int kv_fp16 = -1;              // 1: "Fp16", 0: "Int8", -1: absent
        std::string architecture, attention_strategy, lm_head_backend;
    } plan;
};

namespace prism {

int fail(prism_cuda_ctx *ctx, int code, const std::string &msg);
int cuda_fail(prism_cuda_ctx *ctx, cudaError_t e, const char *what);

#define PRISM_CUDA_TRY(ctx, expr)                                         \
    do {                                                                  \
        cudaError_t _e = (expr);                                          \
        if (_e != cudaSuccess) return prism::cuda_fail((ctx), _e, #expr); \
    } while (0)

#define PRISM_TRY(expr)           \
    do {                          \
        int _rc = (expr);         \
        if (_rc != 0) return _rc; \
    } while (0)

// Checks the launch that was just issued and counts it.
int after_launch(prism_cuda_ctx *ctx, const char *kernel);

// ---- programmatic dependent launch ------------------------------------------------------------
// Kernels of the decode chain begin with pdl_launch_dependents() (the next kernel of the stream may
// be scheduled as soon as every CTA of this one has started) and call pdl_wait() before they touch
// anything another kernel produces or consumes: it returns when all earlier kernels have completed
// and their writes are visible.  What runs before pdl_wait() (index prefetch, palette loads, table
// build: inputs that no kernel writes) overlaps the tail of the previous kernel, and the launch
// latency between kernels is hidden.  Only kernels that call pdl_wait() may be launched with
// launch_pdl(); a kernel that never calls pdl_launch_dependents() releases its dependents when it
// exits, which is the ordinary stream order.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

// Launch with a thread-block cluster of `cluster_x` CTAs along x (1: none) and, when the context
// allows it, the programmatic-dependent-launch attribute.
template <typename... KArgs, typename... Args>
inline void launch_cluster_pdl(prism_cuda_ctx *ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                               unsigned cluster_x, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    unsigned n = 0;
    if (cluster_x > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster_x;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        n++;
    }
    if (ctx->pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        n++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    (void)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);  // a failure stays in the last-error slot: after_launch() reports it
}
template <typename... KArgs, typename... Args>
inline void launch_pdl(prism_cuda_ctx *ctx, const char *name, void (*kernel)(KArgs...), dim3 grid, dim3 block,
                       size_t smem, Args &&...args) {
    (void)name;
    launch_cluster_pdl(ctx, kernel, grid, block, smem, 1u, static_cast<Args &&>(args)...);
}
#endif

int ensure_stage(prism_cuda_ctx *ctx, size_t in_bytes, size_t out_bytes);
int ensure_splitk(prism_cuda_ctx *ctx, size_t floats, size_t counters);
int ensure_act(prism_cuda_ctx *ctx, size_t halfs);
int ensure_tmp(prism_cuda_ctx *ctx, size_t halfs);
LutTensor *get_tensor(prism_cuda_ctx *ctx, int32_t handle);
int probe_smem_base(prism_cuda_ctx *ctx);
// tp.cu
int tp_all_reduce_f32(prism_cuda_ctx *ctx, float *buf, size_t n);
int tp_all_gather_bytes(prism_cuda_ctx *ctx, const void *send, void *recv, size_t bytes_per_rank);
// h[i] = f16( f32(f16(sum over ranks of part[i])) + f32(h[i]) ): the all-reduce of a row-parallel
// matmul's fp32 partial sums fused with the residual add, through peer memory (one kernel, no NCCL).
bool tp_peer_ar_ok(prism_cuda_ctx *ctx, size_t n);
int tp_all_reduce_resid_peer(prism_cuda_ctx *ctx, const float *part, uint16_t *h, size_t n);
// the same after a GEMV_TP kernel that only delivered (option tp_fused_ar = 1): flags, wait, reduction, residual
int tp_all_reduce_flags_resid(prism_cuda_ctx *ctx, uint16_t *h, size_t n);
// after a GEMV_TP kernel that delivered flagged words (tp_fused_ar = 3): poll the words, reduction, residual
int tp_all_reduce_ll_resid(prism_cuda_ctx *ctx, uint16_t *h, size_t n);
// Synchronises the stream and reads the device error word.  Codes kernels leave there:
//   1  a kernel found its shared-memory layout assumption broken and refused to run  -> PRISM_E_STATE
//   2  an mbarrier hand-over inside a warp-specialised GEMV gave up                    -> PRISM_E_TIMEOUT
//   3  the peer-memory all-reduce gave up waiting for a peer's slice                   -> PRISM_E_TIMEOUT
//   4  a grid-wide arrival inside a persistent kernel gave up                          -> PRISM_E_TIMEOUT
//   5  an mbarrier wait inside a tcgen05 kernel gave up                                -> PRISM_E_TIMEOUT
// The word is cleared, so the context stays usable.
int check_device_error(prism_cuda_ctx *ctx);
// The same translation for a caller that has already copied the word to the host (clears it if set).
int device_error_result(prism_cuda_ctx *ctx, unsigned int word);
// The wait bound kernels use: the option when set, else `builtin`.
inline uint32_t wait_limit(const prism_cuda_ctx *ctx, uint32_t builtin) {
    return ctx->wait_limit_polls ? ctx->wait_limit_polls : builtin;
}

// ---- kernels' host-side launchers (device pointers, context stream) -------

// relay.cu
int launch_relay(prism_cuda_ctx *ctx, const uint8_t *payload_dev, uint32_t src_m, uint32_t src_k,
                 uint32_t row0, uint32_t col0, LutTensor &t);
int launch_unrelay(prism_cuda_ctx *ctx, const LutTensor &t, uint8_t *payload_dev);
int launch_dequant(prism_cuda_ctx *ctx, const LutTensor &t, uint16_t *out_dev);
int launch_synth(prism_cuda_ctx *ctx, LutTensor &t, uint64_t seed, float sigma, uint32_t row0, uint32_t col0);
int launch_embed(prism_cuda_ctx *ctx, const LutTensor &t, const uint32_t *tokens_dev, uint32_t batch,
                 uint16_t *out_dev, uint16_t *out2_dev);

// gemv.cu
enum GemvMode { GEMV_PLAIN = 0, GEMV_RESID = 1, GEMV_SWIGLU = 2, GEMV_F32 = 3, GEMV_TP = 4 };
// y[b] = W x[b] for b < batch; x rows are x_stride halfs apart, y rows y_stride.
// GEMV_RESID adds resid (same strides as y) after rounding to fp16.
// GEMV_SWIGLU: t = gate, t2 = up, y = f16(f16(silu(f16(g))) * f16(u)).
// GEMV_F32: y is float[batch][y_stride], the unrounded sums (partial products of a
// K-sharded tensor-parallel rank, reduced across ranks before rounding).
// GEMV_TP (one activation row): the same partial products, all-reduced over the tensor-parallel ranks
// through peer memory inside the kernel and added to the residual stream y in place:
// y = f16( f16(sum over ranks) + y )  (tp_push.cuh).  gemv_tp_ok says whether a tensor can take it.
bool gemv_tp_ok(prism_cuda_ctx *ctx, const LutTensor &t);
int launch_gemv(prism_cuda_ctx *ctx, GemvMode mode, const LutTensor &t, const LutTensor *t2,
                const uint16_t *x, uint32_t x_stride, uint16_t *y, uint32_t y_stride,
                const uint16_t *resid, uint32_t batch);

// gemv_sk.cu: persistent stream-K form of the pair-table tensor-core GEMV (4-bit, K % 32 == 0);
// norm_eps >= 0 folds RMSNorm of x into the staging
bool sk_eligible(const LutTensor &t);
int launch_gemv_sk(prism_cuda_ctx *ctx, GemvMode mode, const LutTensor &t, const LutTensor *t2, const uint16_t *x,
                   uint32_t x_stride, void *y, uint32_t y_stride, const uint16_t *resid, uint32_t batch,
                   float norm_eps);

// gemv_ws.cu: warp-specialised persistent form (one CTA per SM; builder warps prepare tables and x
// while compute warps stream), same arguments as launch_gemv_sk
bool ws_eligible(const LutTensor &t);
bool ws_preferred(prism_cuda_ctx *ctx, const LutTensor &t, bool swiglu, uint32_t batch);
int launch_gemv_ws(prism_cuda_ctx *ctx, GemvMode mode, const LutTensor &t, const LutTensor *t2, const uint16_t *x,
                   uint32_t x_stride, void *y, uint32_t y_stride, const uint16_t *resid, uint32_t batch,
                   float norm_eps);

// gemv_cl.cu: small matrices -- one cluster of s CTAs per 64-row block, indices prefetched into registers
// before the dependency wait, sums reduced through distributed shared memory.  cl_cluster_size returns
// s, or 0 when the matrix is not one for this kernel.
uint32_t cl_cluster_size(prism_cuda_ctx *ctx, const LutTensor &t, bool swiglu, uint32_t batch);
int launch_gemv_cl(prism_cuda_ctx *ctx, GemvMode mode, const LutTensor &t, const LutTensor *t2, const uint16_t *x,
                   uint32_t x_stride, void *y, uint32_t y_stride, const uint16_t *resid, uint32_t batch, float norm_eps,
                   uint32_t s);

// gemv_wsb.cu: the warp-specialised kernel for 2..8 activation rows at once (weights streamed once);
// the rows must already be normalised
bool wsb_eligible(const LutTensor &t, uint32_t batch);
int launch_gemv_wsb(prism_cuda_ctx *ctx, GemvMode mode, const LutTensor &t, const LutTensor *t2, const uint16_t *x,
                    uint32_t x_stride, void *y, uint32_t y_stride, const uint16_t *resid, uint32_t batch);

// gemv_tc5.cu: tcgen05/TMEM GEMV (4-bit, K % 32 == 0, one activation vector)
bool tc5_eligible(prism_cuda_ctx *ctx, const LutTensor &t, uint32_t batch);
int launch_gemv_tc5(prism_cuda_ctx *ctx, GemvMode mode, const LutTensor &t, const LutTensor *t2, const uint16_t *x,
                    void *y, const uint16_t *resid);

// gemm_tc5.cu: tcgen05/TMEM prefill GEMM (4-bit, K % 32 == 0, >= 32 tokens)
bool gemm_tc5_eligible(prism_cuda_ctx *ctx, const LutTensor &t, uint32_t m_tok);
int launch_gemm_tc5(prism_cuda_ctx *ctx, const LutTensor &t, const uint16_t *X, uint32_t m_tok, uint16_t *Y);

// glue.cu
int launch_rms_norm(prism_cuda_ctx *ctx, const uint16_t *in, uint16_t *out, uint32_t n, float eps,
                    uint32_t batch);
int launch_rope(prism_cuda_ctx *ctx, uint16_t *x, uint32_t n, const int32_t *pos_dev, int64_t pos_host,
                uint32_t head_dim, float base, uint32_t batch, uint32_t x_stride);
int launch_vec_add(prism_cuda_ctx *ctx, uint16_t *a, const uint16_t *b, uint32_t n);
int launch_silu(prism_cuda_ctx *ctx, uint16_t *x, uint32_t n);
int launch_silu_mul(prism_cuda_ctx *ctx, uint16_t *out, const uint16_t *g, const uint16_t *u, uint32_t n);
int launch_softmax(prism_cuda_ctx *ctx, const uint16_t *in, uint16_t *out, uint32_t n);
int launch_argmax(prism_cuda_ctx *ctx, const uint16_t *logits, uint32_t n, uint32_t stride, uint32_t batch,
                  uint32_t *out_dev);
struct AttnArgs {
    const uint16_t *q;      // [batch] rows of nh*hd, q_stride halfs apart
    uint32_t q_stride;
    const void *k, *v;      // cache base of this layer slot
    uint16_t *out;          // [batch][nh*hd]
    // cached positions = pos*slot_mul + slot_add + 1, pos read from pos_dev (device scalar,
    // so a captured graph can be replayed) or pos_host when pos_dev == nullptr
    const int32_t *pos_dev; int32_t pos_host; uint32_t slot_mul, slot_add;
    uint32_t nh, nkv, hd, batch;
    uint64_t seq_stride;    // elements (fp16) or bytes (int8) between sequences in the cache
    uint32_t int8;          // cache holds [f32 scale][kvd x i8] per position
    uint32_t max_seq;
    // fused kernel only: the `batch` rows are consecutive prompt tokens of cache sequence prefill_seq,
    // row t at position pos + t (causal attention over the cache after their keys/values were appended)
    uint32_t prefill = 0, prefill_seq = 0;
    // fused kernel only: paged cache (page table on the device, [sequence][tbl_stride] page numbers of 2^page_shift rows)
    const int32_t *page_tbl = nullptr;
    uint32_t page_shift = 0, tbl_stride = 0;
    // fused kernel only: the caller guarantees that the kernel enqueued right before this one does not write the
    // cache (a decode step: the q/k/v projection), so cached rows may be requested before the dependency wait
    uint32_t early_cache = 0;
};
int launch_attention(prism_cuda_ctx *ctx, const AttnArgs &a);
struct KvAppendArgs {
    const uint16_t *k, *v;  // [batch] rows of kvd, src_stride halfs apart
    uint32_t src_stride;
    void *kc, *vc;
    const int32_t *pos_dev; int32_t pos_host; uint32_t slot_mul, slot_add;  // slot = pos*mul+add
    uint32_t kvd, batch; uint64_t seq_stride; uint32_t int8; uint32_t max_seq;
};
int launch_kv_append(prism_cuda_ctx *ctx, const KvAppendArgs &a);

// attn.cu: RoPE(q), RoPE(k) when rope_k, cache append and attention in one kernel (fp16 cache,
// head_dim 32/64/128/256).  a.q is this step's (un-rotated) query rows, a.k / a.v the cache of the
// layer slot, k_src / v_src this step's key/value rows (a.q_stride apart, like a.q).
bool attn_fused_eligible(const AttnArgs &a);
int launch_attn_fused(prism_cuda_ctx *ctx, const AttnArgs &a, const uint16_t *k_src, const uint16_t *v_src,
                      uint32_t rope_k, float rope_base);

}  // namespace prism

namespace prism {
// Allocates an empty tensor of the device layout (indices and palettes uninitialised).
int alloc_tensor(prism_cuda_ctx *ctx, const char *name, uint32_t m, uint32_t k, uint32_t bits, int32_t *handle);
int synth_shard(prism_cuda_ctx *ctx, const char *name, uint32_t rows, uint32_t cols, uint32_t bits,
                uint64_t seed, float sigma, uint32_t row0, uint32_t col0, int32_t *handle);
// gemm.cu: Y[m_tok][m] = X[m_tok][k] * W^T (fp16 in/out, fp32 accumulate)
int launch_gemm(prism_cuda_ctx *ctx, const LutTensor &t, const uint16_t *X, uint32_t m_tok, uint16_t *Y);
}  // namespace prism
