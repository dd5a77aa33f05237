/*
 * prism_cuda.h -- C ABI of the B200 (sm_100a) backend for Prism Engine's
 * palettized-LUT matmul path.
 *
 * This is the boundary a Rust `CudaBackend` (a peer of `MetalBackend`,
 * src/lut/engine_impl.rs:26-492) binds through `extern "C"`: plain pointers
 * and sizes, no C++ types.  Each entry point names the reference interface it
 * replaces (paths relative to the reference repository root).
 *
 * Conventions (those of the reference's existing C ABI, prism-ffi/src/lib.rs:18-72):
 *   - every function returns 0 on success and a negative PRISM_E_* code on
 *     failure; constructors hand back NULL/-1 handles on failure;
 *   - prism_cuda_last_error(ctx) gives the text the Rust side would put in
 *     its `Err(String)`;
 *   - fp16 values are IEEE binary16 bit patterns carried as uint16_t
 *     (`&[u16]` in the reference);
 *   - a context is used from one host thread at a time (the reference wraps
 *     its engine in a mutex, src/bin/prism_server.rs:282); calls on one
 *     context are ordered on its stream; entry points taking HOST pointers
 *     block until the result is in the caller's buffer, `_dev` entry points
 *     take DEVICE pointers, enqueue on the context stream and return;
 *   - shape and alignment violations are rejected on the host before any
 *     launch; nothing here falls back to a CPU implementation.
 */
#ifndef PRISM_CUDA_H
#define PRISM_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PRISM_OK 0
#define PRISM_E_NULL (-1)      /* null argument */
#define PRISM_E_ARG (-2)       /* bad shape / size / alignment / unsupported bits */
#define PRISM_E_NOTFOUND (-3)  /* unknown tensor key or handle ("miss {key}") */
#define PRISM_E_CUDA (-4)      /* CUDA runtime error (text in last_error) */
#define PRISM_E_STATE (-5)     /* call not valid in this state (e.g. KV cache full) */
#define PRISM_E_IO (-6)        /* file / container error */
#define PRISM_E_COMM (-7)      /* collective (NCCL) error */
#define PRISM_E_TIMEOUT (-8)   /* a bounded device-side wait gave up */

typedef struct prism_cuda_ctx prism_cuda_ctx;
typedef struct prism_cuda_engine prism_cuda_engine;

/* ---- context: MetalBackend::new (src/lut/engine_impl.rs:51-153) ---------- */

/* Creates a backend on CUDA device `device`.  Fails (no fallback) when the
 * device is missing or is not compute capability 10.x. */
int prism_cuda_create(int device, prism_cuda_ctx **out);
void prism_cuda_destroy(prism_cuda_ctx *ctx);
/* Text of the most recent failure on this context ("" if none).  With a NULL
 * context: the failure text of the last prism_cuda_create on this thread. */
const char *prism_cuda_last_error(prism_cuda_ctx *ctx);
/* The CUDA stream (cudaStream_t) the context launches on. */
void *prism_cuda_stream(prism_cuda_ctx *ctx);
int prism_cuda_synchronize(prism_cuda_ctx *ctx);
/* Tunables: "gemv_variant" (0 = plain CUDA-core kernel; 1 = default: pair-table mma.sync kernels,
 * the warp-specialised persistent one for large matrices and the stream-K one for small;
 * 2 = pair-table tcgen05/TMEM kernel where eligible; 3 = the pair-table mma.sync kernel on a
 * (block, K split) grid; 4 / 5 = the warp-specialised / the stream-K kernel for every shape),
 * "gemm_variant" (1 = tcgen05/TMEM
 * prefill GEMM, default; 0 = activation rows through the GEMV kernel), "fuse" (0/1,
 * default 1: fused epilogues), "pdl" (0/1, default 1: programmatic dependent launch between
 * the kernels of a decode step, so a kernel's weight-only prologue overlaps its predecessor),
 * "batch_gemv_max" (default 8: decode batches up to this many sequences stream the weights once
 * through the batched GEMV, in groups of 8; larger batches use the tcgen05 GEMM),
 * "attn_cluster" (0 = from max_seq, default; 1/2/4/8 CTAs per KV head and sequence in the fused
 * attention kernel),
 * "attn_group" (0 = from the shape, default; 1/2/4/8 = most query heads of a KV group one cluster of the
 * fused attention kernel serves),
 * "tp_peer_ar" (0/1, default 1: tensor-parallel partial sums are reduced by one kernel through
 * peer memory instead of ncclAllReduce + add; set it identically on every rank),
 * "sk_min_chunks" (default 8: fewest 1 KB index chunks the GEMV gives one CTA of a small matrix),
 * "sk_stream_chunks" (default 64: chunks per CTA from which the GEMV deals contiguous, balanced
 * ranges to a persistent grid instead of cutting every 64-row block into equal parts),
 * "cl_max_units" (default 16384: matrices of at most this many (64-row block x 1 KB index chunk) units go to
 * the cluster GEMV, whose CTAs hold all their indices in registers before the previous kernel has
 * finished and reduce through distributed shared memory; 0 = never),
 * "ws_whole_blocks" (default 1024: when a matrix has fewer 64-row blocks than the GPU has SMs, but at least
 * "ws_whole_fill" per 100 (default 50; 85 for batches), and rows of at most this many 1 KB chunks, the
 * warp-specialised GEMV gives every CTA one whole block and leaves the other SMs idle, instead of cutting
 * blocks between CTAs; 0 = never),
 * "wait_limit_polls" (default 0 = built-in, about fifteen seconds: polls after which a kernel stops
 * waiting for a tensor-parallel peer or a grid-wide arrival, records a device error code and goes on;
 * the next synchronising call then returns PRISM_E_TIMEOUT and the context stays usable),
 * "prefill_chunk" (default 512: prism_cuda_engine_generate puts up to this many prompt tokens of a sequence
 * through the layers at once -- tensor-core GEMMs, causal attention over the cache, no LM head -- instead of
 * one step per token as the reference's prefill_cpu does; 0 = one step per token.  Single GPU, fp16 KV),
 * "tp_fused_ar" (batch-1 tensor-parallel decode, how the partial sums of a row-parallel matmul are reduced:
 * 0 = the GEMV leaves fp32 partial sums, one kernel pushes them to the peers and reduces; 1 = the GEMV's epilogue
 * stores its sums into every rank's receive area, a small kernel publishes flags, waits and reduces; 2 = flags,
 * wait and reduction inside the GEMV kernel too; 3 (default) = the GEMV's epilogue stores 8-byte words that carry
 * their epoch, a small kernel polls the words and reduces -- no flags and no system-scope fence; 4 = flagged
 * words polled and reduced at the end of the GEMV kernel itself (matmul and all-reduce in one kernel).  Set it
 * identically on every rank),
 * "cimage_cache" (0/1, default 0: prism_cuda_engine_load_cimage keeps the re-laid image beside the file).
 * A captured decode graph is rebuilt after any option change. */
int prism_cuda_set_option(prism_cuda_ctx *ctx, const char *key, int64_t value);
/* Number of kernels this library has launched on the context so far. */
uint64_t prism_cuda_launch_count(prism_cuda_ctx *ctx);
/* Host arithmetic only (no context, no GPU): how the persistent GEMV kernels deal a matrix of
 * n_blocks 64-row blocks x n_chunks 1 KB index chunks to `slots` resident CTAs.  Writes the number of
 * CTAs and, when `bounds` is given (cap >= CTAs + 1 entries), the first (block, chunk) unit of every
 * CTA's range followed by the total.  No counterpart in the reference; exists so the partition can be
 * checked without a device. */
int prism_cuda_gemv_partition(uint32_t n_blocks, uint32_t n_chunks, uint32_t slots, uint32_t stream_chunks,
                              uint32_t min_chunks, uint32_t *n_ctas, uint32_t *bounds, uint32_t cap);
/* Host arithmetic only: the `slots` value the warp-specialised GEMV hands to the partition above -- all the
 * resident CTA slots, or one per block when the matrix has fewer blocks than slots but at least fill_pct per
 * 100 and rows of at most whole_max_chunks chunks (options "ws_whole_fill", "ws_whole_blocks"). */
uint32_t prism_cuda_gemv_partition_ctas(uint32_t n_blocks, uint32_t n_chunks, uint32_t slots, uint32_t whole_max_chunks,
                                        uint32_t fill_pct);

/* ---- weights: the upload loop of MetalBackend::new (engine_impl.rs:123-133)
 *      and PrismEngine::load (engine_impl.rs:597-676) ---------------------- */

/* Copies one palettized tensor to the device.  `payload` is the UNMODIFIED
 * split-block byte string of the .cimage container (all palettes, then all
 * index rows; src/quantization/cimage.rs:98-125, src/lut/compiler.rs:50-61);
 * it is re-laid in HBM for coalesced 128-bit loads and the caller keeps
 * ownership.  bits = 4 (16-entry palette, the reference's only format) or 2
 * (4-entry palette).  dim_n*bits must be a multiple of 32 (the reference
 * needs dim_n % 8 == 0, cpu_fallback.rs:24).  *handle receives a tensor id. */
int prism_cuda_upload_palettized(prism_cuda_ctx *ctx, const char *name, const uint8_t *payload,
                                 size_t len, uint32_t dim_m, uint32_t dim_n, uint32_t bits,
                                 int32_t *handle);
/* Same, keeping only rows [row0,row0+rows) and columns [col0,col0+cols) of the
 * tensor: the shard a tensor-parallel rank owns.  col0 and cols must be
 * multiples of 128/bits. */
int prism_cuda_upload_palettized_shard(prism_cuda_ctx *ctx, const char *name,
                                       const uint8_t *payload, size_t len, uint32_t dim_m,
                                       uint32_t dim_n, uint32_t bits, uint32_t row0, uint32_t rows,
                                       uint32_t col0, uint32_t cols, int32_t *handle);
/* Synthesises a tensor of the benchmark distribution directly on the device
 * (palette entries N(0, sigma) sorted ascending, uniform indices; seeded).
 * Used where a model is too large to stage through host memory. */
int prism_cuda_synth_palettized(prism_cuda_ctx *ctx, const char *name, uint32_t dim_m,
                                uint32_t dim_n, uint32_t bits, uint64_t seed, float sigma,
                                int32_t *handle);
/* Looks a tensor up by the key it was uploaded under (weight_bufs.get(key),
 * engine_impl.rs:156-159). */
int prism_cuda_find_tensor(prism_cuda_ctx *ctx, const char *name, int32_t *handle);
int prism_cuda_tensor_dims(prism_cuda_ctx *ctx, int32_t handle, uint32_t *dim_m, uint32_t *dim_n,
                           uint32_t *bits);
/* Inverse of the re-lay: writes the tensor back as a reference-format payload
 * (len must equal dim_m*2^bits*2 + dim_m*dim_n*bits/8). */
int prism_cuda_download_payload(prism_cuda_ctx *ctx, int32_t handle, uint8_t *payload, size_t len);

/* ---- offline quantiser: palettize_matrix (src/quantization/palette.rs:230-275) + payload assembly
 *      (src/lut/compiler.rs:50-61) -------------------------------------------------------------
 * Fits a k-entry (k <= 16) palette per row of the fp32 matrix weights[dim_m][dim_n] with the
 * reference's deterministic k-means (fit_palette, palette.rs:75-174; max_iter = 50 there), encodes
 * the row (encode_channel, :189-217) and writes the reference payload (dim_m x 16 fp16 palettes,
 * then dim_m rows of dim_n/2 index bytes), bit-identical to the CPU quantiser.  dim_n must be even;
 * len must be dim_m*32 + dim_m*dim_n/2.  Host pointers; _dev takes device pointers and runs on the
 * context stream. */
int prism_cuda_palettize(prism_cuda_ctx *ctx, const float *weights, uint32_t dim_m, uint32_t dim_n, uint32_t k,
                         uint32_t max_iter, uint8_t *payload, size_t len);
int prism_cuda_palettize_dev(prism_cuda_ctx *ctx, const float *weights_dev, uint32_t dim_m, uint32_t dim_n,
                             uint32_t k, uint32_t max_iter, uint8_t *payload_dev);
/* Dequantised weights, row-major [dim_m][dim_n] fp16 bit patterns: the gather
 * of PrismEngine::embed (engine_impl.rs:1407-1446) / dequantize_matrix
 * (src/quantization/palette.rs:280-292) for every row.  Bit-exact. */
int prism_cuda_dequant(prism_cuda_ctx *ctx, int32_t handle, uint16_t *out_host);
int prism_cuda_dequant_dev(prism_cuda_ctx *ctx, int32_t handle, void *out_dev);
int prism_cuda_free_tensor(prism_cuda_ctx *ctx, int32_t handle);
/* Uploads every Palettized4Bit tensor of a reference-format .cimage file
 * (src/quantization/cimage.rs:242-277) under its own key; *n_out = tensors uploaded. */
int prism_cuda_load_cimage(prism_cuda_ctx *ctx, const char *path, uint32_t *n_out);
/* The same with a cache of the RE-LAID image (the device layout of every tensor) kept in `cache_path`
 * (NULL or "": `path` + ".b200relay"): a later load of the same container reads only its header and the
 * cache, and copies each tensor's index array and palettes to the device as they are -- no payload read,
 * no re-lay kernels.  The cache is keyed by a hash of the container's header and size; a stale or
 * foreign file is ignored and rewritten.  *hit_out = 1 when the cache was used.  Stands where
 * PrismEngine::load re-reads and re-copies every payload on each start (engine_impl.rs:600-616). */
int prism_cuda_load_cimage_cached(prism_cuda_ctx *ctx, const char *path, const char *cache_path, uint32_t *n_out,
                                  int *hit_out);
/* ExecutionPlan of the last container loaded on this context (CImageHeader::execution_plan,
 * src/quantization/cimage.rs:54-60; schema src/lut/graph.rs:552-589), as PrismEngine::load parses it
 * (engine_impl.rs:637-641).  version == 0: the container had no plan or one that does not parse (both
 * tolerated, as in the reference).  The reference keeps the plan and never dispatches on it; neither does
 * this backend -- kv_fp16 tells the caller which KV mode the compiler assumed. */
typedef struct prism_cimage_plan {
    uint32_t version, num_layers, n_nodes, n_gemm_nodes; /* n_gemm_nodes: MetalGemm + CpuGemm assignments */
    int32_t kv_fp16;                                     /* 1 "Fp16", 0 "Int8", -1 absent */
    char architecture[32], attention_strategy[24], lm_head_backend[16];
} prism_cimage_plan;
int prism_cuda_cimage_plan(prism_cuda_ctx *ctx, prism_cimage_plan *out);

/* ---- palettized GEMV: MetalBackend::gemv (engine_impl.rs:155-190), i.e.
 *      lut_gemv_cpu (src/lut/cpu_fallback.rs:12-35) on the device ---------- */

/* y[dim_m] = f16( sum_k f32(x[k]) * f32(palette[row][idx[row,k]]) ), fp32 accumulate. */
int prism_cuda_gemv(prism_cuda_ctx *ctx, int32_t handle, const uint16_t *x, uint16_t *y);
int prism_cuda_gemv_key(prism_cuda_ctx *ctx, const char *key, const uint16_t *x, size_t x_len,
                        uint16_t *y, size_t y_len);
int prism_cuda_gemv_dev(prism_cuda_ctx *ctx, int32_t handle, const void *x_dev, void *y_dev);
/* (No counterpart in the reference.)  The same GEMV for hosts that cannot allocate on this
 * path -- a server whose own pools already hold all of HBM, or a decode loop with a fixed
 * memory budget: split-K scratch comes from a fixed 2 MiB + 16 KiB array inside the
 * library instead of cudaMalloc, and nothing is allocated or freed.  4-bit tensors with
 * dim_n % 32 == 0 only; a shape whose split-K scratch exceeds the array (more than 524 288
 * partial sums or 4096 row blocks) returns PRISM_E_ARG.  All calls on a device share the array:
 * calls on one context are stream-ordered and safe, kernels overlapping from different
 * streams/contexts of one device race.  The first call on a device looks up the array's
 * address; make that call before any stream capture. */
int prism_cuda_gemv_static_dev(prism_cuda_ctx *ctx, int32_t handle, const void *x_dev, void *y_dev);
/* y = f16( f32(f16(W x)) + f32(resid) ): GEMV followed by vec_add_inplace, the
 * OProj / DownProj arms of step() (engine_impl.rs:1158-1162, 1196-1203). */
int prism_cuda_gemv_residual_dev(prism_cuda_ctx *ctx, int32_t handle, const void *x_dev,
                                 const void *resid_dev, void *y_dev);

/* ---- fused gate/up SwiGLU: MetalBackend::fused_gate_up (engine_impl.rs:443-490)
 *      with the CPU path's numerics (engine_impl.rs:1163-1195, 1349-1367) --- */

/* out[i] = f16( f32(f16(silu(g_i))) * f32(u_i) ), g = f16(Wg x), u = f16(Wu x),
 * silu(g) = g/(1+exp(-g)) in fp32; both GEMVs share one pass over x. */
int prism_cuda_fused_gate_up(prism_cuda_ctx *ctx, int32_t gate, int32_t up, const uint16_t *x,
                             uint16_t *out);
int prism_cuda_fused_gate_up_key(prism_cuda_ctx *ctx, const char *gate_key, const char *up_key,
                                 const uint16_t *x, size_t x_len, uint16_t *out, size_t out_len);
int prism_cuda_fused_gate_up_dev(prism_cuda_ctx *ctx, int32_t gate, int32_t up, const void *x_dev,
                                 void *out_dev);
/* Whole MLP: out = f16(Wd * fused_gate_up(x)).  The [inter] activation between
 * the two kernels lives in context-owned scratch memory. */
int prism_cuda_mlp(prism_cuda_ctx *ctx, int32_t gate, int32_t up, int32_t down, const uint16_t *x,
                   uint16_t *out);
int prism_cuda_mlp_dev(prism_cuda_ctx *ctx, int32_t gate, int32_t up, int32_t down,
                       const void *x_dev, void *out_dev);

/* ---- prefill GEMM: the palettized_gemm kernel (templates/palettized_gemm.metal:16-117),
 *      with the CPU prefill's numerics: one lut_gemv_cpu per activation row
 *      (prefill_cpu, engine_impl.rs:1046-1053) ----------------------------- */

/* Y[m_tok][dim_m] = X[m_tok][dim_n] * W^T, fp16 in, fp32 accumulate, fp16 out. */
int prism_cuda_gemm(prism_cuda_ctx *ctx, int32_t handle, const uint16_t *X, uint32_t m_tok,
                    uint16_t *Y);
int prism_cuda_gemm_dev(prism_cuda_ctx *ctx, int32_t handle, const void *X_dev, uint32_t m_tok,
                        void *Y_dev);

/* ---- decode glue: MetalBackend::{norm_metal, rope_metal, softmax_metal,
 *      silu_metal, vec_add_metal, attention, append_kv} (engine_impl.rs:194-441)
 *      with the CPU ops' numerics (src/lut/cpu_fallback.rs:39-143) ---------- */

/* rms_norm_inplace (cpu_fallback.rs:39-54): no learned weight. */
int prism_cuda_rms_norm(prism_cuda_ctx *ctx, const uint16_t *in, uint16_t *out, uint32_t n, float eps);
/* rope_inplace (cpu_fallback.rs:131-143): half-split pairs, base passed explicitly
 * (the reference CPU path always uses 10000). */
int prism_cuda_rope(prism_cuda_ctx *ctx, uint16_t *x, uint32_t n, int64_t pos, uint32_t head_dim,
                    float base);
int prism_cuda_softmax(prism_cuda_ctx *ctx, const uint16_t *in, uint16_t *out, uint32_t n);
int prism_cuda_silu(prism_cuda_ctx *ctx, uint16_t *x, uint32_t n);
int prism_cuda_vec_add(prism_cuda_ctx *ctx, uint16_t *a, const uint16_t *b, uint32_t n);
/* attention_cpu (cpu_fallback.rs:84-127): GQA decode attention of one query
 * token over `seq_len` cached positions, K/V laid [pos][kv_head][head_dim]. */
int prism_cuda_attention(prism_cuda_ctx *ctx, const uint16_t *q, const uint16_t *k,
                         const uint16_t *v, uint32_t seq_len, uint32_t num_heads,
                         uint32_t kv_heads, uint32_t head_dim, uint16_t *out);
/* The backend-held fp16 KV cache of MetalBackend: `new(.., num_layers, kv_stride)` allocates a K and a V
 * buffer per layer (engine_impl.rs:109-119), append_kv(layer, k, v, token_idx) copies one token's rows in
 * (:256-286), and attention_decode reads them.  kv_init sizes the cache ([layer][max_seq][kv_dim] fp16;
 * the reference fixes max_seq at 4096); kv_append copies kv_dim values each of k and v into position
 * token_idx; attention_kv is prism_cuda_attention over the first seq_len positions of that layer's
 * cache.  Where the reference silently ignores a layer or token outside the cache, kv_append returns
 * PRISM_E_ARG.  (RoPE of q on a host slice is prism_cuda_rope above.) */
int prism_cuda_kv_init(prism_cuda_ctx *ctx, uint32_t num_layers, uint32_t kv_dim, uint32_t max_seq);
int prism_cuda_kv_append(prism_cuda_ctx *ctx, uint32_t layer, const uint16_t *k, const uint16_t *v, uint64_t token_idx);
int prism_cuda_attention_kv(prism_cuda_ctx *ctx, uint32_t layer, const uint16_t *q, uint32_t seq_len, uint32_t num_heads,
                            uint32_t kv_heads, uint32_t head_dim, uint16_t *out);
/* One decode step's attention nodes on the backend-held cache, as ONE kernel (the one the engine's step
 * uses): RoPE of q (rope_inplace, cpu_fallback.rs:131-143; `rope_base` explicit), RoPE of k when rope_k
 * is set (the reference caches K un-rotated, engine_impl.rs:1131 precedes :1211), KVCache::append of this
 * token's k and v at position token_idx, and attention_cpu over positions 0..token_idx.  head_dim must be
 * 32, 64, 128 or 256.  q: num_heads*head_dim, k / v: kv_dim values (host). */
int prism_cuda_attention_step_kv(prism_cuda_ctx *ctx, uint32_t layer, const uint16_t *q, const uint16_t *k,
                                 const uint16_t *v, uint64_t token_idx, uint32_t num_heads, uint32_t kv_heads,
                                 uint32_t head_dim, uint32_t rope_k, float rope_base, uint16_t *out);
/* argmax (engine_impl.rs:1448-1459): first strictly greatest. */
int prism_cuda_argmax(prism_cuda_ctx *ctx, const uint16_t *logits, uint32_t n, uint32_t *index);

/* ---- engine: PrismEngine (src/lut/engine_impl.rs:503-512; load :597, generate
 *      :933-1044, step :1076-1405) with every op on the device -------------- */

typedef struct prism_model_config {
    /* the fields UnifiedConfig reads from config.json (src/lut/graph.rs:164-292) */
    uint32_t num_layers, hidden_size, num_heads, num_kv_heads, head_dim, intermediate_size,
        vocab_size;
    float norm_eps, rope_theta;
    uint32_t tie_word_embeddings;
    uint32_t bits;       /* 4 (reference) or 2 */
    uint32_t max_seq;    /* KV capacity in positions (MAX_SEQ = 4096 in the reference) */
    uint32_t max_batch;  /* concurrent sequences (the reference has 1) */
    /* behaviour switches; the reference CPU path is {0, 0, 1, 1} */
    uint32_t rope_use_theta; /* 0: base 10000 regardless of rope_theta (cpu_fallback.rs:137) */
    uint32_t rope_k;         /* 0: K cached un-rotated (engine_impl.rs:1131 precedes :1211) */
    uint32_t kv_int8;        /* 1: int8 + f32 scale per token (engine_impl.rs:516-567) */
    uint32_t down_guard;     /* 1: keep the dim test at engine_impl.rs:1124-1126 that skips
                                DownProj when intermediate_size != hidden_size */
    /* Paged KV cache (not in the reference, whose KVCache is one Vec per layer, engine_impl.rs:514-530):
     * kv_page_size > 0 (a power of two >= 16) keeps the fp16 cache of every layer as a pool of pages of
     * that many positions, handed to sequences as they grow; kv_pool_pages sizes the pool (0 = enough for
     * max_batch sequences of max_seq positions).  A pool smaller than that serves more or longer
     * sequences than a slab per sequence could, until it runs out (PRISM_E_STATE).  fp16 cache only. */
    uint32_t kv_page_size, kv_pool_pages;
} prism_model_config;

/* Tensor roles of TensorRole (src/lut/graph.rs) as used by step(). */
enum {
    PRISM_ROLE_Q = 0, PRISM_ROLE_K = 1, PRISM_ROLE_V = 2, PRISM_ROLE_O = 3, PRISM_ROLE_GATE = 4,
    PRISM_ROLE_UP = 5, PRISM_ROLE_DOWN = 6, PRISM_ROLE_EMBED = 7, PRISM_ROLE_LM_HEAD = 8
};

int prism_cuda_engine_create(prism_cuda_ctx *ctx, const prism_model_config *cfg,
                             prism_cuda_engine **out);
void prism_cuda_engine_destroy(prism_cuda_engine *eng);
/* Binds an uploaded tensor to (role, layer); layer is ignored for EMBED / LM_HEAD. */
int prism_cuda_engine_bind(prism_cuda_engine *eng, uint32_t role, uint32_t layer, int32_t handle);
/* Binds by the reference's tensor keys, "model.layers.{i}.self_attn.q_proj.weight" ...
 * (src/lut/graph.rs:304-531), for every tensor already uploaded to the context. */
int prism_cuda_engine_bind_by_keys(prism_cuda_engine *eng, const char *key_prefix);
/* PrismEngine::load: reads a reference-format .cimage (src/quantization/cimage.rs:242-277),
 * uploads every palettized tensor and binds it. */
int prism_cuda_engine_load_cimage(prism_cuda_engine *eng, const char *path, const char *key_prefix);
/* Fills every weight of the model with seeded synthetic tensors on the device. */
int prism_cuda_engine_synth_weights(prism_cuda_engine *eng, uint64_t seed, float sigma);
/* PrismEngine::generate for `batch` sequences at once: prompts is
 * [batch][n_prompt] token ids, out_tokens receives [batch][max_new].  Prefill is
 * one step per prompt token and the first decode step re-feeds the last prompt
 * token, as the reference does (engine_impl.rs:1015,1034,1046-1053).
 * last_logits (optional) receives the fp16 logits [batch][vocab] of the final step. */
int prism_cuda_engine_generate(prism_cuda_engine *eng, const uint32_t *prompts, uint32_t batch,
                               uint32_t n_prompt, uint32_t max_new, uint32_t *out_tokens,
                               uint16_t *last_logits);
/* Finer-grained driving (what generate() is made of). */
int prism_cuda_engine_reset(prism_cuda_engine *eng, uint32_t batch);
/* One step(): feeds tokens[batch] at the current position, advances it, and
 * returns the greedy next tokens; logits (optional, host) gets [batch][vocab]. */
int prism_cuda_engine_step(prism_cuda_engine *eng, const uint32_t *tokens, uint32_t *next_tokens,
                           uint16_t *logits);
/* Runs `n_steps` decode steps back to back on the device, each feeding the
 * previous step's greedy token (no host round trip between steps); tokens_in
 * [batch] seeds the first step, out_tokens receives [batch][n_steps]. */
int prism_cuda_engine_decode(prism_cuda_engine *eng, const uint32_t *tokens_in, uint32_t n_steps,
                             uint32_t *out_tokens);
/* Algorithmic HBM bytes of one decode step at the current position (weights +
 * KV read), and the device time of the last generate/decode call. */
uint64_t prism_cuda_engine_step_bytes(prism_cuda_engine *eng);
/* Device time of the last generate/decode call: whole call including the
 * host<->device token copies (last_ms) and the kernel region only (last_device_ms). */
double prism_cuda_engine_last_ms(prism_cuda_engine *eng);
double prism_cuda_engine_last_device_ms(prism_cuda_engine *eng);
uint32_t prism_cuda_engine_position(prism_cuda_engine *eng);
/* Kernels one step launches (counted when the step was first enqueued). */
uint32_t prism_cuda_engine_kernels_per_step(prism_cuda_engine *eng);
/* ---- tensor parallelism (not in the reference; column/row-sharded linears
 *      with an all-reduce after each row-parallel matmul) ------------------- */

#define PRISM_NCCL_ID_BYTES 128
/* Rank 0 fills `id` and hands the bytes to the other ranks (any transport). */
int prism_cuda_tp_unique_id(uint8_t id[PRISM_NCCL_ID_BYTES]);
/* Joins this context to a `world`-rank NCCL communicator and, when every rank can map every
 * other rank's memory (one process per GPU, peer access over NVLink), sets up the receive areas of
 * the peer-memory all-reduce the decode step then uses after its row-parallel matmuls. */
int prism_cuda_tp_init(prism_cuda_ctx *ctx, int world, int rank, const uint8_t id[PRISM_NCCL_ID_BYTES]);
int prism_cuda_tp_world(prism_cuda_ctx *ctx, int *world, int *rank);
/* 1 when the peer-memory all-reduce is set up on this context (same answer on every rank), 0 when
 * the step falls back to ncclAllReduce. */
int prism_cuda_tp_peer_ready(prism_cuda_ctx *ctx);
/* Why prism_cuda_tp_peer_ready is 0 ("" when the peer path is set up or tensor parallelism is off). */
const char *prism_cuda_tp_peer_reason(prism_cuda_ctx *ctx);
/* h[i] = f16( f32(f16(sum over ranks of partial[i])) + f32(h[i]) ) for n values (n % 4 == 0), device pointers,
 * on the context stream: the peer-memory all-reduce of a row-parallel matmul's fp32 partial sums fused with
 * the residual add, as the decode step uses it.  Every rank must call it the same number of times.  A rank
 * whose peers do not deliver within the wait limit ("wait_limit_polls") goes on and the next synchronising
 * call (prism_cuda_synchronize, engine step/decode/generate) returns PRISM_E_TIMEOUT. */
int prism_cuda_tp_all_reduce_resid_dev(prism_cuda_ctx *ctx, const void *partial_f32_dev, void *h_f16_dev, size_t n);
/* Bring-up and diagnostics on ONE GPU, without NCCL: makes this context rank `rank` of a `world`-rank group
 * whose peers are all this context's own receive area.  Nothing ever delivers the other ranks' slices, so
 * prism_cuda_tp_all_reduce_resid_dev on such a context exercises exactly the give-up path of the bounded
 * wait.  No engine can be created on it. */
int prism_cuda_tp_init_loopback(prism_cuda_ctx *ctx, int world, int rank);
/* In-place fp16 sum over ranks of a device vector, on the context stream. */
int prism_cuda_tp_all_reduce_dev(prism_cuda_ctx *ctx, void *buf_dev, size_t n_halfs);

#ifdef __cplusplus
}
#endif
#endif /* PRISM_CUDA_H */
