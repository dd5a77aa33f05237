// Device-resident twin of PrismEngine (src/lut/engine_impl.rs:503-512): the
// node walk of step() (:1076-1405) for the Qwen2-family graph that
// ModelGraph::build emits (src/lut/graph.rs:304-531) --
//   Norm, Q, K, V, RoPE, SDPA, O, Norm, Gate, Up, Activation, Down   per layer,
//   final Norm, LM head (or the tied embedding table)
// -- enqueued as one fixed kernel sequence whose position-dependent values are
// read from device memory, so the whole step is captured once in a CUDA graph
// and replayed per token with no host round trip.  generate() follows
// engine_impl.rs:933-1044: prefill is one step per prompt token and the first
// decode step feeds the last prompt token again.
#include <algorithm>
#include <cstring>

#include "../../include/prism_cuda_bench.h"
#include "common.cuh"

namespace prism {
int synth_shard(prism_cuda_ctx *ctx, const char *name, uint32_t rows, uint32_t cols, uint32_t bits,
                uint64_t seed, float sigma, uint32_t row0, uint32_t col0, int32_t *handle);
}  // namespace prism

struct prism_cuda_engine {
    prism_cuda_ctx *ctx = nullptr;
    prism_model_config cfg{};
    int T = 1, rank = 0;
    // local (per-rank) dimensions
    uint32_t H = 0, nh_l = 0, nkv_l = 0, hd = 0, qd_l = 0, kvd_l = 0, I_l = 0, V_l = 0;
    uint32_t head0 = 0, kvhead0 = 0, i0 = 0, v0 = 0;  // first local q head / kv head / inter row / vocab row
    std::vector<int32_t> wq, wk, wv, wo, wg, wu, wd;
    std::vector<int32_t> wqkv;   // q, k, v rows stacked into one tensor (one launch instead of three)
    bool fused_ready = false;
    uint16_t *gu = nullptr;      // [2][B][max(I_l, H)] scratch of the batched (GEMM) path
    uint16_t *qkv = nullptr;     // [B][qkv_stride]: q | k | v of a sequence side by side
    uint32_t qkv_stride = 0;
    int32_t embed = -1, lm_head = -1;
    // activations
    uint16_t *h = nullptr, *xn = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *att = nullptr,
             *act = nullptr, *logits = nullptr;
    float *part = nullptr;       // [B][H] fp32 partial sums of row-parallel matmuls (TP)
    uint32_t *tok = nullptr, *next = nullptr, *out_tokens = nullptr, *prompts = nullptr;
    uint64_t *pairs_send = nullptr, *pairs_recv = nullptr;  // TP argmax: (value bits << 32 | ~index)
    int32_t *scalars = nullptr;  // [0] pos, [1] step, [2] record
    size_t prompts_cap = 0;
    uint32_t act_stride = 0, out_cap = 0;
    void *kc = nullptr, *vc = nullptr;
    size_t kv_layer_bytes = 0;
    uint64_t kv_seq_stride = 0;  // fp16: elements, int8: bytes
    uint32_t kv_slots = 0;       // positions a layer slot can hold
    uint32_t batch = 0, pos = 0;
    bool guard_skip = false;     // down_guard && inter != hidden
    // paged KV cache (cfg.kv_page_size > 0): page table on the device and its host mirror, free pages
    int32_t *page_tbl = nullptr;             // [max_batch][pages_per_seq]
    std::vector<int32_t> page_tbl_host, free_pages;
    std::vector<uint32_t> seq_pages;         // pages each sequence holds
    uint32_t page_shift = 0, pages_per_seq = 0, pool_pages = 0;
    // batched prefill scratch (one chunk of prompt tokens of one sequence), grown on demand
    uint16_t *pf_x = nullptr, *pf_xn = nullptr, *pf_qkv = nullptr, *pf_att = nullptr, *pf_g = nullptr, *pf_u = nullptr,
             *pf_act = nullptr;
    uint32_t *pf_tok = nullptr;
    uint32_t pf_cap = 0;         // tokens the buffers hold
    cudaGraphExec_t graph = nullptr;
    uint32_t graph_batch = 0;
    uint64_t graph_epoch = ~0ull;  // option epoch of the context when the graph (or its eager warm-up) was made
    cudaEvent_t ev0 = nullptr, ev1 = nullptr, ev2 = nullptr, ev3 = nullptr;
    double last_ms = 0.0, last_device_ms = 0.0;
    uint32_t kernels_per_step = 0;
};

namespace prism {

static void split_units(uint32_t total_units, int T, int r, uint32_t *u0, uint32_t *u1) {
    *u0 = (uint32_t)((uint64_t)total_units * r / T);
    *u1 = (uint32_t)((uint64_t)total_units * (r + 1) / T);
}

// h = f16( f32(f16(sum)) + f32(h) ): the rounding of a GEMV output followed by
// vec_add_inplace with the residual (engine_impl.rs:1158-1162), applied to the
// all-reduced fp32 sums of a row-parallel matmul.
__global__ void round_add_resid_kernel(const float *__restrict__ sum, uint16_t *__restrict__ h, uint32_t n) {
    pdl_launch_dependents();
    pdl_wait();
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        float y = __half2float(__float2half_rn(sum[i]));
        h[i] = __half_as_ushort(__float2half_rn(y + __half2float(__ushort_as_half(h[i]))));
    }
}

// End of a step: pos += 1; when recording, out_tokens[b][step] = next[b],
// tok[b] = next[b] (the greedy token feeds the next step), step += 1.
__global__ void advance_kernel(int32_t *scalars, const uint32_t *__restrict__ next, uint32_t *__restrict__ tok,
                               uint32_t *__restrict__ out_tokens, uint32_t batch, uint32_t out_cap) {
    pdl_launch_dependents();
    pdl_wait();
    const int32_t step = scalars[1], record = scalars[2];
    if (record) {
        for (uint32_t b = threadIdx.x; b < batch; b += blockDim.x) {
            const uint32_t t = next[b];
            tok[b] = t;
            if ((uint32_t)step < out_cap) out_tokens[(size_t)b * out_cap + step] = t;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        scalars[0] += 1;
        if (record) scalars[1] = step + 1;
    }
}

// Tensor-parallel argmax.  Each rank reduces its vocabulary slice to one
// (value, global index) pair per sequence, packed so that a plain unsigned
// max picks the greatest value and, among equals, the smallest index --
// argmax's "first strictly greatest" (engine_impl.rs:1448-1459).
__device__ __forceinline__ uint64_t pack_pair(float v, uint32_t idx) {
    uint32_t b = __float_as_uint(v);
    b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);  // monotone map of float order to unsigned order
    return ((uint64_t)b << 32) | (uint32_t)(~idx);
}
__global__ void local_pair_kernel(const uint16_t *__restrict__ logits, uint32_t n, uint32_t stride,
                                  uint32_t idx0, uint64_t *__restrict__ pairs) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ uint64_t sh[32];
    const uint16_t *lg = logits + (size_t)blockIdx.x * stride;
    uint64_t best = 0;  // below every real value; index 0 wins if nothing compares greater than -inf
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        float f = __half2float(__ushort_as_half(lg[i]));
        if (f > -INFINITY) {  // NaN and -inf never win, as in the reference
            uint64_t p = pack_pair(f, idx0 + i);
            best = p > best ? p : best;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        uint64_t other = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        best = other > best ? other : best;
    }
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (uint32_t w = 1; w < (blockDim.x >> 5); w++) best = sh[w] > best ? sh[w] : best;
        pairs[blockIdx.x] = best;
    }
}
__global__ void final_pair_kernel(const uint64_t *__restrict__ pairs, uint32_t batch, int T,
                                  uint32_t *__restrict__ next) {
    pdl_launch_dependents();
    pdl_wait();
    uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= batch) return;
    uint64_t best = 0;
    for (int r = 0; r < T; r++) {
        uint64_t p = pairs[(size_t)r * batch + b];
        best = p > best ? p : best;
    }
    next[b] = best ? ~(uint32_t)(best & 0xFFFFFFFFu) : 0u;
}

// Row-parallel matmul epilogue of a tensor-parallel rank: h = f16(f16(sum over ranks of part) + h).
// One kernel through peer memory when the ranks could map each other, else ncclAllReduce + add.
static int tp_reduce_add_resid(prism_cuda_engine *e, uint32_t n) {
    prism_cuda_ctx *ctx = e->ctx;
    if (tp_peer_ar_ok(ctx, n)) return tp_all_reduce_resid_peer(ctx, e->part, e->h, n);
    PRISM_TRY(tp_all_reduce_f32(ctx, e->part, n));
    launch_pdl(ctx, "round_add_resid_kernel", round_add_resid_kernel, (n + 255) / 256, 256, 0, e->part, e->h, n);
    return after_launch(ctx, "round_add_resid_kernel");
}

// One palettized linear of the step.  A batch of 8 or more sequences goes through the tensor-core
// GEMM (weights streamed once for the whole batch) followed by the same elementwise kernels the
// unfused path uses, so the fp16 rounding points stay those of the reference; smaller batches use
// the GEMV kernels with their fused epilogues.
static int linear(prism_cuda_engine *e, GemvMode mode, const LutTensor &t, const LutTensor *t2, const uint16_t *x,
                  uint32_t xs, uint16_t *y, uint32_t ys, const uint16_t *resid, uint32_t B) {
    prism_cuda_ctx *ctx = e->ctx;
    const bool gemm_ok = B > (uint32_t)ctx->batch_gemv_max && ctx->gemm_variant == 1 && e->gu && gemm_tc5_eligible(ctx, t, B) && xs == t.k &&
                         (mode == GEMV_SWIGLU ? ys == t.m : ys == t.m);
    if (!gemm_ok) return launch_gemv(ctx, mode, t, t2, x, xs, y, ys, resid, B);
    if (mode == GEMV_PLAIN) return launch_gemm(ctx, t, x, B, y);
    if (mode == GEMV_RESID) {  // y (== resid, in place) = f16( f16(W x) + resid )
        PRISM_TRY(launch_gemm(ctx, t, x, B, e->gu));
        if (y == resid) return launch_vec_add(ctx, y, e->gu, B * t.m);  // in place: the add commutes
        PRISM_TRY(launch_vec_add(ctx, e->gu, resid, B * t.m));
        PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(y, e->gu, (size_t)B * t.m * 2, cudaMemcpyDeviceToDevice, ctx->stream));
        return PRISM_OK;
    }
    // SwiGLU: gate and up GEMMs, then f16(f16(silu(g)) * u)
    uint16_t *g = e->gu, *u = e->gu + (size_t)B * t.m;
    PRISM_TRY(launch_gemm(ctx, t, x, B, g));
    ctx->gemm_reuse_x = 1;  // same activations, same token tile: the re-laid copy is still in scratch
    const int rc_up = launch_gemm(ctx, *t2, x, B, u);
    ctx->gemm_reuse_x = 0;
    PRISM_TRY(rc_up);
    return launch_silu_mul(ctx, y, g, u, B * t.m);
}

// Rope(q), Rope(k), KV append and Attention of layer l (cache slot li): one fused kernel when the
// configuration allows, else the four separate ones.
static int enqueue_attention(prism_cuda_engine *e, uint32_t l, uint32_t li) {
    prism_cuda_ctx *ctx = e->ctx;
    const prism_model_config &c = e->cfg;
    const uint32_t B = e->batch, qs = e->qkv_stride;
    const float base = c.rope_use_theta ? c.rope_theta : 10000.0f;
    const int32_t *pos_dev = e->scalars;
    const uint32_t slot_mul = e->guard_skip ? c.num_layers : 1, slot_add = e->guard_skip ? l : 0;
    KvAppendArgs ka{};
    ka.k = e->k; ka.v = e->v; ka.src_stride = qs;
    ka.kc = (char *)e->kc + (size_t)li * e->kv_layer_bytes;
    ka.vc = (char *)e->vc + (size_t)li * e->kv_layer_bytes;
    ka.pos_dev = pos_dev; ka.slot_mul = slot_mul; ka.slot_add = slot_add;
    ka.kvd = e->kvd_l; ka.batch = B; ka.seq_stride = e->kv_seq_stride; ka.int8 = c.kv_int8; ka.max_seq = e->kv_slots;
    AttnArgs aa{};
    aa.q = e->q; aa.q_stride = qs; aa.k = ka.kc; aa.v = ka.vc; aa.out = e->att;
    aa.pos_dev = pos_dev; aa.slot_mul = slot_mul; aa.slot_add = slot_add;
    aa.nh = e->nh_l; aa.nkv = e->nkv_l; aa.hd = e->hd; aa.batch = B;
    aa.seq_stride = e->kv_seq_stride; aa.int8 = c.kv_int8; aa.max_seq = e->kv_slots;
    aa.page_tbl = e->page_tbl; aa.page_shift = e->page_shift; aa.tbl_stride = e->pages_per_seq;
    aa.early_cache = 1;  // what precedes this launch in a step is the q/k/v projection, which leaves the cache alone
    if (ctx->fuse != 0 && attn_fused_eligible(aa)) return launch_attn_fused(ctx, aa, e->k, e->v, c.rope_k, base);
    if (e->page_tbl) return fail(ctx, PRISM_E_STATE, "the paged KV cache needs the fused attention kernel (option fuse = 1)");
    if (c.rope_k) PRISM_TRY(launch_rope(ctx, e->k, e->kvd_l, pos_dev, 0, e->hd, base, B, qs));
    PRISM_TRY(launch_kv_append(ctx, ka));
    PRISM_TRY(launch_rope(ctx, e->q, e->qd_l, pos_dev, 0, e->hd, base, B, qs));
    return launch_attention(ctx, aa);
}

static int enqueue_step(prism_cuda_engine *e) {
    prism_cuda_ctx *ctx = e->ctx;
    const prism_model_config &c = e->cfg;
    const uint32_t B = e->batch, H = e->H;
    const bool tp = e->T > 1;
    const bool fused = ctx->fuse != 0;
    const LutTensor &emb = ctx->tensors[e->embed];
    PRISM_TRY(launch_embed(ctx, emb, e->tok, B, e->h, nullptr));
    uint32_t li = 0;
    for (uint32_t l = 0; l < c.num_layers; l++) {
        const LutTensor &tq = ctx->tensors[e->wq[l]], &tk = ctx->tensors[e->wk[l]], &tv = ctx->tensors[e->wv[l]],
                        &to = ctx->tensors[e->wo[l]], &tg = ctx->tensors[e->wg[l]], &tu = ctx->tensors[e->wu[l]];
        const uint32_t qs = e->qkv_stride;
        // the Norm node is folded into the x staging of the matmul that consumes it (small batches)
        const bool fold = fused && B == 1;  // batches go through the one-pass batched GEMV, which takes normalised rows
        if (fold && e->wqkv[l] >= 0) {
            ctx->pending_norm_eps = c.norm_eps;
            PRISM_TRY(launch_gemv(ctx, GEMV_PLAIN, ctx->tensors[e->wqkv[l]], nullptr, e->h, H, e->qkv, qs, nullptr, B));
        } else if (e->wqkv[l] >= 0) {
            PRISM_TRY(launch_rms_norm(ctx, e->h, e->xn, H, c.norm_eps, B));
            PRISM_TRY(linear(e, GEMV_PLAIN, ctx->tensors[e->wqkv[l]], nullptr, e->xn, H, e->qkv, qs, nullptr, B));
        } else {
            PRISM_TRY(launch_rms_norm(ctx, e->h, e->xn, H, c.norm_eps, B));
            PRISM_TRY(linear(e, GEMV_PLAIN, tq, nullptr, e->xn, H, e->q, qs, nullptr, B));
            PRISM_TRY(linear(e, GEMV_PLAIN, tk, nullptr, e->xn, H, e->k, qs, nullptr, B));
            PRISM_TRY(linear(e, GEMV_PLAIN, tv, nullptr, e->xn, H, e->v, qs, nullptr, B));
        }
        PRISM_TRY(enqueue_attention(e, l, li));
        if (tp && B == 1 && gemv_tp_ok(ctx, to)) {
            // partial products, their all-reduce over the ranks and the residual add in one kernel
            PRISM_TRY(launch_gemv(ctx, GEMV_TP, to, nullptr, e->att, e->qd_l, e->h, H, e->h, B));
            if (ctx->tp_fused_ar == 1) PRISM_TRY(tp_all_reduce_flags_resid(ctx, e->h, H));
            if (ctx->tp_fused_ar == 3) PRISM_TRY(tp_all_reduce_ll_resid(ctx, e->h, H));
        } else if (tp) {
            PRISM_TRY(launch_gemv(ctx, GEMV_F32, to, nullptr, e->att, e->qd_l, (uint16_t *)e->part, H, nullptr, B));
            PRISM_TRY(tp_reduce_add_resid(e, B * H));
        } else if (fused) {
            PRISM_TRY(linear(e, GEMV_RESID, to, nullptr, e->att, e->qd_l, e->h, H, e->h, B));
        } else {
            PRISM_TRY(linear(e, GEMV_PLAIN, to, nullptr, e->att, e->qd_l, e->xn, H, nullptr, B));
            PRISM_TRY(launch_vec_add(ctx, e->xn, e->h, B * H));  // xn = f16(o + hr)
            PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(e->h, e->xn, (size_t)B * H * 2, cudaMemcpyDeviceToDevice, ctx->stream));
        }
        if (fold) {
            ctx->pending_norm_eps = c.norm_eps;
            PRISM_TRY(launch_gemv(ctx, GEMV_SWIGLU, tg, &tu, e->h, H, e->act, e->act_stride, nullptr, B));
        } else {
            PRISM_TRY(launch_rms_norm(ctx, e->h, e->xn, H, c.norm_eps, B));
            PRISM_TRY(linear(e, GEMV_SWIGLU, tg, &tu, e->xn, H, e->act, e->act_stride, nullptr, B));
        }
        if (e->guard_skip) continue;  // DownProj skipped by the dim test (engine_impl.rs:1124-1126)
        const LutTensor &td = ctx->tensors[e->wd[l]];
        if (tp && B == 1 && gemv_tp_ok(ctx, td)) {
            PRISM_TRY(launch_gemv(ctx, GEMV_TP, td, nullptr, e->act, e->act_stride, e->h, H, e->h, B));
            if (ctx->tp_fused_ar == 1) PRISM_TRY(tp_all_reduce_flags_resid(ctx, e->h, H));
            if (ctx->tp_fused_ar == 3) PRISM_TRY(tp_all_reduce_ll_resid(ctx, e->h, H));
        } else if (tp) {
            PRISM_TRY(launch_gemv(ctx, GEMV_F32, td, nullptr, e->act, e->act_stride, (uint16_t *)e->part, H, nullptr, B));
            PRISM_TRY(tp_reduce_add_resid(e, B * H));
        } else if (fused) {
            PRISM_TRY(linear(e, GEMV_RESID, td, nullptr, e->act, e->act_stride, e->h, H, e->h, B));
        } else {
            PRISM_TRY(linear(e, GEMV_PLAIN, td, nullptr, e->act, e->act_stride, e->xn, H, nullptr, B));
            PRISM_TRY(launch_vec_add(ctx, e->xn, e->h, B * H));
            PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(e->h, e->xn, (size_t)B * H * 2, cudaMemcpyDeviceToDevice, ctx->stream));
        }
        li += 1;
    }
    const bool fold_head = fused && B == 1;
    if (!fold_head) PRISM_TRY(launch_rms_norm(ctx, e->h, e->xn, H, c.norm_eps, B));
    const LutTensor &head = ctx->tensors[(c.tie_word_embeddings || e->lm_head < 0) ? e->embed : e->lm_head];
    const uint32_t lstride = round_up_u32(e->V_l, 8);
    if (fold_head) {
        ctx->pending_norm_eps = c.norm_eps;
        PRISM_TRY(launch_gemv(ctx, GEMV_PLAIN, head, nullptr, e->h, H, e->logits, lstride, nullptr, B));
    } else {
        PRISM_TRY(linear(e, GEMV_PLAIN, head, nullptr, e->xn, H, e->logits, lstride, nullptr, B));
    }
    if (tp) {
        launch_pdl(ctx, "local_pair_kernel", local_pair_kernel, B, 1024, 0, e->logits, e->V_l, lstride, e->v0, e->pairs_send);
        PRISM_TRY(after_launch(ctx, "local_pair_kernel"));
        PRISM_TRY(tp_all_gather_bytes(ctx, e->pairs_send, e->pairs_recv, (size_t)B * 8));
        launch_pdl(ctx, "final_pair_kernel", final_pair_kernel, (B + 63) / 64, 64, 0, e->pairs_recv, B, e->T, e->next);
        PRISM_TRY(after_launch(ctx, "final_pair_kernel"));
    } else {
        PRISM_TRY(launch_argmax(ctx, e->logits, e->V_l, lstride, B, e->next));
    }
    launch_pdl(ctx, "advance_kernel", advance_kernel, 1, 64, 0, e->scalars, e->next, e->tok, e->out_tokens, B, e->out_cap);
    return after_launch(ctx, "advance_kernel");
}

// Stacks the rows of q, k and v of a layer into one tensor (device-to-device copies of
// whole half-blocks), so the three projections of the same activation are one launch.
static int build_fused_qkv(prism_cuda_engine *e) {
    prism_cuda_ctx *ctx = e->ctx;
    for (uint32_t l = 0; l < e->cfg.num_layers; l++) {
        if (e->wqkv[l] >= 0) continue;
        const LutTensor tq = ctx->tensors[e->wq[l]], tk = ctx->tensors[e->wk[l]], tv = ctx->tensors[e->wv[l]];
        if (tq.m % 32 || tk.m % 32 || tv.m % 32) continue;  // rows must fill whole half-blocks
        if (tk.k != tq.k || tv.k != tq.k || tk.bits != tq.bits || tv.bits != tq.bits) continue;
        int32_t h;
        PRISM_TRY(alloc_tensor(ctx, "", tq.m + tk.m + tv.m, tq.k, tq.bits, &h));
        LutTensor &f = ctx->tensors[h];
        uint8_t *di = f.idx;
        uint16_t *dp = f.pal;
        PRISM_CUDA_TRY(ctx, cudaMemsetAsync(f.idx, 0, f.idx_bytes, ctx->stream));
        PRISM_CUDA_TRY(ctx, cudaMemsetAsync(f.pal, 0, f.pal_bytes, ctx->stream));
        for (const LutTensor *t : {&tq, &tk, &tv}) {
            const size_t ib = (size_t)(t->m / 32) * t->n_chunks * 512, pb = (size_t)t->m * t->n_ent() * 2;
            PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(di, t->idx, ib, cudaMemcpyDeviceToDevice, ctx->stream));
            PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(dp, t->pal, pb, cudaMemcpyDeviceToDevice, ctx->stream));
            di += ib;
            dp += (size_t)t->m * t->n_ent();
        }
        e->wqkv[l] = h;
    }
    return PRISM_OK;
}

static int check_bound(prism_cuda_engine *e) {
    if (e->embed < 0) return fail(e->ctx, PRISM_E_STATE, "emb miss: no embedding tensor bound");
    for (uint32_t l = 0; l < e->cfg.num_layers; l++) {
        if (e->wq[l] < 0 || e->wk[l] < 0 || e->wv[l] < 0 || e->wo[l] < 0 || e->wg[l] < 0 || e->wu[l] < 0 ||
            (!e->guard_skip && e->wd[l] < 0))
            return fail(e->ctx, PRISM_E_STATE, "layer " + std::to_string(l) + " has unbound tensors");
    }
    if (!e->fused_ready) {
        PRISM_TRY(build_fused_qkv(e));
        e->fused_ready = true;
    }
    return PRISM_OK;
}

// Paged cache: every sequence of the current batch gets the pages its first `upto` positions need.
static int ensure_pages(prism_cuda_engine *e, uint32_t upto) {
    if (!e->page_tbl) return PRISM_OK;
    const uint32_t P = 1u << e->page_shift, need = (upto + P - 1) / P;
    bool changed = false;
    for (uint32_t b = 0; b < e->batch; b++) {
        while (e->seq_pages[b] < need) {
            if (e->free_pages.empty())
                return fail(e->ctx, PRISM_E_STATE, "KV page pool exhausted: " + std::to_string(e->pool_pages) + " pages of " +
                                                       std::to_string(P) + " positions are all in use");
            e->page_tbl_host[(size_t)b * e->pages_per_seq + e->seq_pages[b]] = e->free_pages.back();
            e->free_pages.pop_back();
            e->seq_pages[b] += 1;
            changed = true;
        }
    }
    if (changed) {
        // the mirror outlives the copy (it belongs to the engine), so the asynchronous copy may read it later
        PRISM_CUDA_TRY(e->ctx, cudaMemcpyAsync(e->page_tbl, e->page_tbl_host.data(), e->page_tbl_host.size() * sizeof(int32_t),
                                               cudaMemcpyHostToDevice, e->ctx->stream));
        PRISM_CUDA_TRY(e->ctx, cudaStreamSynchronize(e->ctx->stream));
    }
    return PRISM_OK;
}
static void release_pages(prism_cuda_engine *e) {
    if (!e->page_tbl) return;
    e->free_pages.clear();
    for (uint32_t p = e->pool_pages; p > 0; p--) e->free_pages.push_back((int32_t)(p - 1));
    std::fill(e->seq_pages.begin(), e->seq_pages.end(), 0u);
}

static int capacity_ok(prism_cuda_engine *e, uint32_t steps) {
    const uint64_t need = e->guard_skip ? (uint64_t)(e->pos + steps) * e->cfg.num_layers : (uint64_t)e->pos + steps;
    if (need > e->kv_slots)
        return fail(e->ctx, PRISM_E_STATE, "KV cache full: " + std::to_string(need) + " > " + std::to_string(e->kv_slots));
    return ensure_pages(e, (uint32_t)need);
}

// Runs one step: the first call per (batch, options) runs eagerly (this sizes
// every scratch buffer and sets kernel attributes), the second captures the
// graph, later ones replay it.
static int run_step(prism_cuda_engine *e) {
    prism_cuda_ctx *ctx = e->ctx;
    // every option can change which kernels a step launches, so a graph is good for one option epoch
    const bool same_cfg = e->graph_batch == e->batch && e->graph_epoch == ctx->option_epoch;
    if (e->graph && same_cfg) {
        PRISM_CUDA_TRY(ctx, cudaGraphLaunch(e->graph, ctx->stream));
        ctx->launches += 1;
        return PRISM_OK;
    }
    if (!same_cfg) {
        // configuration changed: drop the old graph and warm up eagerly once
        if (e->graph) {
            cudaGraphExecDestroy(e->graph);
            e->graph = nullptr;
        }
        e->graph_batch = e->batch;
        e->graph_epoch = ctx->option_epoch;
        const uint64_t l0 = ctx->launches;
        PRISM_TRY(enqueue_step(e));
        e->kernels_per_step = (uint32_t)(ctx->launches - l0);
        return PRISM_OK;
    }
    cudaGraph_t g = nullptr;
    PRISM_CUDA_TRY(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    const uint64_t before = ctx->launches;
    int rc = enqueue_step(e);
    cudaError_t ce = cudaStreamEndCapture(ctx->stream, &g);
    ctx->launches = before;
    if (rc != PRISM_OK) {
        if (g) cudaGraphDestroy(g);
        return rc;
    }
    if (ce != cudaSuccess) return cuda_fail(ctx, ce, "cudaStreamEndCapture");
    ce = cudaGraphInstantiate(&e->graph, g, 0);
    cudaGraphDestroy(g);
    if (ce != cudaSuccess) {
        e->graph = nullptr;
        return cuda_fail(ctx, ce, "cudaGraphInstantiate");
    }
    PRISM_CUDA_TRY(ctx, cudaGraphLaunch(e->graph, ctx->stream));
    ctx->launches += 1;
    return PRISM_OK;
}

static int set_scalars(prism_cuda_engine *e, int32_t pos, int32_t step, int32_t record);

// ---- batched prefill -------------------------------------------------------------------------------
// The reference prefills with one step() per prompt token (prefill_cpu, engine_impl.rs:1046-1053) and
// throws every prefill logit away; all that survives is the KV cache.  Here a chunk of T prompt tokens
// of one sequence goes through every layer at once: the linears are T-row GEMMs on the tensor cores
// (each row = the GEMV of that token, up to fp32 summation order), the keys and values of the T tokens
// are rotated and appended together, token t attends causally to positions 0 .. pos0 + t, and the LM
// head is skipped.  Rounding points are those of step(): fp16 after every matmul, norm, residual add,
// SiLU and gate*up product.
static bool prefill_batched_ok(prism_cuda_engine *e) {
    prism_cuda_ctx *ctx = e->ctx;
    const prism_model_config &c = e->cfg;
    if (ctx->prefill_chunk <= 0 || e->T != 1 || c.kv_int8 || e->guard_skip || !ctx->fuse) return false;
    if (!(e->hd == 32 || e->hd == 64 || e->hd == 128 || e->hd == 256)) return false;
    for (uint32_t l = 0; l < c.num_layers; l++)
        if (e->wqkv[l] < 0 || ctx->tensors[e->wqkv[l]].m % 8) return false;
    return e->I_l % 8 == 0 && e->H % 8 == 0 && e->qd_l % 8 == 0;
}

static int ensure_prefill(prism_cuda_engine *e, uint32_t T) {
    if (T <= e->pf_cap) return PRISM_OK;
    prism_cuda_ctx *ctx = e->ctx;
    PRISM_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    void **ptrs[] = {(void **)&e->pf_x, (void **)&e->pf_xn, (void **)&e->pf_qkv, (void **)&e->pf_att, (void **)&e->pf_g,
                     (void **)&e->pf_u, (void **)&e->pf_act, (void **)&e->pf_tok};
    for (void **p : ptrs) {
        cudaFree(*p);
        *p = nullptr;
    }
    e->pf_cap = 0;
    const uint32_t wq = e->qd_l + 2 * e->kvd_l;
    const size_t wide = std::max<size_t>(e->I_l, e->H);
    const size_t bytes[] = {(size_t)T * e->H * 2, (size_t)T * e->H * 2, (size_t)T * wq * 2, (size_t)T * e->qd_l * 2,
                            (size_t)T * wide * 2, (size_t)T * wide * 2, (size_t)T * wide * 2, (size_t)T * 4};
    for (size_t i = 0; i < sizeof(ptrs) / sizeof(ptrs[0]); i++) {
        cudaError_t ce = cudaMalloc(ptrs[i], (bytes[i] + 255) / 256 * 256);
        if (ce != cudaSuccess) return cuda_fail(ctx, ce, "cudaMalloc(prefill scratch)");
    }
    e->pf_cap = T;
    return PRISM_OK;
}

// Prompt tokens [pos0, pos0 + T) of sequence b (device array `toks`, contiguous) through all layers.
static int prefill_chunk(prism_cuda_engine *e, uint32_t b, uint32_t pos0, uint32_t T, const uint32_t *toks) {
    prism_cuda_ctx *ctx = e->ctx;
    const prism_model_config &c = e->cfg;
    const uint32_t H = e->H, I = e->I_l, wq = e->qd_l + 2 * e->kvd_l;
    const float base = c.rope_use_theta ? c.rope_theta : 10000.0f;
    PRISM_TRY(set_scalars(e, (int32_t)pos0, 0, 0));
    PRISM_TRY(launch_embed(ctx, ctx->tensors[e->embed], toks, T, e->pf_x, nullptr));
    for (uint32_t l = 0; l < c.num_layers; l++) {
        const LutTensor &tqkv = ctx->tensors[e->wqkv[l]], &to = ctx->tensors[e->wo[l]], &tg = ctx->tensors[e->wg[l]],
                        &tu = ctx->tensors[e->wu[l]], &td = ctx->tensors[e->wd[l]];
        PRISM_TRY(launch_rms_norm(ctx, e->pf_x, e->pf_xn, H, c.norm_eps, T));
        PRISM_TRY(launch_gemm(ctx, tqkv, e->pf_xn, T, e->pf_qkv));
        AttnArgs aa{};
        aa.q = e->pf_qkv; aa.q_stride = wq;
        aa.k = (char *)e->kc + (size_t)l * e->kv_layer_bytes;
        aa.v = (char *)e->vc + (size_t)l * e->kv_layer_bytes;
        aa.out = e->pf_att;
        aa.pos_dev = e->scalars; aa.slot_mul = 1; aa.slot_add = 0;
        aa.nh = e->nh_l; aa.nkv = e->nkv_l; aa.hd = e->hd; aa.batch = T;
        aa.seq_stride = e->kv_seq_stride; aa.int8 = 0; aa.max_seq = e->kv_slots;
        aa.prefill = 1; aa.prefill_seq = b;
        aa.page_tbl = e->page_tbl; aa.page_shift = e->page_shift; aa.tbl_stride = e->pages_per_seq;
        PRISM_TRY(launch_attn_fused(ctx, aa, e->pf_qkv + e->qd_l, e->pf_qkv + e->qd_l + e->kvd_l, c.rope_k, base));
        PRISM_TRY(launch_gemm(ctx, to, e->pf_att, T, e->pf_g));
        PRISM_TRY(launch_vec_add(ctx, e->pf_x, e->pf_g, T * H));            // h = f16(o + hr)
        PRISM_TRY(launch_rms_norm(ctx, e->pf_x, e->pf_xn, H, c.norm_eps, T));
        PRISM_TRY(launch_gemm(ctx, tg, e->pf_xn, T, e->pf_g));
        ctx->gemm_reuse_x = 1;  // same activations, same token tile: the re-laid copy is still in scratch
        const int rc_up = launch_gemm(ctx, tu, e->pf_xn, T, e->pf_u);
        ctx->gemm_reuse_x = 0;
        PRISM_TRY(rc_up);
        PRISM_TRY(launch_silu_mul(ctx, e->pf_act, e->pf_g, e->pf_u, T * I));
        PRISM_TRY(launch_gemm(ctx, td, e->pf_act, T, e->pf_g));
        PRISM_TRY(launch_vec_add(ctx, e->pf_x, e->pf_g, T * H));            // h = f16(d + hr)
    }
    return PRISM_OK;
}

// All prompts of a generate call; e->prompts holds them position-major ([position][sequence]).
static int prefill_batched(prism_cuda_engine *e, uint32_t batch, uint32_t n_prompt) {
    prism_cuda_ctx *ctx = e->ctx;
    const uint32_t chunk = std::min<uint32_t>((uint32_t)ctx->prefill_chunk, n_prompt);
    PRISM_TRY(ensure_prefill(e, chunk));
    for (uint32_t b = 0; b < batch; b++) {
        for (uint32_t p0 = 0; p0 < n_prompt; p0 += chunk) {
            const uint32_t T = std::min(chunk, n_prompt - p0);
            // this sequence's tokens of the chunk, made contiguous
            PRISM_CUDA_TRY(ctx, cudaMemcpy2DAsync(e->pf_tok, 4, e->prompts + (size_t)p0 * batch + b, (size_t)batch * 4, 4, T,
                                                  cudaMemcpyDeviceToDevice, ctx->stream));
            PRISM_TRY(prefill_chunk(e, b, p0, T, e->pf_tok));
        }
    }
    // the first decode step feeds the last prompt token again, at position n_prompt (engine_impl.rs:1015, 1034)
    PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(e->tok, e->prompts + (size_t)(n_prompt - 1) * batch, (size_t)batch * 4,
                                        cudaMemcpyDeviceToDevice, ctx->stream));
    return set_scalars(e, (int32_t)n_prompt, 0, 0);
}

static int set_scalars(prism_cuda_engine *e, int32_t pos, int32_t step, int32_t record) {
    int32_t v[3] = {pos, step, record};
    // pageable source: the copy is complete on return, `v` may go out of scope
    PRISM_CUDA_TRY(e->ctx, cudaMemcpyAsync(e->scalars, v, sizeof v, cudaMemcpyHostToDevice, e->ctx->stream));
    PRISM_CUDA_TRY(e->ctx, cudaStreamSynchronize(e->ctx->stream));
    return PRISM_OK;
}

}  // namespace prism

using namespace prism;

extern "C" {

int prism_cuda_engine_create(prism_cuda_ctx *ctx, const prism_model_config *cfg, prism_cuda_engine **out) {
    if (!ctx || !cfg || !out) return fail(ctx, PRISM_E_NULL, "null argument");
    *out = nullptr;
    const prism_model_config &c = *cfg;
    if (!c.num_layers || !c.hidden_size || !c.num_heads || !c.num_kv_heads || !c.head_dim ||
        !c.intermediate_size || !c.vocab_size || !c.max_seq || !c.max_batch)
        return fail(ctx, PRISM_E_ARG, "model config has a zero dimension");
    if (c.num_heads % c.num_kv_heads) return fail(ctx, PRISM_E_ARG, "num_heads must be a multiple of num_kv_heads");
    if (c.bits != 2 && c.bits != 4) return fail(ctx, PRISM_E_ARG, "bits must be 2 or 4");
    if (c.head_dim & 1) return fail(ctx, PRISM_E_ARG, "head_dim must be even");
    if (c.kv_page_size) {
        if (c.kv_page_size < 16 || (c.kv_page_size & (c.kv_page_size - 1))) return fail(ctx, PRISM_E_ARG, "kv_page_size must be a power of two >= 16");
        if (c.kv_int8 || (c.down_guard && c.intermediate_size != c.hidden_size) ||
            !(c.head_dim == 32 || c.head_dim == 64 || c.head_dim == 128 || c.head_dim == 256))
            return fail(ctx, PRISM_E_ARG, "the paged KV cache is fp16 only, head_dim 32/64/128/256, without the reference's DownProj guard");
    }
    const int T = ctx->tp_world, r = ctx->tp_rank;
    if (ctx->tp_loopback) return fail(ctx, PRISM_E_STATE, "a loopback tensor-parallel context has no peers: it cannot run a model");
    if (T > 1) {
        if (c.num_kv_heads % T || c.num_heads % T)
            return fail(ctx, PRISM_E_ARG, "tensor parallel degree must divide the head counts");
        if (c.down_guard && c.intermediate_size != c.hidden_size)
            return fail(ctx, PRISM_E_ARG, "down_guard is a single-GPU reference-compatibility switch");
        if (c.bits != 4) return fail(ctx, PRISM_E_ARG, "tensor parallel decode needs 4-bit palettes");
        if ((c.num_heads / T * c.head_dim) % 32 || c.intermediate_size % 32 || c.hidden_size % 32)
            return fail(ctx, PRISM_E_ARG, "sharded K ranges must be multiples of 32");
    }
    PRISM_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    prism_cuda_engine *e = new prism_cuda_engine();
    e->ctx = ctx; e->cfg = c; e->T = T; e->rank = r;
    e->H = c.hidden_size; e->hd = c.head_dim;
    e->nh_l = c.num_heads / T; e->nkv_l = c.num_kv_heads / T;
    e->head0 = e->nh_l * r; e->kvhead0 = e->nkv_l * r;
    e->qd_l = e->nh_l * e->hd; e->kvd_l = e->nkv_l * e->hd;
    uint32_t u0, u1;
    if (T > 1) {
        split_units(c.intermediate_size / 32, T, r, &u0, &u1);
        e->i0 = u0 * 32; e->I_l = (u1 - u0) * 32;
        split_units((c.vocab_size + 31) / 32, T, r, &u0, &u1);
        e->v0 = u0 * 32; e->V_l = std::min(c.vocab_size, u1 * 32) - e->v0;
    } else {
        e->i0 = 0; e->I_l = c.intermediate_size; e->v0 = 0; e->V_l = c.vocab_size;
    }
    e->guard_skip = c.down_guard && c.intermediate_size != c.hidden_size;
    e->kv_slots = e->guard_skip ? c.max_seq * c.num_layers : c.max_seq;
    if ((size_t)e->kv_slots * 4 > 160 * 1024) {
        delete e;
        return fail(ctx, PRISM_E_ARG, "max_seq too large for the attention score buffer (<= 40960 cached positions per layer slot)");
    }
    const uint32_t L = c.num_layers, B = c.max_batch;
    e->wq.assign(L, -1); e->wk.assign(L, -1); e->wv.assign(L, -1); e->wo.assign(L, -1);
    e->wg.assign(L, -1); e->wu.assign(L, -1); e->wd.assign(L, -1); e->wqkv.assign(L, -1);
    e->qkv_stride = round_up_u32(e->qd_l + 2 * e->kvd_l, 8);
    e->act_stride = round_up_u32(round_up_u32(e->I_l, 64), 8);
    e->out_cap = c.max_seq;
    const uint32_t kv_layers = e->guard_skip ? 1 : L;
    if (c.kv_page_size) {
        e->page_shift = 0;
        while ((1u << e->page_shift) < c.kv_page_size) e->page_shift++;
        e->pages_per_seq = (c.max_seq + c.kv_page_size - 1) / c.kv_page_size;
        e->pool_pages = c.kv_pool_pages ? c.kv_pool_pages : B * e->pages_per_seq;
        e->kv_seq_stride = (uint64_t)e->kv_slots * e->kvd_l;   // not used for addressing: rows come from the page table
        e->kv_layer_bytes = (size_t)e->pool_pages * c.kv_page_size * e->kvd_l * 2;
        e->page_tbl_host.assign((size_t)B * e->pages_per_seq, 0);
        e->seq_pages.assign(B, 0);
    } else if (c.kv_int8) {
        e->kv_seq_stride = (uint64_t)e->kv_slots * (e->kvd_l + 4);
        e->kv_layer_bytes = (size_t)B * e->kv_seq_stride;
    } else {
        e->kv_seq_stride = (uint64_t)e->kv_slots * e->kvd_l;
        e->kv_layer_bytes = (size_t)B * e->kv_seq_stride * 2;
    }
    auto A = [&](void **p, size_t bytes) { return cudaMalloc(p, (bytes + 255) / 256 * 256); };
    cudaError_t ce = cudaSuccess;
#define ALLOC(ptr, bytes) if (ce == cudaSuccess) ce = A((void **)&(ptr), (bytes))
    ALLOC(e->h, (size_t)B * e->H * 2);
    ALLOC(e->xn, (size_t)B * e->H * 2);
    ALLOC(e->qkv, (size_t)B * e->qkv_stride * 2);
    if (B >= 8) ALLOC(e->gu, 2 * (size_t)B * std::max(e->act_stride, e->H) * 2);
    ALLOC(e->att, (size_t)B * e->qd_l * 2);
    ALLOC(e->act, (size_t)B * e->act_stride * 2);
    ALLOC(e->logits, (size_t)B * round_up_u32(e->V_l, 8) * 2);
    ALLOC(e->part, (size_t)B * e->H * 4);
    ALLOC(e->tok, (size_t)B * 4);
    ALLOC(e->next, (size_t)B * 4);
    ALLOC(e->out_tokens, (size_t)B * e->out_cap * 4);
    ALLOC(e->pairs_send, (size_t)B * 8);
    ALLOC(e->pairs_recv, (size_t)B * 8 * T);
    ALLOC(e->scalars, 64);
    if (c.kv_page_size) ALLOC(e->page_tbl, (size_t)B * e->pages_per_seq * sizeof(int32_t));
    ALLOC(e->kc, e->kv_layer_bytes * kv_layers);
    ALLOC(e->vc, e->kv_layer_bytes * kv_layers);
#undef ALLOC
    e->q = e->qkv;
    e->k = e->qkv ? e->qkv + e->qd_l : nullptr;
    e->v = e->qkv ? e->qkv + e->qd_l + e->kvd_l : nullptr;
    if (ce == cudaSuccess) ce = cudaEventCreate(&e->ev0);
    if (ce == cudaSuccess) ce = cudaEventCreate(&e->ev1);
    if (ce == cudaSuccess) ce = cudaEventCreate(&e->ev2);
    if (ce == cudaSuccess) ce = cudaEventCreate(&e->ev3);
    if (ce == cudaSuccess) ce = cudaMemsetAsync(e->act, 0, (size_t)B * e->act_stride * 2, ctx->stream);
    if (ce == cudaSuccess) ce = cudaMemsetAsync(e->scalars, 0, 64, ctx->stream);
    if (ce != cudaSuccess) {
        prism_cuda_engine_destroy(e);
        return cuda_fail(ctx, ce, "engine allocation");
    }
    e->batch = 1;
    if (e->page_tbl) {
        cudaMemsetAsync(e->page_tbl, 0, (size_t)B * e->pages_per_seq * sizeof(int32_t), ctx->stream);
        release_pages(e);
    }
    *out = e;
    return PRISM_OK;
}

void prism_cuda_engine_destroy(prism_cuda_engine *e) {
    if (!e) return;
    cudaSetDevice(e->ctx->device);
    cudaStreamSynchronize(e->ctx->stream);
    if (e->graph) cudaGraphExecDestroy(e->graph);
    for (int32_t h : e->wqkv)
        if (h >= 0) prism_cuda_free_tensor(e->ctx, h);
    void *ptrs[] = {e->page_tbl, e->pf_x, e->pf_xn, e->pf_qkv, e->pf_att, e->pf_g, e->pf_u, e->pf_act, e->pf_tok, e->gu, e->h, e->xn, e->qkv, e->att, e->act, e->logits, e->part, e->tok, e->next,
                    e->out_tokens, e->prompts, e->pairs_send, e->pairs_recv, e->scalars, e->kc, e->vc};
    for (void *p : ptrs) cudaFree(p);
    if (e->ev0) cudaEventDestroy(e->ev0);
    if (e->ev1) cudaEventDestroy(e->ev1);
    if (e->ev2) cudaEventDestroy(e->ev2);
    if (e->ev3) cudaEventDestroy(e->ev3);
    delete e;
}

int prism_cuda_engine_bind(prism_cuda_engine *e, uint32_t role, uint32_t layer, int32_t handle) {
    if (!e) return PRISM_E_NULL;
    prism_cuda_ctx *ctx = e->ctx;
    LutTensor *t = get_tensor(ctx, handle);
    if (!t) return PRISM_E_NOTFOUND;
    const prism_model_config &c = e->cfg;
    if (role <= PRISM_ROLE_DOWN && layer >= c.num_layers) return fail(ctx, PRISM_E_ARG, "layer out of range");
    uint32_t want_m = 0, want_k = 0;
    std::vector<int32_t> *slot = nullptr;
    switch (role) {
    case PRISM_ROLE_Q: want_m = e->qd_l; want_k = e->H; slot = &e->wq; break;
    case PRISM_ROLE_K: want_m = e->kvd_l; want_k = e->H; slot = &e->wk; break;
    case PRISM_ROLE_V: want_m = e->kvd_l; want_k = e->H; slot = &e->wv; break;
    case PRISM_ROLE_O: want_m = e->H; want_k = e->qd_l; slot = &e->wo; break;
    case PRISM_ROLE_GATE: want_m = e->I_l; want_k = e->H; slot = &e->wg; break;
    case PRISM_ROLE_UP: want_m = e->I_l; want_k = e->H; slot = &e->wu; break;
    case PRISM_ROLE_DOWN: want_m = e->H; want_k = e->I_l; slot = &e->wd; break;
    case PRISM_ROLE_EMBED: want_m = c.vocab_size; want_k = e->H; break;
    case PRISM_ROLE_LM_HEAD: want_m = e->V_l; want_k = e->H; break;
    default: return fail(ctx, PRISM_E_ARG, "unknown role");
    }
    if (t->m != want_m || t->k != want_k || t->bits != c.bits)
        return fail(ctx, PRISM_E_ARG, "tensor " + t->name + " is " + std::to_string(t->m) + "x" + std::to_string(t->k) +
                                          ", role needs " + std::to_string(want_m) + "x" + std::to_string(want_k));
    if (slot) {
        (*slot)[layer] = handle;
        if (role <= PRISM_ROLE_V && e->wqkv[layer] >= 0) {  // rebinding q/k/v: the stacked copy is stale
            prism_cuda_free_tensor(ctx, e->wqkv[layer]);
            e->wqkv[layer] = -1;
        }
        if (role <= PRISM_ROLE_V) e->fused_ready = false;
    }
    else if (role == PRISM_ROLE_EMBED) e->embed = handle;
    else e->lm_head = handle;
    if (e->graph) {  // pointers baked into the graph are stale
        cudaGraphExecDestroy(e->graph);
        e->graph = nullptr;
        e->graph_batch = 0;
    }
    return PRISM_OK;
}

int prism_cuda_engine_bind_by_keys(prism_cuda_engine *e, const char *key_prefix) {
    if (!e) return PRISM_E_NULL;
    prism_cuda_ctx *ctx = e->ctx;
    if (e->T > 1) return fail(ctx, PRISM_E_STATE, "bind_by_keys binds whole tensors; shard and bind explicitly under tensor parallelism");
    const std::string p = key_prefix && *key_prefix ? key_prefix : "model";
    struct { const char *suffix; uint32_t role; } names[] = {
        {"self_attn.q_proj.weight", PRISM_ROLE_Q}, {"self_attn.k_proj.weight", PRISM_ROLE_K},
        {"self_attn.v_proj.weight", PRISM_ROLE_V}, {"self_attn.o_proj.weight", PRISM_ROLE_O},
        {"mlp.gate_proj.weight", PRISM_ROLE_GATE}, {"mlp.up_proj.weight", PRISM_ROLE_UP},
        {"mlp.down_proj.weight", PRISM_ROLE_DOWN}};
    int32_t h;
    for (uint32_t l = 0; l < e->cfg.num_layers; l++) {
        for (auto &n : names) {
            const std::string key = p + ".layers." + std::to_string(l) + "." + n.suffix;
            PRISM_TRY(prism_cuda_find_tensor(ctx, key.c_str(), &h));
            PRISM_TRY(prism_cuda_engine_bind(e, n.role, l, h));
        }
    }
    PRISM_TRY(prism_cuda_find_tensor(ctx, (p + ".embed_tokens.weight").c_str(), &h));
    PRISM_TRY(prism_cuda_engine_bind(e, PRISM_ROLE_EMBED, 0, h));
    if (!e->cfg.tie_word_embeddings) {
        // graph.rs:516-524 keys the head "{p}.lm_head.weight"
        PRISM_TRY(prism_cuda_find_tensor(ctx, (p + ".lm_head.weight").c_str(), &h));
        PRISM_TRY(prism_cuda_engine_bind(e, PRISM_ROLE_LM_HEAD, 0, h));
    }
    return PRISM_OK;
}

int prism_cuda_engine_synth_weights(prism_cuda_engine *e, uint64_t seed, float sigma) {
    if (!e) return PRISM_E_NULL;
    prism_cuda_ctx *ctx = e->ctx;
    const prism_model_config &c = e->cfg;
    const uint32_t H = e->H, bits = c.bits;
    int32_t h;
    auto S = [&](const std::string &name, uint64_t id, uint32_t rows, uint32_t cols, uint32_t row0, uint32_t col0,
                 uint32_t role, uint32_t layer) -> int {
        PRISM_TRY(synth_shard(ctx, name.c_str(), rows, cols, bits, seed * 1000003ull + id, sigma, row0, col0, &h));
        return prism_cuda_engine_bind(e, role, layer, h);
    };
    for (uint32_t l = 0; l < c.num_layers; l++) {
        const std::string p = "model.layers." + std::to_string(l) + ".";
        const uint64_t id = (uint64_t)l * 16;
        PRISM_TRY(S(p + "self_attn.q_proj.weight", id + 0, e->qd_l, H, e->head0 * e->hd, 0, PRISM_ROLE_Q, l));
        PRISM_TRY(S(p + "self_attn.k_proj.weight", id + 1, e->kvd_l, H, e->kvhead0 * e->hd, 0, PRISM_ROLE_K, l));
        PRISM_TRY(S(p + "self_attn.v_proj.weight", id + 2, e->kvd_l, H, e->kvhead0 * e->hd, 0, PRISM_ROLE_V, l));
        PRISM_TRY(S(p + "self_attn.o_proj.weight", id + 3, H, e->qd_l, 0, e->head0 * e->hd, PRISM_ROLE_O, l));
        PRISM_TRY(S(p + "mlp.gate_proj.weight", id + 4, e->I_l, H, e->i0, 0, PRISM_ROLE_GATE, l));
        PRISM_TRY(S(p + "mlp.up_proj.weight", id + 5, e->I_l, H, e->i0, 0, PRISM_ROLE_UP, l));
        PRISM_TRY(S(p + "mlp.down_proj.weight", id + 6, H, e->I_l, 0, e->i0, PRISM_ROLE_DOWN, l));
    }
    PRISM_TRY(S("model.embed_tokens.weight", 1ull << 40, c.vocab_size, H, 0, 0, PRISM_ROLE_EMBED, 0));
    if (!c.tie_word_embeddings)
        PRISM_TRY(S("model.lm_head.weight", (1ull << 40) + 1, e->V_l, H, e->v0, 0, PRISM_ROLE_LM_HEAD, 0));
    else if (e->T > 1)  // tied head under TP: this rank's vocabulary rows of the same table
        PRISM_TRY(S("model.embed_tokens.weight#shard", 1ull << 40, e->V_l, H, e->v0, 0, PRISM_ROLE_LM_HEAD, 0));
    return PRISM_OK;
}

int prism_cuda_engine_reset(prism_cuda_engine *e, uint32_t batch) {
    if (!e) return PRISM_E_NULL;
    if (batch == 0 || batch > e->cfg.max_batch) return fail(e->ctx, PRISM_E_ARG, "batch outside [1, max_batch]");
    PRISM_CUDA_TRY(e->ctx, cudaSetDevice(e->ctx->device));
    e->batch = batch;
    e->pos = 0;
    release_pages(e);  // a reset returns every page to the pool
    return set_scalars(e, 0, 0, 0);
}

int prism_cuda_engine_step(prism_cuda_engine *e, const uint32_t *tokens, uint32_t *next_tokens, uint16_t *logits) {
    if (!e || !tokens) return fail(e ? e->ctx : nullptr, PRISM_E_NULL, "null argument");
    prism_cuda_ctx *ctx = e->ctx;
    PRISM_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    PRISM_TRY(check_bound(e));
    PRISM_TRY(capacity_ok(e, 1));
    PRISM_TRY(set_scalars(e, (int32_t)e->pos, 0, 0));
    PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(e->tok, tokens, (size_t)e->batch * 4, cudaMemcpyHostToDevice, ctx->stream));
    PRISM_TRY(run_step(e));
    e->pos += 1;
    if (next_tokens)
        PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(next_tokens, e->next, (size_t)e->batch * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (logits) {
        if (e->T > 1) return fail(ctx, PRISM_E_STATE, "logits are sharded under tensor parallelism");
        const uint32_t ls = round_up_u32(e->V_l, 8);
        PRISM_CUDA_TRY(ctx, cudaMemcpy2DAsync(logits, (size_t)e->V_l * 2, e->logits, (size_t)ls * 2, (size_t)e->V_l * 2,
                                              e->batch, cudaMemcpyDeviceToHost, ctx->stream));
    }
    unsigned int errw = 0;
    PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(&errw, ctx->dev_err, 4, cudaMemcpyDeviceToHost, ctx->stream));
    PRISM_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return device_error_result(ctx, errw);
}

int prism_cuda_engine_decode(prism_cuda_engine *e, const uint32_t *tokens_in, uint32_t n_steps, uint32_t *out_tokens) {
    if (!e || !tokens_in || !out_tokens) return fail(e ? e->ctx : nullptr, PRISM_E_NULL, "null argument");
    prism_cuda_ctx *ctx = e->ctx;
    PRISM_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    PRISM_TRY(check_bound(e));
    if (n_steps == 0) return PRISM_OK;
    if (n_steps > e->out_cap) return fail(ctx, PRISM_E_ARG, "n_steps exceeds max_seq");
    PRISM_TRY(capacity_ok(e, n_steps));
    PRISM_TRY(set_scalars(e, (int32_t)e->pos, 0, 1));
    PRISM_CUDA_TRY(ctx, cudaEventRecord(e->ev0, ctx->stream));
    PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(e->tok, tokens_in, (size_t)e->batch * 4, cudaMemcpyHostToDevice, ctx->stream));
    PRISM_CUDA_TRY(ctx, cudaEventRecord(e->ev2, ctx->stream));
    for (uint32_t i = 0; i < n_steps; i++) PRISM_TRY(run_step(e));
    PRISM_CUDA_TRY(ctx, cudaEventRecord(e->ev3, ctx->stream));
    e->pos += n_steps;
    PRISM_CUDA_TRY(ctx, cudaMemcpy2DAsync(out_tokens, (size_t)n_steps * 4, e->out_tokens, (size_t)e->out_cap * 4,
                                          (size_t)n_steps * 4, e->batch, cudaMemcpyDeviceToHost, ctx->stream));
    PRISM_CUDA_TRY(ctx, cudaEventRecord(e->ev1, ctx->stream));
    unsigned int errw = 0;
    PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(&errw, ctx->dev_err, 4, cudaMemcpyDeviceToHost, ctx->stream));
    PRISM_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e->ev0, e->ev1);
    e->last_ms = ms;
    cudaEventElapsedTime(&ms, e->ev2, e->ev3);
    e->last_device_ms = ms;
    return device_error_result(ctx, errw);
}

int prism_cuda_engine_generate(prism_cuda_engine *e, const uint32_t *prompts, uint32_t batch, uint32_t n_prompt,
                               uint32_t max_new, uint32_t *out_tokens, uint16_t *last_logits) {
    if (!e || (!prompts && n_prompt) || (!out_tokens && max_new))
        return fail(e ? e->ctx : nullptr, PRISM_E_NULL, "null argument");
    prism_cuda_ctx *ctx = e->ctx;
    PRISM_TRY(check_bound(e));
    PRISM_TRY(prism_cuda_engine_reset(e, batch));
    if (max_new > e->out_cap) return fail(ctx, PRISM_E_ARG, "max_new exceeds max_seq");
    PRISM_TRY(capacity_ok(e, n_prompt + max_new));
    // prompts -> device, position-major so a step's tokens are contiguous
    const size_t need = (size_t)std::max<uint32_t>(n_prompt, 1) * batch;
    if (need > e->prompts_cap) {
        PRISM_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
        cudaFree(e->prompts);
        e->prompts = nullptr;
        e->prompts_cap = 0;
        PRISM_CUDA_TRY(ctx, cudaMalloc((void **)&e->prompts, need * 4));
        e->prompts_cap = need;
    }
    std::vector<uint32_t> tr(need, 0);
    for (uint32_t b = 0; b < batch; b++)
        for (uint32_t i = 0; i < n_prompt; i++) tr[(size_t)i * batch + b] = prompts[(size_t)b * n_prompt + i];
    PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(e->prompts, tr.data(), need * 4, cudaMemcpyHostToDevice, ctx->stream));
    PRISM_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    PRISM_CUDA_TRY(ctx, cudaEventRecord(e->ev0, ctx->stream));
    if (n_prompt >= 2 && prefill_batched_ok(e)) {
        PRISM_TRY(prefill_batched(e, batch, n_prompt));
    } else {
        // prefill_cpu (engine_impl.rs:1046-1053): one step per prompt token
        for (uint32_t i = 0; i < n_prompt; i++) {
            PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(e->tok, e->prompts + (size_t)i * batch, (size_t)batch * 4,
                                                cudaMemcpyDeviceToDevice, ctx->stream));
            PRISM_TRY(run_step(e));
        }
    }
    e->pos = n_prompt;
    // decode: `nt = *prompt.last().unwrap_or(&0)` (engine_impl.rs:1015) is fed first
    if (n_prompt == 0) PRISM_CUDA_TRY(ctx, cudaMemsetAsync(e->tok, 0, (size_t)batch * 4, ctx->stream));
    {
        int32_t one = 1;  // record = 1; pos and step are already right (step stayed 0 while not recording)
        PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(e->scalars + 2, &one, 4, cudaMemcpyHostToDevice, ctx->stream));
    }
    PRISM_CUDA_TRY(ctx, cudaEventRecord(e->ev2, ctx->stream));
    for (uint32_t i = 0; i < max_new; i++) PRISM_TRY(run_step(e));
    PRISM_CUDA_TRY(ctx, cudaEventRecord(e->ev3, ctx->stream));
    e->pos += max_new;
    PRISM_CUDA_TRY(ctx, cudaEventRecord(e->ev1, ctx->stream));
    if (max_new)
        PRISM_CUDA_TRY(ctx, cudaMemcpy2DAsync(out_tokens, (size_t)max_new * 4, e->out_tokens, (size_t)e->out_cap * 4,
                                              (size_t)max_new * 4, batch, cudaMemcpyDeviceToHost, ctx->stream));
    if (last_logits) {
        if (e->T > 1) return fail(ctx, PRISM_E_STATE, "logits are sharded under tensor parallelism");
        const uint32_t ls = round_up_u32(e->V_l, 8);
        PRISM_CUDA_TRY(ctx, cudaMemcpy2DAsync(last_logits, (size_t)e->V_l * 2, e->logits, (size_t)ls * 2,
                                              (size_t)e->V_l * 2, batch, cudaMemcpyDeviceToHost, ctx->stream));
    }
    unsigned int errw = 0;
    PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(&errw, ctx->dev_err, 4, cudaMemcpyDeviceToHost, ctx->stream));
    PRISM_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e->ev0, e->ev1);
    e->last_ms = ms;
    cudaEventElapsedTime(&ms, e->ev2, e->ev3);
    e->last_device_ms = ms;  // the decode steps alone (prefill excluded)
    return device_error_result(ctx, errw);
}

uint64_t prism_cuda_engine_step_bytes(prism_cuda_engine *e) {
    if (!e) return 0;
    prism_cuda_ctx *ctx = e->ctx;
    uint64_t bytes = 0;
    auto add = [&](int32_t h) {
        if (h >= 0 && ctx->tensors[h].live) bytes += ctx->tensors[h].algorithmic_bytes();
    };
    for (uint32_t l = 0; l < e->cfg.num_layers; l++) {
        add(e->wq[l]); add(e->wk[l]); add(e->wv[l]); add(e->wo[l]); add(e->wg[l]); add(e->wu[l]);
        if (!e->guard_skip) add(e->wd[l]);
    }
    add((e->cfg.tie_word_embeddings || e->lm_head < 0) ? e->embed : e->lm_head);
    // KV read: K and V of every cached position, every layer
    const uint64_t per_pos = e->cfg.kv_int8 ? 2ull * (e->kvd_l + 4) : 4ull * e->kvd_l;
    bytes += per_pos * (uint64_t)(e->pos + 1) * e->cfg.num_layers;
    return bytes;
}

double prism_cuda_engine_last_ms(prism_cuda_engine *e) { return e ? e->last_ms : 0.0; }
double prism_cuda_engine_last_device_ms(prism_cuda_engine *e) { return e ? e->last_device_ms : 0.0; }
uint32_t prism_cuda_engine_kernels_per_step(prism_cuda_engine *e) { return e ? e->kernels_per_step : 0; }

// Times only the palettized GEMV launches of one decode step (every layer's q, k, v, o,
// fused gate/up, down, and the head), back to back on the context stream between two
// events, `reps` times.  The weights of a whole model exceed L2, so every launch streams
// from HBM.  Outputs: elapsed ms, algorithmic bytes and launches over all reps.
extern "C" int prism_cuda_engine_profile_gemv(prism_cuda_engine *e, uint32_t reps, double *ms_out, uint64_t *bytes_out,
                                   uint32_t *launches_out) {
    if (!e || !ms_out) return fail(e ? e->ctx : nullptr, PRISM_E_NULL, "null argument");
    prism_cuda_ctx *ctx = e->ctx;
    PRISM_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    PRISM_TRY(check_bound(e));
    const uint32_t B = e->batch ? e->batch : 1, H = e->H;
    uint64_t bytes = 0;
    uint32_t launches = 0;
    auto one_pass = [&](bool count) -> int {
        for (uint32_t l = 0; l < e->cfg.num_layers; l++) {
            const LutTensor &tq = ctx->tensors[e->wq[l]], &tk = ctx->tensors[e->wk[l]], &tv = ctx->tensors[e->wv[l]],
                            &to = ctx->tensors[e->wo[l]], &tg = ctx->tensors[e->wg[l]], &tu = ctx->tensors[e->wu[l]];
            if (e->wqkv[l] >= 0) {
                PRISM_TRY(launch_gemv(ctx, GEMV_PLAIN, ctx->tensors[e->wqkv[l]], nullptr, e->xn, H, e->qkv, e->qkv_stride, nullptr, B));
                if (count) launches -= 2;
            } else {
                PRISM_TRY(launch_gemv(ctx, GEMV_PLAIN, tq, nullptr, e->xn, H, e->q, e->qkv_stride, nullptr, B));
                PRISM_TRY(launch_gemv(ctx, GEMV_PLAIN, tk, nullptr, e->xn, H, e->k, e->qkv_stride, nullptr, B));
                PRISM_TRY(launch_gemv(ctx, GEMV_PLAIN, tv, nullptr, e->xn, H, e->v, e->qkv_stride, nullptr, B));
            }
            PRISM_TRY(launch_gemv(ctx, GEMV_PLAIN, to, nullptr, e->att, e->qd_l, e->xn, H, nullptr, B));
            PRISM_TRY(launch_gemv(ctx, GEMV_SWIGLU, tg, &tu, e->xn, H, e->act, e->act_stride, nullptr, B));
            if (count) {
                bytes += tq.algorithmic_bytes() + tk.algorithmic_bytes() + tv.algorithmic_bytes() +
                         to.algorithmic_bytes() + tg.algorithmic_bytes() + tu.algorithmic_bytes() - 2ull * tg.k;
                launches += 5;
            }
            if (!e->guard_skip) {
                const LutTensor &td = ctx->tensors[e->wd[l]];
                PRISM_TRY(launch_gemv(ctx, GEMV_PLAIN, td, nullptr, e->act, e->act_stride, e->xn, H, nullptr, B));
                if (count) { bytes += td.algorithmic_bytes(); launches += 1; }
            }
        }
        const LutTensor &head = ctx->tensors[(e->cfg.tie_word_embeddings || e->lm_head < 0) ? e->embed : e->lm_head];
        PRISM_TRY(launch_gemv(ctx, GEMV_PLAIN, head, nullptr, e->xn, H, e->logits, round_up_u32(e->V_l, 8), nullptr, B));
        if (count) { bytes += head.algorithmic_bytes(); launches += 1; }
        return PRISM_OK;
    };
    PRISM_TRY(one_pass(false));  // warm-up: sizes scratch, sets attributes
    PRISM_CUDA_TRY(ctx, cudaEventRecord(e->ev2, ctx->stream));
    for (uint32_t r = 0; r < reps; r++) PRISM_TRY(one_pass(true));
    PRISM_CUDA_TRY(ctx, cudaEventRecord(e->ev3, ctx->stream));
    PRISM_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e->ev2, e->ev3);
    *ms_out = ms;
    if (bytes_out) *bytes_out = bytes;
    if (launches_out) *launches_out = launches;
    return PRISM_OK;
}
extern "C" int prism_cuda_engine_profile_part(prism_cuda_engine *e, uint32_t part, uint32_t reps, double *ms_out,
                                              uint32_t *launches_out) {
    if (!e || !ms_out) return fail(e ? e->ctx : nullptr, PRISM_E_NULL, "null argument");
    prism_cuda_ctx *ctx = e->ctx;
    if (part != 1 && part != 2) return fail(ctx, PRISM_E_ARG, "profile_part: 1 = attention, 2 = tensor-parallel reductions");
    PRISM_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    PRISM_TRY(check_bound(e));
    const uint32_t L = e->cfg.num_layers, B = e->batch ? e->batch : 1;
    // the attention kernel appends at the current position: keep that inside the cache
    PRISM_TRY(capacity_ok(e, 1));
    PRISM_TRY(set_scalars(e, (int32_t)e->pos, 0, 0));
    const uint64_t l0 = ctx->launches;
    auto one_pass = [&]() -> int {
        for (uint32_t l = 0; l < L; l++) {
            if (part == 1) {
                PRISM_TRY(enqueue_attention(e, l, e->guard_skip ? 0 : l));
            } else if (e->T > 1) {
                PRISM_TRY(tp_reduce_add_resid(e, B * e->H));
                PRISM_TRY(tp_reduce_add_resid(e, B * e->H));
            }
        }
        return PRISM_OK;
    };
    PRISM_TRY(one_pass());
    const uint64_t per_pass = ctx->launches - l0;
    PRISM_CUDA_TRY(ctx, cudaEventRecord(e->ev2, ctx->stream));
    for (uint32_t r = 0; r < reps; r++) PRISM_TRY(one_pass());
    PRISM_CUDA_TRY(ctx, cudaEventRecord(e->ev3, ctx->stream));
    PRISM_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e->ev2, e->ev3);
    *ms_out = ms;
    if (launches_out) *launches_out = (uint32_t)(per_pass * reps);
    return check_device_error(ctx);
}
prism_cuda_ctx *prism_cuda_engine_ctx(prism_cuda_engine *e) { return e ? e->ctx : nullptr; }
uint32_t prism_cuda_engine_position(prism_cuda_engine *e) { return e ? e->pos : 0; }

}  // extern "C"
