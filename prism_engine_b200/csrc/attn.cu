// Fused attention of one decode step: RoPE of q (and of k where the profile asks for it), append
// of the new token's k/v to the fp16 cache, and attention over the cached positions, in ONE
// kernel.  It stands for four nodes of step() (src/lut/engine_impl.rs:1076-1459): Rope(q),
// Rope(k), KVCache::append and Attention (attention_cpu, src/lut/cpu_fallback.rs:84-127;
// rope_inplace, cpu_fallback.rs:131-143), with the same fp16 rounding points: q and k are rounded
// to fp16 after the rotation, the output after the weighted sum.
//
// A thread-block cluster of S CTAs serves one (query head, sequence): CTA r scores and weighs the
// positions [r*chunk, (r+1)*chunk) of the cache.  The softmax is the reference's two-pass form
// (global maximum, exp, global sum, `* inv` inside the weighted sum); the S CTAs exchange their
// maxima, sums and partial outputs through distributed shared memory, so nothing goes through
// global scratch and the result does not depend on scheduling.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace prism {

constexpr int FA_THREADS = 256;
constexpr int FA_WARPS = FA_THREADS / 32;
constexpr int FA_INFLIGHT = 8;  // cached rows a warp has in flight

__device__ __forceinline__ float fa_h2f(uint16_t v) { return __half2float(__ushort_as_half(v)); }
__device__ __forceinline__ uint16_t fa_f2h(float v) { return __half_as_ushort(__float2half_rn(v)); }
__device__ __forceinline__ float fa_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

struct FusedAttnArgs {
    const uint16_t *q, *k, *v;  // this step's projections: rows of nh*hd / nkv*hd halfs, src_stride apart
    uint32_t src_stride;
    uint16_t *kc, *vc;          // fp16 cache of this layer slot: [seq][slot][nkv*hd]
    uint16_t *out;              // [batch][nh*hd]
    const int32_t *pos_dev;     // token position (device scalar, so a captured graph can be replayed)
    uint32_t slot_mul, slot_add;  // cache slot of the new token = pos*slot_mul + slot_add
    uint32_t nh, nkv, batch;
    uint64_t seq_stride;        // halfs between sequences in the cache
    uint32_t max_seq;           // slots per sequence
    uint32_t chunk_cap;         // floats of score buffer per CTA
    uint32_t rope_k;
    float rope_base;
};

// Rotates the VEC elements a lane owns (elements lane*VEC .. +VEC-1 of a head of 32*VEC): the
// partner element j +- hd/2 lives in lane ^ 16.
template <int VEC>
__device__ __forceinline__ void fa_rope(float (&x)[VEC], uint32_t lane, float pos, float base) {
    constexpr uint32_t hd = 32 * VEC, half = hd / 2;
#pragma unroll
    for (int i = 0; i < VEC; i++) {
        const float other = __shfl_xor_sync(0xFFFFFFFFu, x[i], 16);
        const uint32_t d = lane * VEC + i;
        const uint32_t j = d < half ? d : d - half;
        const float ang = pos * powf(base, -2.0f * (float)j / (float)hd);
        float sa, ca;
        sincosf(ang, &sa, &ca);
        // d < half: (a, b) = (mine, other) -> a*cos - b*sin;  else (a, b) = (other, mine) -> a*sin + b*cos
        const float r = d < half ? __fsub_rn(__fmul_rn(x[i], ca), __fmul_rn(other, sa))
                                 : __fadd_rn(__fmul_rn(other, sa), __fmul_rn(x[i], ca));
        x[i] = fa_h2f(fa_f2h(r));
    }
}

template <int VEC>
__global__ void __launch_bounds__(FA_THREADS) attn_fused_kernel(const FusedAttnArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t S = cluster.dim_blocks().x, rank = cluster.block_rank();
    extern __shared__ float sc[];                 // [chunk_cap] scores, then exp
    __shared__ float sh[32];
    __shared__ float xch[2];                      // this CTA's maximum and sum, read by its peers
    __shared__ float part[FA_WARPS * 32 * VEC];   // per-warp partial outputs; row 0 ends as the CTA's partial
    constexpr uint32_t hd = 32 * VEC;
    const uint32_t h = blockIdx.x / S, b = blockIdx.y;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t g = a.nh / a.nkv, kh = h / g, kvd = a.nkv * hd;

    const int32_t pos = *a.pos_dev;
    const int64_t slot64 = (int64_t)pos * a.slot_mul + a.slot_add;
    const bool have_new = slot64 >= 0 && slot64 < (int64_t)a.max_seq;  // a full cache takes no new row
    uint32_t sl = (uint32_t)(slot64 + 1);
    if (slot64 < 0) sl = 0;
    if (sl > a.max_seq) sl = a.max_seq;
    const uint32_t new_slot = have_new ? (uint32_t)slot64 : 0xFFFFFFFFu;
    uint32_t chunk = (sl + S - 1) / S;
    if (chunk > a.chunk_cap) chunk = a.chunk_cap;  // cannot happen with chunk_cap = ceil(max_seq / S)
    const uint32_t p_begin = min(sl, rank * chunk), p_end = min(sl, p_begin + chunk);

    // ---- q, and the new token's k and v, in registers (lane: elements lane*VEC..) ---------------
    float qf[VEC], kn[VEC], vn[VEC];
    {
        const uint16_t *q = a.q + (size_t)b * a.src_stride + (size_t)h * hd + lane * VEC;
        const uint16_t *k = a.k + (size_t)b * a.src_stride + (size_t)kh * hd + lane * VEC;
        const uint16_t *v = a.v + (size_t)b * a.src_stride + (size_t)kh * hd + lane * VEC;
#pragma unroll
        for (int i = 0; i < VEC; i++) {
            qf[i] = fa_h2f(q[i]);
            kn[i] = fa_h2f(k[i]);
            vn[i] = fa_h2f(v[i]);
        }
        fa_rope<VEC>(qf, lane, (float)pos, a.rope_base);
        if (a.rope_k) fa_rope<VEC>(kn, lane, (float)pos, a.rope_base);
    }
    uint16_t *kcb = a.kc + (size_t)b * a.seq_stride + (size_t)kh * hd + lane * VEC;
    uint16_t *vcb = a.vc + (size_t)b * a.seq_stride + (size_t)kh * hd + lane * VEC;
    const bool own_new = have_new && new_slot >= p_begin && new_slot < p_end;
    // KVCache::append: the first query head of a group stores the row for all later steps
    if (own_new && h % g == 0 && warp == 0) {
#pragma unroll
        for (int i = 0; i < VEC; i++) {
            kcb[(size_t)new_slot * kvd + i] = fa_f2h(kn[i]);
            vcb[(size_t)new_slot * kvd + i] = fa_f2h(vn[i]);
        }
    }

    // ---- scores of this CTA's positions: one warp per position, FA_INFLIGHT rows in flight -------
    const float div = sqrtf((float)hd);
    struct alignas(2 * VEC) Row { uint16_t e[VEC]; };
    for (uint32_t p0 = p_begin + warp; p0 < p_end; p0 += FA_INFLIGHT * FA_WARPS) {
        Row r[FA_INFLIGHT];
#pragma unroll
        for (int u = 0; u < FA_INFLIGHT; u++) {
            const uint32_t p = p0 + u * FA_WARPS;
            if (p < p_end && p != new_slot) r[u] = *reinterpret_cast<const Row *>(kcb + (size_t)p * kvd);
        }
#pragma unroll
        for (int u = 0; u < FA_INFLIGHT; u++) {
            const uint32_t p = p0 + u * FA_WARPS;
            if (p < p_end) {  // warp-uniform
                float s = 0.0f;
                if (p == new_slot) {
#pragma unroll
                    for (int i = 0; i < VEC; i++) s += qf[i] * kn[i];
                } else {
#pragma unroll
                    for (int i = 0; i < VEC; i++) s += qf[i] * fa_h2f(r[u].e[i]);
                }
                s = fa_warp_sum(s);
                if (lane == 0) sc[p - p_begin] = s / div;
            }
        }
    }
    __syncthreads();

    // ---- maximum over all positions: local, then across the cluster ------------------------------
    const uint32_t n_loc = p_end - p_begin;
    float mx = -INFINITY;
    for (uint32_t p = threadIdx.x; p < n_loc; p += FA_THREADS) mx = fmaxf(mx, sc[p]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    if (lane == 0) sh[warp] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
        float m = -INFINITY;
        for (int w = 0; w < FA_WARPS; w++) m = fmaxf(m, sh[w]);
        xch[0] = m;
    }
    cluster.sync();
    mx = -INFINITY;
    for (uint32_t r = 0; r < S; r++) mx = fmaxf(mx, *cluster.map_shared_rank(&xch[0], r));

    // ---- exp and its sum: local in warp order, then across the cluster in rank order -------------
    float es = 0.0f;
    for (uint32_t p = threadIdx.x; p < n_loc; p += FA_THREADS) {
        const float e = expf(sc[p] - mx);
        sc[p] = e;
        es += e;
    }
    es = fa_warp_sum(es);
    if (lane == 0) sh[warp] = es;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int w = 0; w < FA_WARPS; w++) t += sh[w];
        xch[1] = t;
    }
    cluster.sync();
    es = 0.0f;
    for (uint32_t r = 0; r < S; r++) es += *cluster.map_shared_rank(&xch[1], r);
    const float inv = 1.0f / (es + 1e-10f);

    // ---- weighted sum of the value rows -----------------------------------------------------------
    float ac[VEC];
#pragma unroll
    for (int i = 0; i < VEC; i++) ac[i] = 0.0f;
    for (uint32_t p0 = p_begin + warp; p0 < p_end; p0 += FA_INFLIGHT * FA_WARPS) {
        Row r[FA_INFLIGHT];
        float e[FA_INFLIGHT];
#pragma unroll
        for (int u = 0; u < FA_INFLIGHT; u++) {
            const uint32_t p = p0 + u * FA_WARPS;
            e[u] = 0.0f;
            if (p < p_end) {
                if (p != new_slot) r[u] = *reinterpret_cast<const Row *>(vcb + (size_t)p * kvd);
                e[u] = sc[p - p_begin];
            }
        }
#pragma unroll
        for (int u = 0; u < FA_INFLIGHT; u++) {
            const uint32_t p = p0 + u * FA_WARPS;
            if (p < p_end) {
#pragma unroll
                for (int i = 0; i < VEC; i++) {
                    const float vv = (p == new_slot) ? vn[i] : fa_h2f(r[u].e[i]);
                    ac[i] += __fmul_rn(__fmul_rn(e[u], vv), inv);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < VEC; i++) part[warp * hd + lane * VEC + i] = ac[i];
    __syncthreads();
    if (threadIdx.x < hd) {
        float t = 0.0f;
#pragma unroll
        for (uint32_t w = 0; w < (uint32_t)FA_WARPS; w++) t += part[w * hd + threadIdx.x];
        part[threadIdx.x] = t;  // row 0: only this thread reads and writes element threadIdx.x of it
    }
    cluster.sync();
    if (rank == 0 && threadIdx.x < hd) {
        float t = 0.0f;
        for (uint32_t r = 0; r < S; r++) t += *cluster.map_shared_rank(&part[threadIdx.x], r);
        a.out[(size_t)b * a.nh * hd + (size_t)h * hd + threadIdx.x] = fa_f2h(t);
    }
    cluster.sync();  // peers keep their shared memory alive until rank 0 has read it
}

bool attn_fused_eligible(const AttnArgs &a) {
    return !a.int8 && (a.hd == 32 || a.hd == 64 || a.hd == 128 || a.hd == 256) && a.pos_dev != nullptr &&
           a.nkv != 0 && a.nh % a.nkv == 0 && (a.seq_stride * 2) % 16 == 0 &&
           reinterpret_cast<uintptr_t>(a.k) % 16 == 0 && reinterpret_cast<uintptr_t>(a.v) % 16 == 0;
}

template <int VEC>
static int launch_attn_fused_v(prism_cuda_ctx *ctx, const FusedAttnArgs &fa, uint32_t S, size_t smem) {
    static bool configured[PRISM_MAX_DEVICES] = {false};
    if (smem > 32 * 1024 && !configured[ctx->device]) {
        PRISM_CUDA_TRY(ctx, cudaFuncSetAttribute(attn_fused_kernel<VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 160 * 1024));
        configured[ctx->device] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(fa.nh * S, fa.batch);
    cfg.blockDim = dim3(FA_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = S;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->pdl ? 2 : 1;
    (void)cudaLaunchKernelEx(&cfg, attn_fused_kernel<VEC>, fa);
    return after_launch(ctx, "attn_fused_kernel");
}

// q_src/k_src/v_src: this step's projection rows (src_stride halfs apart); a.k / a.v: the cache.
int launch_attn_fused(prism_cuda_ctx *ctx, const AttnArgs &a, const uint16_t *k_src, const uint16_t *v_src,
                      uint32_t rope_k, float rope_base) {
    if (!attn_fused_eligible(a)) return fail(ctx, PRISM_E_ARG, "fused attention: fp16 cache and head_dim 32/64/128/256 only");
    FusedAttnArgs fa{};
    fa.q = a.q; fa.k = k_src; fa.v = v_src; fa.src_stride = a.q_stride;
    fa.kc = static_cast<uint16_t *>(const_cast<void *>(a.k));
    fa.vc = static_cast<uint16_t *>(const_cast<void *>(a.v));
    fa.out = a.out;
    fa.pos_dev = a.pos_dev; fa.slot_mul = a.slot_mul; fa.slot_add = a.slot_add;
    fa.nh = a.nh; fa.nkv = a.nkv; fa.batch = a.batch;
    fa.seq_stride = a.seq_stride; fa.max_seq = a.max_seq;
    fa.rope_k = rope_k; fa.rope_base = rope_base;
    // cluster size: enough CTAs per head to keep every SM loading cache rows at long contexts
    uint32_t S = a.max_seq >= 512 ? 8 : a.max_seq >= 256 ? 4 : a.max_seq >= 128 ? 2 : 1;
    if (ctx->attn_cluster == 1 || ctx->attn_cluster == 2 || ctx->attn_cluster == 4 || ctx->attn_cluster == 8)
        S = (uint32_t)ctx->attn_cluster;
    fa.chunk_cap = (a.max_seq + S - 1) / S;
    const size_t smem = (size_t)fa.chunk_cap * sizeof(float);
    if (smem > 160 * 1024) return fail(ctx, PRISM_E_ARG, "fused attention: max_seq too large for the score buffer");
    switch (a.hd) {
    case 32: return launch_attn_fused_v<1>(ctx, fa, S, smem);
    case 64: return launch_attn_fused_v<2>(ctx, fa, S, smem);
    case 128: return launch_attn_fused_v<4>(ctx, fa, S, smem);
    default: return launch_attn_fused_v<8>(ctx, fa, S, smem);
    }
}

}  // namespace prism
