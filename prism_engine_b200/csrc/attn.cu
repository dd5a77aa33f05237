// Fused attention of one decode step: RoPE of q (and of k where the profile asks for it), append
// of the new token's k/v to the fp16 cache, and attention over the cached positions, in ONE
// kernel.  It stands for four nodes of step() (src/lut/engine_impl.rs:1076-1459): Rope(q),
// Rope(k), KVCache::append and Attention (attention_cpu, src/lut/cpu_fallback.rs:84-127;
// rope_inplace, cpu_fallback.rs:131-143), with the same fp16 rounding points: q and k are rounded
// to fp16 after the rotation, the output after the weighted sum.
//
// A thread-block cluster of S CTAs serves one (KV head, sequence) and ALL the query heads that
// share that KV head (grouped-query attention: up to GT = 8 heads per pass over the cache), so a
// cached row is read once per group instead of once per query head.  CTA r scores and weighs the
// positions [r*chunk, (r+1)*chunk): one warp per cached row, every row of a pass in flight at once,
// the value rows requested together with the key rows so that their latency hides behind the
// softmax.  The softmax is the reference's two-pass form (global maximum, exp, global sum, `* inv`
// inside the weighted sum); the S CTAs exchange their maxima, sums and partial outputs through
// distributed shared memory, so nothing goes through global scratch and the result does not
// depend on scheduling.
#include <cooperative_groups.h>

#include <cmath>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace prism {

constexpr int FA_THREADS = 256;
constexpr int FA_WARPS = FA_THREADS / 32;

__device__ __forceinline__ float fa_h2f(uint16_t v) { return __half2float(__ushort_as_half(v)); }
__device__ __forceinline__ uint16_t fa_f2h(float v) { return __half_as_ushort(__float2half_rn(v)); }

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
    uint32_t chunk_cap;         // positions of score buffer per CTA
    uint32_t rope_k;
    const float *inv_freq;      // [hd/2] rotation frequencies base^(-2j/hd), computed once on the host
    // Prefill: the `batch` rows are consecutive tokens of ONE sequence (cache sequence `seq`), row t at
    // position *pos_dev + t; their keys and values are already in the cache (prefill_kv_kernel), so
    // nothing is appended and row t attends to positions 0 .. *pos_dev + t.
    uint32_t prefill, seq;
    // Paged cache: position p of cache sequence c lives in row (page_tbl[c*tbl_stride + (p >> page_shift)]
    // << page_shift) + (p & (page - 1)) of the layer's page pool; nullptr: one contiguous slab per sequence.
    const int32_t *page_tbl;
    uint32_t page_shift, tbl_stride;
    uint32_t early_cache;       // 1: the kernel before this one in the stream does not write the cache (see the kernel)
};

// Row (in units of cached rows of the layer) of position p of cache sequence c.
__device__ __forceinline__ size_t fa_row(const int32_t *__restrict__ tbl, uint32_t shift, uint32_t tbl_stride, uint64_t seq_rows,
                                         uint32_t c, uint32_t p) {
    if (tbl == nullptr) return (size_t)c * seq_rows + p;
    const uint32_t page = (uint32_t)__ldg(tbl + (size_t)c * tbl_stride + (p >> shift));
    return ((size_t)page << shift) + (p & ((1u << shift) - 1u));
}

// cos / sin of the rotation of the VEC elements a lane owns (elements lane*VEC .. +VEC-1 of a head
// of 32*VEC): the angle depends on the position and the pair index only, so it is computed once
// and applied to every query head and to k.
template <int VEC>
__device__ __forceinline__ void fa_rope_angles(float (&ca)[VEC], float (&sa)[VEC], uint32_t lane, float pos,
                                               const float *__restrict__ inv_freq) {
    constexpr uint32_t half = 16 * VEC;
#pragma unroll
    for (int i = 0; i < VEC; i++) {
        const uint32_t d = lane * VEC + i;
        const uint32_t j = d < half ? d : d - half;
        const float ang = pos * __ldg(inv_freq + j);
        sincosf(ang, &sa[i], &ca[i]);
    }
}

// Stores a value into the same shared-memory word of every CTA of the cluster (at most 8), its own included.
template <typename G>
__device__ __forceinline__ void fa_scatter(G &cluster, float *word, uint32_t S, float value) {
#pragma unroll
    for (uint32_t r = 0; r < 8; r++)
        if (r < S) *cluster.map_shared_rank(word, r) = value;
}
// Rotates a lane's elements; the partner element j +- hd/2 lives in lane ^ 16.
template <int VEC>
__device__ __forceinline__ void fa_rope_apply(float (&x)[VEC], const float (&ca)[VEC], const float (&sa)[VEC], uint32_t lane) {
    constexpr uint32_t half = 16 * VEC;
#pragma unroll
    for (int i = 0; i < VEC; i++) {
        const float other = __shfl_xor_sync(0xFFFFFFFFu, x[i], 16);
        const uint32_t d = lane * VEC + i;
        // d < half: (a, b) = (mine, other) -> a*cos - b*sin;  else (a, b) = (other, mine) -> a*sin + b*cos
        const float r = d < half ? __fsub_rn(__fmul_rn(x[i], ca[i]), __fmul_rn(other, sa[i]))
                                 : __fadd_rn(__fmul_rn(other, sa[i]), __fmul_rn(x[i], ca[i]));
        x[i] = fa_h2f(fa_f2h(r));
    }
}

// Sums each of GT per-lane values over the 32 lanes of a warp.  log2(GT) exchange rounds halve the
// number of values a lane carries (offsets 16, 8, ...), the rest are plain butterfly adds: 9
// shuffles for GT = 8 instead of 40.  Returns the total of value number (lane >> (5 - log2 GT)).
template <int GT>
__device__ __forceinline__ float fa_reduce_heads(float (&s)[GT], uint32_t lane) {
    int off = 16;
#pragma unroll
    for (int n = GT; n > 1; n >>= 1, off >>= 1) {
        const bool up = (lane & off) != 0;
#pragma unroll
        for (int j = 0; j < n / 2; j++) {
            const float send = up ? s[j] : s[j + n / 2];
            const float keep = up ? s[j + n / 2] : s[j];
            s[j] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, off);
        }
    }
    float v = s[0];
#pragma unroll
    for (; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
    return v;
}

// 16-byte asynchronous copy global -> shared (the cached rows of a pass are all requested before any is used)
__device__ __forceinline__ void fa_cp16(void *dst_smem, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src)
                 : "memory");
}
__device__ __forceinline__ void fa_cp_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
}

// rows of a tile: K and V tiles together take 48 KB of shared memory
__host__ __device__ constexpr uint32_t fa_tile_rows(uint32_t hd) { return 24576u / (hd * 2u); }

// The loops over cached rows are real loops (two rows per trip): a kernel that runs once per layer and
// token pays for every instruction it has to fetch, so the code is kept small and the memory
// parallelism comes from the asynchronous copies, not from unrolling.
template <int VEC, int GT>
__global__ void __launch_bounds__(FA_THREADS) attn_fused_kernel(const FusedAttnArgs a) {
    pdl_launch_dependents();
    // first half of a cluster barrier that only says "this CTA has started": its second half stands before the
    // first store into a peer's shared memory and has long completed by then
    asm volatile("barrier.cluster.arrive.relaxed.aligned;\n" ::: "memory");
    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t S = cluster.dim_blocks().x, rank = cluster.block_rank();
    constexpr uint32_t hd = 32 * VEC;
    constexpr uint32_t PR = fa_tile_rows(hd);      // cached rows staged per pass
    constexpr uint32_t HL = 32 / GT;               // lanes that end up with the same head's score
    extern __shared__ __align__(16) float fa_dyn[];
    float *sc = fa_dyn;                                            // [chunk_cap][GT] scores, then exp
    float *qs = fa_dyn + (((size_t)a.chunk_cap * GT + 3) & ~(size_t)3);  // [GT][hd] rotated q (16-byte aligned)
    uint16_t *newk = reinterpret_cast<uint16_t *>(qs + GT * hd);   // [hd] this token's rotated k, [hd] its v
    uint16_t *newv = newk + hd;
    uint16_t *kt = newv + hd;                                      // [PR][hd] key tile
    uint16_t *vt = kt + PR * hd;                                   // [PR][hd] value tile
    float *part = reinterpret_cast<float *>(kt);                   // after the last tile: [FA_WARPS][GT*hd] partial outputs
    float *recv = reinterpret_cast<float *>(vt + PR * hd);         // [S][slice]: every rank's partial sums of the outputs this CTA finishes
    __shared__ float sh[FA_WARPS][GT];
    __shared__ float xall[2][8][GT];               // maxima and sums of every CTA of the cluster, stored here by their owners
    __shared__ float sinv[GT];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, b = blockIdx.y;
    const uint32_t g = a.nh / a.nkv, n_tiles = (g + GT - 1) / GT, kvd = a.nkv * hd;
    const uint32_t cl = blockIdx.x / S, kh = cl / n_tiles, tile = cl - kh * n_tiles;
    const uint32_t h0 = kh * g + tile * GT;        // first query head of this cluster
    const uint32_t nhl = min((uint32_t)GT, g - tile * GT);

    const uint32_t cseq = a.prefill ? a.seq : b;   // which sequence's cache
    uint16_t *kcb = a.kc + (size_t)kh * hd;
    uint16_t *vcb = a.vc + (size_t)kh * hd;
    const uint64_t seq_rows = a.seq_stride / kvd;  // rows of a sequence's slab (contiguous cache)
    auto row_of = [&](uint32_t p) { return fa_row(a.page_tbl, a.page_shift, a.tbl_stride, seq_rows, cseq, p) * kvd; };
    constexpr uint32_t PPR = hd / 8;               // 16-byte pieces per row

    // Everything that follows from the token position: which cache rows this CTA covers, where the new row goes.
    int32_t pos;
    bool have_new;
    uint32_t sl, new_slot, p_begin, p_end, n_loc, n_pass;
    auto place = [&](int32_t pos_now) {
        pos = pos_now + (a.prefill ? (int32_t)b : 0);
        const int64_t slot64 = (int64_t)pos * a.slot_mul + a.slot_add;
        have_new = !a.prefill && slot64 >= 0 && slot64 < (int64_t)a.max_seq;  // a full cache takes no new row
        sl = (uint32_t)(slot64 + 1);
        if (slot64 < 0) sl = 0;
        if (sl > a.max_seq) sl = a.max_seq;
        new_slot = have_new ? (uint32_t)slot64 : 0xFFFFFFFFu;
        uint32_t chunk = (sl + S - 1) / S;
        if (chunk > a.chunk_cap) chunk = a.chunk_cap;  // cannot happen with chunk_cap = ceil(max_seq / S)
        p_begin = min(sl, rank * chunk);
        p_end = min(sl, p_begin + chunk);
        n_loc = p_end - p_begin;
        n_pass = (n_loc + PR - 1) / PR;
    };
    // rows [r0, r0 + n) of this CTA's range into the tiles (the new token's row comes from registers instead)
    auto stage = [&](uint32_t r0, uint32_t n, bool with_k) {
        for (uint32_t i = threadIdx.x; i < n * PPR; i += FA_THREADS) {
            const uint32_t r = i / PPR, c = i - r * PPR, p = p_begin + r0 + r;
            if (p == new_slot) continue;
            const size_t ro = row_of(p);
            if (with_k) fa_cp16(kt + r * hd + c * 8, kcb + ro + c * 8);
            fa_cp16(vt + r * hd + c * 8, vcb + ro + c * 8);
        }
    };
    // A decode step's predecessor in the stream (the q/k/v projection) does not touch the cache, and the rows
    // below the new token's were written steps ago: with `early_cache` the first tiles are requested and the
    // rotation angles computed BEFORE the dependency wait, on the position as it reads now.  The position is
    // read again after the wait; should it have changed (the kernel that advances it had not finished yet),
    // the speculative tiles are dropped and everything is placed again.  Prefill rows are written by the
    // kernel right before this one, so prefill waits first.
    const volatile int32_t *pos_ptr = a.pos_dev;
    const bool early = a.early_cache && !a.prefill;
    if (!early) pdl_wait();
    const int32_t pos_seen = *pos_ptr;
    place(pos_seen);
    stage(0, min(n_loc, PR), true);                // requested before anything else is computed
    float ca[VEC], sa[VEC];
    fa_rope_angles<VEC>(ca, sa, lane, (float)pos, a.inv_freq);
    if (early) {
        pdl_wait();
        const int32_t pos_now = *pos_ptr;
        if (pos_now != pos_seen) {                 // the same value in every thread of the cluster
            fa_cp_wait_all();
            __syncthreads();
            place(pos_now);
            stage(0, min(n_loc, PR), true);
            fa_rope_angles<VEC>(ca, sa, lane, (float)pos, a.inv_freq);
        }
    }

    // ---- rotation: warp w prepares query head w of the group, warp 0 also the new token's k and v ----
    {
        for (uint32_t hh = warp; hh < (uint32_t)GT; hh += FA_WARPS) {
            float x[VEC];
            const uint16_t *q = a.q + (size_t)b * a.src_stride + (size_t)(h0 + hh) * hd + lane * VEC;
#pragma unroll
            for (int i = 0; i < VEC; i++) x[i] = hh < nhl ? fa_h2f(q[i]) : 0.0f;
            fa_rope_apply<VEC>(x, ca, sa, lane);
#pragma unroll
            for (int i = 0; i < VEC; i++) qs[hh * hd + lane * VEC + i] = x[i];
        }
        if (warp == 0) {
            float kn[VEC];
            const uint16_t *k = a.k + (size_t)b * a.src_stride + (size_t)kh * hd + lane * VEC;
            const uint16_t *v = a.v + (size_t)b * a.src_stride + (size_t)kh * hd + lane * VEC;
#pragma unroll
            for (int i = 0; i < VEC; i++) kn[i] = fa_h2f(k[i]);
            if (a.rope_k) fa_rope_apply<VEC>(kn, ca, sa, lane);
            const bool own_new = have_new && new_slot >= p_begin && new_slot < p_end;
            const size_t new_off = (own_new && tile == 0) ? row_of(new_slot) : 0;
#pragma unroll
            for (int i = 0; i < VEC; i++) {
                const uint16_t kb = fa_f2h(kn[i]), vb = v[i];
                newk[lane * VEC + i] = kb;
                newv[lane * VEC + i] = vb;
                // KVCache::append: the first head tile of a group stores the row for all later steps
                if (own_new && tile == 0) {
                    kcb[new_off + lane * VEC + i] = kb;
                    vcb[new_off + lane * VEC + i] = vb;
                }
            }
        }
    }
    fa_cp_wait_all();
    __syncthreads();

    // ---- q of every head of the group in registers --------------------------------------------------
    float qf[GT][VEC];
#pragma unroll
    for (int hh = 0; hh < GT; hh++)
#pragma unroll
        for (int i = 0; i < VEC; i++) qf[hh][i] = qs[hh * hd + lane * VEC + i];

    // ---- scores of this CTA's positions: one warp per position, GT heads per row -------------------
    const float div = sqrtf((float)hd);
    for (uint32_t ps = 0; ps < n_pass; ps++) {
        const uint32_t r0 = ps * PR, n = min(PR, n_loc - r0);
        if (ps > 0) {
            __syncthreads();                       // every warp is done with the previous tile
            stage(r0, n, true);
            fa_cp_wait_all();
            __syncthreads();
        }
#pragma unroll 2
        for (uint32_t r = warp; r < n; r += FA_WARPS) {
            const uint32_t p = p_begin + r0 + r;
            const uint16_t *krow = (p == new_slot ? newk : kt + r * hd) + lane * VEC;
            float kf[VEC], s[GT];
#pragma unroll
            for (int i = 0; i < VEC; i++) kf[i] = fa_h2f(krow[i]);
#pragma unroll
            for (int hh = 0; hh < GT; hh++) {
                s[hh] = 0.0f;
#pragma unroll
                for (int i = 0; i < VEC; i++) s[hh] += qf[hh][i] * kf[i];
            }
            const float tot = fa_reduce_heads<GT>(s, lane);
            if ((lane & (HL - 1)) == 0) sc[(size_t)(r0 + r) * GT + lane / HL] = tot / div;
        }
    }
    __syncthreads();

    // ---- maximum over all positions, per head: local, then across the cluster --------------------
    // entry idx of the score buffer belongs to head idx % GT; FA_THREADS is a multiple of GT, so a
    // thread only ever sees its own head hm = threadIdx.x % GT
    const uint32_t hm = threadIdx.x % GT;
    float mx = -INFINITY;
    for (uint32_t idx = threadIdx.x; idx < n_loc * GT; idx += FA_THREADS) mx = fmaxf(mx, sc[idx]);
#pragma unroll
    for (int o = 16; o >= GT; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    if (lane < GT) sh[warp][lane] = mx;
    __syncthreads();
    asm volatile("barrier.cluster.wait.aligned;\n" ::: "memory");
    if (threadIdx.x < GT) {
        float m = -INFINITY;
        for (int w = 0; w < FA_WARPS; w++) m = fmaxf(m, sh[w][threadIdx.x]);
        fa_scatter(cluster, &xall[0][rank][threadIdx.x], S, m);
    }
    cluster.sync();
    mx = -INFINITY;
    for (uint32_t r = 0; r < S; r++) mx = fmaxf(mx, xall[0][r][hm]);

    // ---- exp and its sum: local in warp order, then across the cluster in rank order -------------
    float es = 0.0f;
    for (uint32_t idx = threadIdx.x; idx < n_loc * GT; idx += FA_THREADS) {
        const float e = expf(sc[idx] - mx);
        sc[idx] = e;
        es += e;
    }
#pragma unroll
    for (int o = 16; o >= GT; o >>= 1) es += __shfl_xor_sync(0xFFFFFFFFu, es, o);
    if (lane < GT) sh[warp][lane] = es;
    __syncthreads();
    if (threadIdx.x < GT) {
        float t = 0.0f;
        for (int w = 0; w < FA_WARPS; w++) t += sh[w][threadIdx.x];
        fa_scatter(cluster, &xall[1][rank][threadIdx.x], S, t);
    }
    cluster.sync();
    if (threadIdx.x < GT) {
        float t = 0.0f;
        for (uint32_t r = 0; r < S; r++) t += xall[1][r][threadIdx.x];  // rank order
        sinv[threadIdx.x] = 1.0f / (t + 1e-10f);
    }
    __syncthreads();
    float inv[GT];
#pragma unroll
    for (int hh = 0; hh < GT; hh++) inv[hh] = sinv[hh];

    // ---- weighted sum of the value rows -----------------------------------------------------------
    float ac[GT][VEC];
#pragma unroll
    for (int hh = 0; hh < GT; hh++)
#pragma unroll
        for (int i = 0; i < VEC; i++) ac[hh][i] = 0.0f;
    for (uint32_t ps = 0; ps < n_pass; ps++) {
        const uint32_t r0 = ps * PR, n = min(PR, n_loc - r0);
        if (n_pass > 1) {                          // with one pass the value tile is still the one staged at the start
            __syncthreads();
            stage(r0, n, false);
            fa_cp_wait_all();
            __syncthreads();
        }
#pragma unroll 2
        for (uint32_t r = warp; r < n; r += FA_WARPS) {
            const uint32_t p = p_begin + r0 + r;
            const uint16_t *vrow = (p == new_slot ? newv : vt + r * hd) + lane * VEC;
            const float *ep = sc + (size_t)(r0 + r) * GT;
            float vf[VEC];
#pragma unroll
            for (int i = 0; i < VEC; i++) vf[i] = fa_h2f(vrow[i]);
#pragma unroll
            for (int hh = 0; hh < GT; hh++) {
                const float e = ep[hh];
#pragma unroll
                for (int i = 0; i < VEC; i++) ac[hh][i] += __fmul_rn(__fmul_rn(e, vf[i]), inv[hh]);
            }
        }
    }
    __syncthreads();                               // the tiles are dead: their space takes the partial outputs
#pragma unroll
    for (int hh = 0; hh < GT; hh++)
#pragma unroll
        for (int i = 0; i < VEC; i++) part[(size_t)warp * (GT * hd) + hh * hd + lane * VEC + i] = ac[hh][i];
    __syncthreads();
    // Output element t is finished by rank t / per: every CTA adds its warps' partial sums and stores the result
    // into slot [its rank] of the finishing CTA's receive buffer; after one cluster barrier the finisher adds the
    // slots in rank order from its own shared memory.  Nobody touches a peer's memory after that barrier.
    const uint32_t n_out = nhl * hd, per = (n_out + S - 1) / S;
    for (uint32_t t = threadIdx.x; t < n_out; t += FA_THREADS) {
        float v = 0.0f;
#pragma unroll
        for (uint32_t w = 0; w < (uint32_t)FA_WARPS; w++) v += part[(size_t)w * (GT * hd) + t];
        const uint32_t owner = t / per;
        *cluster.map_shared_rank(recv + rank * per + (t - owner * per), owner) = v;
    }
    cluster.sync();
    {
        const uint32_t t_end = min(n_out, (rank + 1) * per);
        for (uint32_t t = rank * per + threadIdx.x; t < t_end; t += FA_THREADS) {
            float o = 0.0f;
            for (uint32_t r = 0; r < S; r++) o += recv[r * per + (t - rank * per)];  // rank order
            a.out[(size_t)b * a.nh * hd + (size_t)h0 * hd + t] = fa_f2h(o);
        }
    }
}

bool attn_fused_eligible(const AttnArgs &a) {
    return !a.int8 && (a.hd == 32 || a.hd == 64 || a.hd == 128 || a.hd == 256) && a.pos_dev != nullptr &&
           a.nkv != 0 && a.nh % a.nkv == 0 && (a.seq_stride * 2) % 16 == 0 &&
           reinterpret_cast<uintptr_t>(a.k) % 16 == 0 && reinterpret_cast<uintptr_t>(a.v) % 16 == 0;
}

// Prefill: RoPE of k (when the profile asks for it) and KVCache::append for T consecutive tokens of one
// sequence at once -- what T decode steps would have left in the cache (rope_inplace,
// cpu_fallback.rs:131-143; KVCache::append).  One warp per (token, kv head); rows are src_stride apart.
template <int VEC>
__global__ void __launch_bounds__(256) prefill_kv_kernel(const uint16_t *__restrict__ k, const uint16_t *__restrict__ v,
                                                         uint32_t src_stride, uint16_t *kc, uint16_t *vc, uint32_t nkv,
                                                         uint32_t n_tok, const int32_t *pos_dev, uint32_t max_seq,
                                                         uint32_t rope_k, const float *__restrict__ inv_freq,
                                                         const int32_t *__restrict__ page_tbl, uint32_t page_shift,
                                                         uint32_t tbl_stride, uint64_t seq_rows, uint32_t seq) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr uint32_t hd = 32 * VEC;
    const uint32_t lane = threadIdx.x & 31, w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= n_tok * nkv) return;
    const uint32_t t = w / nkv, kh = w - t * nkv;
    const int32_t pos = *pos_dev + (int32_t)t;
    if (pos < 0 || (uint32_t)pos >= max_seq) return;
    const uint16_t *kr = k + (size_t)t * src_stride + (size_t)kh * hd + lane * VEC;
    const uint16_t *vr = v + (size_t)t * src_stride + (size_t)kh * hd + lane * VEC;
    float kn[VEC];
#pragma unroll
    for (int i = 0; i < VEC; i++) kn[i] = fa_h2f(kr[i]);
    if (rope_k) {
        float ca[VEC], sa[VEC];
        fa_rope_angles<VEC>(ca, sa, lane, (float)pos, inv_freq);
        fa_rope_apply<VEC>(kn, ca, sa, lane);
    }
    const size_t off = fa_row(page_tbl, page_shift, tbl_stride, seq_rows, seq, (uint32_t)pos) * nkv * hd + (size_t)kh * hd + lane * VEC;
#pragma unroll
    for (int i = 0; i < VEC; i++) {
        kc[off + i] = fa_f2h(kn[i]);
        vc[off + i] = vr[i];
    }
}

// shared memory of a launch: the score buffer and the per-warp partial outputs
static size_t fa_smem_bytes(uint32_t chunk_cap, uint32_t gt, uint32_t hd) {
    // scores, rotated q, the new token's k and v, and the key/value tiles (48 KB; the per-warp partial
    // outputs, at most 32 KB, reuse the tiles' space)
    // and the receive buffer of the final reduction (one slice per rank, together at most gt*hd + 8 floats)
    return (((size_t)chunk_cap * gt + 3) & ~(size_t)3) * 4 + (size_t)gt * hd * 4 + 2 * hd * 2 + 2 * (size_t)fa_tile_rows(hd) * hd * 2 +
           ((size_t)gt * hd + 8) * 4;
}

template <int VEC, int GT>
static int launch_attn_fused_v(prism_cuda_ctx *ctx, const FusedAttnArgs &fa, uint32_t S) {
    const uint32_t g = fa.nh / fa.nkv, n_tiles = (g + GT - 1) / GT;
    const size_t smem = fa_smem_bytes(fa.chunk_cap, GT, 32 * VEC);
    if (smem > 215 * 1024) return fail(ctx, PRISM_E_ARG, "fused attention: max_seq too large for the score buffer");
    static bool configured[PRISM_MAX_DEVICES] = {false};
    if (smem > 32 * 1024 && !configured[ctx->device]) {
        PRISM_CUDA_TRY(ctx, cudaFuncSetAttribute(attn_fused_kernel<VEC, GT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 215 * 1024));
        configured[ctx->device] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(fa.nkv * n_tiles * S, fa.batch);
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
    (void)cudaLaunchKernelEx(&cfg, attn_fused_kernel<VEC, GT>, fa);
    return after_launch(ctx, "attn_fused_kernel");
}

template <int VEC>
static int launch_attn_fused_g(prism_cuda_ctx *ctx, const FusedAttnArgs &fa, uint32_t S) {
    // query heads served per pass over the cache: the group size rounded up to a power of two, at
    // most 8 (4 for 256-wide heads: registers)
    const uint32_t g = fa.nh / fa.nkv;
    uint32_t cap = VEC == 8 ? 4 : 8;
    // A small model with few KV heads would leave most of the GPU idle (0.5B: 2 KV heads x 2 CTAs): serve fewer
    // heads per cluster until about two dozen CTAs run; the cached rows are then read once per cluster, from L2.
    while (cap > 1 && fa.nkv * ((g + cap - 1) / cap) * S * fa.batch < 24 && g > cap / 2) cap /= 2;
    if (ctx->attn_group > 0) cap = min(cap, (uint32_t)ctx->attn_group);
    if (g >= 5 && cap >= 8) return launch_attn_fused_v<VEC, (VEC == 8 ? 4 : 8)>(ctx, fa, S);
    if (g >= 3 && cap >= 4) return launch_attn_fused_v<VEC, 4>(ctx, fa, S);
    if (g >= 2 && cap >= 2) return launch_attn_fused_v<VEC, 2>(ctx, fa, S);
    return launch_attn_fused_v<VEC, 1>(ctx, fa, S);
}

// The rotation frequencies base^(-2j/hd), j < hd/2, as the CPU path computes them (powf in fp32,
// cpu_fallback.rs:137), once per (head size, base) on the host and kept on the device.
static int rope_table(prism_cuda_ctx *ctx, uint32_t hd, float base, const float **out) {
    for (auto *t : ctx->rope_tabs) {
        if (t->hd == hd && t->base == base) {
            *out = t->dev;
            return PRISM_OK;
        }
    }
    auto *t = new prism_cuda_ctx::RopeTab{hd, base, nullptr, {0}};
    cudaError_t e = cudaMalloc((void **)&t->dev, 128 * sizeof(float));
    if (e != cudaSuccess) {
        delete t;
        return cuda_fail(ctx, e, "cudaMalloc(rope table)");
    }
    for (uint32_t j = 0; j < hd / 2; j++) t->host[j] = powf(base, -2.0f * (float)j / (float)hd);
    ctx->rope_tabs.push_back(t);
    // the host copy lives as long as the context, so the asynchronous copy may read it after this returns
    PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(t->dev, t->host, (hd / 2) * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    *out = t->dev;
    return PRISM_OK;
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
    fa.rope_k = rope_k;
    fa.prefill = a.prefill; fa.seq = a.prefill_seq;
    fa.page_tbl = a.page_tbl; fa.page_shift = a.page_shift; fa.tbl_stride = a.tbl_stride;
    fa.early_cache = a.early_cache;
    PRISM_TRY(rope_table(ctx, a.hd, rope_base, &fa.inv_freq));
    if (a.prefill) {
        // the tokens' keys and values go to the cache first; the attention launch then finds them there
        const unsigned warps = a.batch * a.nkv, blocks = (warps + 7) / 8;
        const uint64_t seq_rows = a.seq_stride / (a.nkv * a.hd);
#define PRISM_PF_KV(V)                                                                                                  \
    launch_pdl(ctx, "prefill_kv_kernel", prefill_kv_kernel<V>, dim3(blocks), dim3(256), 0, k_src, v_src, a.q_stride, fa.kc, \
               fa.vc, a.nkv, a.batch, a.pos_dev, a.max_seq, rope_k, fa.inv_freq, a.page_tbl, a.page_shift, a.tbl_stride,  \
               seq_rows, a.prefill_seq)
        switch (a.hd) {
        case 32: PRISM_PF_KV(1); break;
        case 64: PRISM_PF_KV(2); break;
        case 128: PRISM_PF_KV(4); break;
        default: PRISM_PF_KV(8); break;
        }
#undef PRISM_PF_KV
        PRISM_TRY(after_launch(ctx, "prefill_kv_kernel"));
    }
    // cluster size: a CTA stages up to 96 cached rows of 128-wide heads per pass; more CTAs per group
    // spread the rows (and the latency of fetching them) over more SMs
    uint32_t S = a.max_seq > 512 ? 8 : a.max_seq > 256 ? 4 : a.max_seq > 128 ? 2 : 1;
    if (ctx->attn_cluster == 1 || ctx->attn_cluster == 2 || ctx->attn_cluster == 4 || ctx->attn_cluster == 8)
        S = (uint32_t)ctx->attn_cluster;
    fa.chunk_cap = (a.max_seq + S - 1) / S;
    switch (a.hd) {
    case 32: return launch_attn_fused_g<1>(ctx, fa, S);
    case 64: return launch_attn_fused_g<2>(ctx, fa, S);
    case 128: return launch_attn_fused_g<4>(ctx, fa, S);
    default: return launch_attn_fused_g<8>(ctx, fa, S);
    }
}

}  // namespace prism
