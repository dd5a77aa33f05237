// Decode-step glue kernels: the device twins of the CPU ops in
// src/lut/cpu_fallback.rs:39-143 and of the helpers inside step()
// (src/lut/engine_impl.rs:1076-1459).  All intermediate math is fp32 and every
// store rounds to fp16 (RNE) at the same points as the reference.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace prism {

__device__ __forceinline__ float h2f(uint16_t v) { return __half2float(__ushort_as_half(v)); }
__device__ __forceinline__ uint16_t f2h(float v) { return __half_as_ushort(__float2half_rn(v)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}

// Block-wide sum; every thread gets the result.  `sh` holds >= 32 floats.
__device__ float block_sum(float v, float *sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    float r = 0.0f;
    for (int i = 0; i < nw; i++) r += sh[i];  // fixed order: deterministic
    return r;
}
__device__ float block_max(float v, float *sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    float r = -INFINITY;
    for (int i = 0; i < nw; i++) r = fmaxf(r, sh[i]);
    return r;
}

// rms_norm_inplace (cpu_fallback.rs:39-54): x * 1/sqrt(mean(x^2)+eps), no weight.
// One block per sequence; each thread keeps its (up to 16) elements in registers between the
// sum of squares and the scaling, so the vector is read once.
constexpr int RMS_THREADS = 1024;
__global__ void __launch_bounds__(RMS_THREADS) rms_norm_kernel(const uint16_t *__restrict__ in,
                                                               uint16_t *__restrict__ out, uint32_t n, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float sh[32];
    const uint16_t *x = in + (size_t)blockIdx.x * n;
    uint16_t *y = out + (size_t)blockIdx.x * n;
    const bool vec = (n % 8 == 0) && n <= RMS_THREADS * 16 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) % 16 == 0);
    if (vec) {
        uint4 v[2];
        float ss = 0.0f;
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const uint32_t i = (threadIdx.x + u * RMS_THREADS) * 8;
            v[u] = make_uint4(0, 0, 0, 0);
            if (i < n) {
                v[u] = *reinterpret_cast<const uint4 *>(x + i);
                const uint16_t *e = reinterpret_cast<const uint16_t *>(&v[u]);
#pragma unroll
                for (int k = 0; k < 8; k++) { const float f = h2f(e[k]); ss += f * f; }
            }
        }
        ss = block_sum(ss, sh);
        const float inv = 1.0f / sqrtf(ss / (float)n + eps);
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const uint32_t i = (threadIdx.x + u * RMS_THREADS) * 8;
            if (i < n) {
                uint4 o;
                const uint16_t *e = reinterpret_cast<const uint16_t *>(&v[u]);
                uint16_t *d = reinterpret_cast<uint16_t *>(&o);
#pragma unroll
                for (int k = 0; k < 8; k++) d[k] = f2h(h2f(e[k]) * inv);
                *reinterpret_cast<uint4 *>(y + i) = o;
            }
        }
        return;
    }
    float ss = 0.0f;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        float f = h2f(x[i]);
        ss += f * f;
    }
    ss = block_sum(ss, sh);
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) y[i] = f2h(h2f(x[i]) * inv);
}

int launch_rms_norm(prism_cuda_ctx *ctx, const uint16_t *in, uint16_t *out, uint32_t n, float eps,
                    uint32_t batch) {
    launch_pdl(ctx, "rms_norm_kernel", rms_norm_kernel, batch, RMS_THREADS, 0, in, out, n, eps);
    return after_launch(ctx, "rms_norm_kernel");
}

// rope_inplace (cpu_fallback.rs:131-143): pairs (j, j+hd/2) of every head chunk.
// The position comes from device memory when pos_dev is set (graph replay).
__global__ void rope_kernel(uint16_t *__restrict__ x, uint32_t n, const int32_t *__restrict__ pos_dev,
                            int64_t pos_host, uint32_t hd, float base, uint32_t x_stride) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t half = hd / 2;
    const uint32_t pairs = (n / hd) * half;
    uint16_t *xb = x + (size_t)blockIdx.y * x_stride;
    const float pos = pos_dev ? (float)(*pos_dev) : (float)pos_host;
    for (uint32_t p = blockIdx.x * blockDim.x + threadIdx.x; p < pairs; p += gridDim.x * blockDim.x) {
        const uint32_t head = p / half, j = p % half;
        const uint32_t i0 = head * hd + j, i1 = i0 + half;
        const float a = h2f(xb[i0]), b = h2f(xb[i1]);
        const float ang = pos * powf(base, -2.0f * (float)j / (float)hd);
        float sa, ca;
        sincosf(ang, &sa, &ca);
        xb[i0] = f2h(__fsub_rn(__fmul_rn(a, ca), __fmul_rn(b, sa)));
        xb[i1] = f2h(__fadd_rn(__fmul_rn(a, sa), __fmul_rn(b, ca)));
    }
}

int launch_rope(prism_cuda_ctx *ctx, uint16_t *x, uint32_t n, const int32_t *pos_dev, int64_t pos_host,
                uint32_t head_dim, float base, uint32_t batch, uint32_t x_stride) {
    const uint32_t pairs = (n / head_dim) * (head_dim / 2);
    dim3 grid((pairs + 127) / 128, batch);
    launch_pdl(ctx, "rope_kernel", rope_kernel, grid, 128, 0, x, n, pos_dev, pos_host, head_dim, base, x_stride);
    return after_launch(ctx, "rope_kernel");
}

// vec_add_inplace (cpu_fallback.rs:56-62)
__global__ void vec_add_kernel(uint16_t *__restrict__ a, const uint16_t *__restrict__ b, uint32_t n) {
    pdl_launch_dependents();
    pdl_wait();
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) a[i] = f2h(h2f(a[i]) + h2f(b[i]));
}
int launch_vec_add(prism_cuda_ctx *ctx, uint16_t *a, const uint16_t *b, uint32_t n) {
    launch_pdl(ctx, "vec_add_kernel", vec_add_kernel, (n + 255) / 256, 256, 0, a, b, n);
    return after_launch(ctx, "vec_add_kernel");
}

// silu_inplace (cpu_fallback.rs:66-71)
__global__ void silu_kernel(uint16_t *__restrict__ x, uint32_t n) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        float f = h2f(x[i]);
        x[i] = f2h(f / (1.0f + expf(-f)));
    }
}
int launch_silu(prism_cuda_ctx *ctx, uint16_t *x, uint32_t n) {
    silu_kernel<<<(n + 255) / 256, 256, 0, ctx->stream>>>(x, n);
    return after_launch(ctx, "silu_kernel");
}

// Activation arm of step() (engine_impl.rs:1355-1366): g = f16(silu(g)); g = f16(g*u).
__global__ void silu_mul_kernel(uint16_t *__restrict__ out, const uint16_t *__restrict__ g,
                                const uint16_t *__restrict__ u, uint32_t n) {
    pdl_launch_dependents();
    pdl_wait();
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        float f = h2f(g[i]);
        float s = h2f(f2h(f / (1.0f + expf(-f))));
        out[i] = f2h(s * h2f(u[i]));
    }
}
int launch_silu_mul(prism_cuda_ctx *ctx, uint16_t *out, const uint16_t *g, const uint16_t *u, uint32_t n) {
    launch_pdl(ctx, "silu_mul_kernel", silu_mul_kernel, (n + 255) / 256, 256, 0, out, g, u, n);
    return after_launch(ctx, "silu_mul_kernel");
}

// Row softmax in fp32, fp16 out (MetalBackend::softmax_metal, engine_impl.rs:348-375).
__global__ void softmax_kernel(const uint16_t *__restrict__ in, uint16_t *__restrict__ out, uint32_t n) {
    __shared__ float sh[32];
    float mx = -INFINITY;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) mx = fmaxf(mx, h2f(in[i]));
    mx = block_max(mx, sh);
    float s = 0.0f;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) s += expf(h2f(in[i]) - mx);
    s = block_sum(s, sh);
    const float inv = 1.0f / s;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) out[i] = f2h(expf(h2f(in[i]) - mx) * inv);
}
int launch_softmax(prism_cuda_ctx *ctx, const uint16_t *in, uint16_t *out, uint32_t n) {
    softmax_kernel<<<1, 256, 0, ctx->stream>>>(in, out, n);
    return after_launch(ctx, "softmax_kernel");
}

// argmax (engine_impl.rs:1448-1459): first index holding the strictly greatest
// value; NaN never wins; an all-NaN/-inf vector gives 0.  A cluster of ARGMAX_CTAS
// blocks per sequence: each scans a slice with 16-byte loads, rank 0 merges the
// slices' winners through distributed shared memory.  Rows of `logits` are
// `stride` apart and 16-byte aligned.
constexpr int ARGMAX_CTAS = 8;
constexpr int ARGMAX_THREADS = 512;
__device__ __forceinline__ void argmax_take(float &bv, uint32_t &bi, float ov, uint32_t oi) {
    if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
    }
}
__global__ void __launch_bounds__(ARGMAX_THREADS) argmax_kernel(const uint16_t *__restrict__ logits, uint32_t n,
                                                                uint32_t stride, uint32_t *__restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t R = cluster.dim_blocks().x, rank = cluster.block_rank();
    __shared__ float sv[32];
    __shared__ uint32_t si[32];
    __shared__ float win_v;
    __shared__ uint32_t win_i;
    const uint32_t seq = blockIdx.x / R;
    const uint16_t *lg = logits + (size_t)seq * stride;
    // slice of this block, in groups of 8 values
    const uint32_t groups = (n + 7) / 8, per = (groups + R - 1) / R;
    const uint32_t g0 = min(groups, rank * per), g1 = min(groups, g0 + per);
    float bv = -INFINITY;
    uint32_t bi = 0xFFFFFFFFu;
    for (uint32_t g = g0 + threadIdx.x; g < g1; g += ARGMAX_THREADS) {
        const uint32_t i0 = g * 8;
        if (i0 + 8 <= n) {
            const uint4 v = *reinterpret_cast<const uint4 *>(lg + i0);
            const uint16_t *e = reinterpret_cast<const uint16_t *>(&v);
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const float f = h2f(e[k]);
                if (f > bv) {  // ascending index per thread: keeps the first maximum
                    bv = f;
                    bi = i0 + k;
                }
            }
        } else {
            for (uint32_t i = i0; i < n; i++) {
                const float f = h2f(lg[i]);
                if (f > bv) {
                    bv = f;
                    bi = i;
                }
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, o);
        const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
        argmax_take(bv, bi, ov, oi);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = ARGMAX_THREADS >> 5;
    if (lane == 0) {
        sv[warp] = bv;
        si[warp] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < nw; w++) argmax_take(bv, bi, sv[w], si[w]);
        win_v = bv;
        win_i = bi;
    }
    cluster.sync();
    if (rank == 0 && threadIdx.x == 0) {
        for (uint32_t r = 1; r < R; r++)
            argmax_take(bv, bi, *cluster.map_shared_rank(&win_v, r), *cluster.map_shared_rank(&win_i, r));
        if (bi == 0xFFFFFFFFu) bi = 0;
        out[seq] = bi;
    }
    cluster.sync();  // peers keep their shared memory alive until rank 0 has read it
}
int launch_argmax(prism_cuda_ctx *ctx, const uint16_t *logits, uint32_t n, uint32_t stride, uint32_t batch,
                  uint32_t *out_dev) {
    if ((reinterpret_cast<uintptr_t>(logits) & 15) || (batch > 1 && stride % 8))
        return fail(ctx, PRISM_E_ARG, "argmax: rows must be 16-byte aligned");
    launch_cluster_pdl(ctx, argmax_kernel, dim3(ARGMAX_CTAS * batch), dim3(ARGMAX_THREADS), 0, ARGMAX_CTAS, logits, n,
                       stride, out_dev);
    return after_launch(ctx, "argmax_kernel");
}

// KV append.  fp16 mode stores the GEMV outputs verbatim at [slot][kvd].
// int8 mode is KVCache::append's q() (engine_impl.rs:532-552): per token
// [f32 scale][kvd x i8], scale = 127/max|x| (1 when max <= 1e-10),
// round-half-away, clamp to [-128,127].
__global__ void kv_append_kernel(KvAppendArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float sh[32];
    const uint32_t b = blockIdx.x, which = blockIdx.y;
    const uint16_t *src = (which ? a.v : a.k) + (size_t)b * a.src_stride;
    const int64_t slot = (int64_t)(a.pos_dev ? *a.pos_dev : a.pos_host) * a.slot_mul + a.slot_add;
    if (slot < 0 || slot >= (int64_t)a.max_seq) return;  // full cache: host checks before launch
    if (!a.int8) {
        uint16_t *dst = reinterpret_cast<uint16_t *>(which ? a.vc : a.kc) + (size_t)b * a.seq_stride +
                        (size_t)slot * a.kvd;
        for (uint32_t i = threadIdx.x; i < a.kvd; i += blockDim.x) dst[i] = src[i];
        return;
    }
    float mx = 0.0f;
    for (uint32_t i = threadIdx.x; i < a.kvd; i += blockDim.x) mx = fmaxf(mx, fabsf(h2f(src[i])));
    mx = block_max(mx, sh);
    const float scale = mx > 1e-10f ? 127.0f / mx : 1.0f;
    uint8_t *dst = reinterpret_cast<uint8_t *>(which ? a.vc : a.kc) + (size_t)b * a.seq_stride +
                   (size_t)slot * (a.kvd + 4);
    if (threadIdx.x == 0) {
        uint32_t sb = __float_as_uint(scale);
        dst[0] = sb & 0xFF; dst[1] = (sb >> 8) & 0xFF; dst[2] = (sb >> 16) & 0xFF; dst[3] = sb >> 24;
    }
    for (uint32_t i = threadIdx.x; i < a.kvd; i += blockDim.x) {
        float v = roundf(h2f(src[i]) * scale);
        v = fminf(fmaxf(v, -128.0f), 127.0f);
        if (v != v) v = 0.0f;
        dst[4 + i] = (uint8_t)(int8_t)v;
    }
}
int launch_kv_append(prism_cuda_ctx *ctx, const KvAppendArgs &a) {
    dim3 grid(a.batch, 2);
    launch_pdl(ctx, "kv_append_kernel", kv_append_kernel, grid, 128, 0, a);
    return after_launch(ctx, "kv_append_kernel");
}

// attention_cpu (cpu_fallback.rs:84-127) for one query token per sequence.
// One block per (head, sequence).  scores = (q.k)/sqrt(hd); e = exp(s - max);
// out[d] = f16( sum_p e_p * v[p][d] * inv ), inv = 1/(sum e + 1e-10), with the
// `* inv` inside the sum as the reference has it.  K/V: [pos][kv_head][hd].
// In int8 mode a cached value is f16(i8 * (1/scale)) (dequant_inline,
// engine_impl.rs:569-584) before use.
constexpr int ATTN_THREADS = 256;

__device__ __forceinline__ float kv_load(const void *base, uint32_t int8, uint32_t kvd, uint32_t p,
                                         uint32_t off) {
    if (!int8) return h2f(reinterpret_cast<const uint16_t *>(base)[(size_t)p * kvd + off]);
    const uint8_t *blk = reinterpret_cast<const uint8_t *>(base) + (size_t)p * (kvd + 4);
    const uint32_t sb = blk[0] | (blk[1] << 8) | (blk[2] << 16) | ((uint32_t)blk[3] << 24);
    const float inv = 1.0f / __uint_as_float(sb);
    return h2f(f2h((float)(int8_t)blk[4 + off] * inv));
}

__global__ void __launch_bounds__(ATTN_THREADS) attention_kernel(AttnArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float sc[];  // [sl] scores, then exp
    __shared__ float sh[32];
    __shared__ float qs[256];
    const uint32_t h = blockIdx.x, b = blockIdx.y;
    uint32_t sl = (uint32_t)((a.pos_dev ? *a.pos_dev : a.pos_host) * (int32_t)a.slot_mul + (int32_t)a.slot_add + 1);
    if (sl > a.max_seq) sl = a.max_seq;  // never index past the score buffer / cache
    const uint32_t g = a.nh / (a.nkv ? a.nkv : 1), kh = h / g, kvd = a.nkv * a.hd, hd = a.hd;
    const uint16_t *q = a.q + (size_t)b * a.q_stride + (size_t)h * hd;
    const char *kb = reinterpret_cast<const char *>(a.k) + (size_t)b * a.seq_stride * (a.int8 ? 1 : 2);
    const char *vb = reinterpret_cast<const char *>(a.v) + (size_t)b * a.seq_stride * (a.int8 ? 1 : 2);
    for (uint32_t d = threadIdx.x; d < hd; d += blockDim.x) qs[d] = h2f(q[d]);
    __syncthreads();
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const float div = sqrtf((float)hd);
    // scores: one warp per position, lanes over head_dim
    for (uint32_t p = warp; p < sl; p += nw) {
        float s = 0.0f;
        for (uint32_t d = lane; d < hd; d += 32) s += qs[d] * kv_load(kb, a.int8, kvd, p, kh * hd + d);
        s = warp_sum(s);
        if (lane == 0) sc[p] = s / div;
    }
    __syncthreads();
    float mx = -INFINITY;
    for (uint32_t p = threadIdx.x; p < sl; p += blockDim.x) mx = fmaxf(mx, sc[p]);
    mx = block_max(mx, sh);
    float es = 0.0f;
    for (uint32_t p = threadIdx.x; p < sl; p += blockDim.x) {
        float e = expf(sc[p] - mx);
        sc[p] = e;
        es += e;
    }
    es = block_sum(es, sh);
    const float inv = 1.0f / (es + 1e-10f);
    // output: thread (d, part) sums positions part, part+parts, ...; parts combined in order
    const uint32_t parts = blockDim.x / hd ? blockDim.x / hd : 1;
    __shared__ float po[ATTN_THREADS];
    const uint32_t d = threadIdx.x % hd, part = threadIdx.x / hd;
    float ac = 0.0f;
    if (part < parts) {
        for (uint32_t p = part; p < sl; p += parts)
            ac += __fmul_rn(__fmul_rn(sc[p], kv_load(vb, a.int8, kvd, p, kh * hd + d)), inv);
    }
    po[threadIdx.x] = ac;
    __syncthreads();
    if (threadIdx.x < hd) {
        float t = 0.0f;
        for (uint32_t i = 0; i < parts; i++) t += po[i * hd + threadIdx.x];
        a.out[(size_t)b * a.nh * hd + (size_t)h * hd + threadIdx.x] = f2h(t);
    }
}

// Same computation for fp16 caches with head_dim = 32*VEC: each lane owns VEC consecutive
// elements of the head, one warp works on one cached position at a time (four in flight), so K
// and V rows are read with coalesced vector loads and the loop over positions is spread over
// all warps of the block.  Partial outputs of the warps are combined in warp order.
template <int VEC>
__global__ void __launch_bounds__(ATTN_THREADS) attention_f16_kernel(AttnArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float sc[];  // [sl] scores, then exp
    __shared__ float sh[32];
    __shared__ float part[(ATTN_THREADS / 32) * 32 * VEC];
    constexpr uint32_t hd = 32 * VEC;
    const uint32_t h = blockIdx.x, b = blockIdx.y;
    uint32_t sl = (uint32_t)((a.pos_dev ? *a.pos_dev : a.pos_host) * (int32_t)a.slot_mul + (int32_t)a.slot_add + 1);
    if (sl > a.max_seq) sl = a.max_seq;
    const uint32_t g = a.nh / (a.nkv ? a.nkv : 1), kh = h / g, kvd = a.nkv * hd;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr uint32_t nw = ATTN_THREADS / 32;
    const uint16_t *q = a.q + (size_t)b * a.q_stride + (size_t)h * hd + lane * VEC;
    const uint16_t *kb = reinterpret_cast<const uint16_t *>(a.k) + (size_t)b * a.seq_stride + (size_t)kh * hd + lane * VEC;
    const uint16_t *vb = reinterpret_cast<const uint16_t *>(a.v) + (size_t)b * a.seq_stride + (size_t)kh * hd + lane * VEC;
    float qf[VEC];
#pragma unroll
    for (int i = 0; i < VEC; i++) qf[i] = h2f(q[i]);
    const float div = sqrtf((float)hd);
    struct alignas(2 * VEC) Row { uint16_t e[VEC]; };
    for (uint32_t p0 = warp; p0 < sl; p0 += 4 * nw) {
        Row r[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const uint32_t p = p0 + u * nw;
            if (p < sl) r[u] = *reinterpret_cast<const Row *>(kb + (size_t)p * kvd);
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const uint32_t p = p0 + u * nw;
            if (p < sl) {  // warp-uniform
                float s = 0.0f;
#pragma unroll
                for (int i = 0; i < VEC; i++) s += qf[i] * h2f(r[u].e[i]);
                s = warp_sum(s);
                if (lane == 0) sc[p] = s / div;
            }
        }
    }
    __syncthreads();
    float mx = -INFINITY;
    for (uint32_t p = threadIdx.x; p < sl; p += blockDim.x) mx = fmaxf(mx, sc[p]);
    mx = block_max(mx, sh);
    float es = 0.0f;
    for (uint32_t p = threadIdx.x; p < sl; p += blockDim.x) {
        float e = expf(sc[p] - mx);
        sc[p] = e;
        es += e;
    }
    es = block_sum(es, sh);
    const float inv = 1.0f / (es + 1e-10f);
    float ac[VEC];
#pragma unroll
    for (int i = 0; i < VEC; i++) ac[i] = 0.0f;
    for (uint32_t p0 = warp; p0 < sl; p0 += 4 * nw) {
        Row r[4];
        float e[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const uint32_t p = p0 + u * nw;
            e[u] = 0.0f;
            if (p < sl) {
                r[u] = *reinterpret_cast<const Row *>(vb + (size_t)p * kvd);
                e[u] = sc[p];
            }
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            if (p0 + u * nw < sl) {
#pragma unroll
                for (int i = 0; i < VEC; i++) ac[i] += __fmul_rn(__fmul_rn(e[u], h2f(r[u].e[i])), inv);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < VEC; i++) part[warp * hd + lane * VEC + i] = ac[i];
    __syncthreads();
    if (threadIdx.x < hd) {
        float t = 0.0f;
#pragma unroll
        for (uint32_t w = 0; w < nw; w++) t += part[w * hd + threadIdx.x];
        a.out[(size_t)b * a.nh * hd + (size_t)h * hd + threadIdx.x] = f2h(t);
    }
}

int launch_attention(prism_cuda_ctx *ctx, const AttnArgs &a) {
    if (a.hd > 256 || a.hd == 0 || ATTN_THREADS % a.hd != 0)
        return fail(ctx, PRISM_E_ARG, "attention: head_dim must divide 256");
    static bool configured[PRISM_MAX_DEVICES] = {false};
    const size_t smem = (size_t)a.max_seq * sizeof(float);
    if (smem > 160 * 1024) return fail(ctx, PRISM_E_ARG, "attention: max_seq too large for the score buffer");
    if (smem > 32 * 1024 && !configured[ctx->device]) {
        PRISM_CUDA_TRY(ctx, cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        PRISM_CUDA_TRY(ctx, cudaFuncSetAttribute(attention_f16_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        PRISM_CUDA_TRY(ctx, cudaFuncSetAttribute(attention_f16_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        PRISM_CUDA_TRY(ctx, cudaFuncSetAttribute(attention_f16_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        PRISM_CUDA_TRY(ctx, cudaFuncSetAttribute(attention_f16_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        configured[ctx->device] = true;
    }
    dim3 grid(a.nh, a.batch);
    const bool vec_ok = !a.int8 && (a.hd == 32 || a.hd == 64 || a.hd == 128 || a.hd == 256) &&
                        (reinterpret_cast<uintptr_t>(a.k) % 16 == 0) && (reinterpret_cast<uintptr_t>(a.v) % 16 == 0) &&
                        (a.seq_stride * 2) % 16 == 0;
    if (vec_ok) {
        switch (a.hd) {
        case 32: launch_pdl(ctx, "attention_f16_kernel", attention_f16_kernel<1>, grid, ATTN_THREADS, smem, a); break;
        case 64: launch_pdl(ctx, "attention_f16_kernel", attention_f16_kernel<2>, grid, ATTN_THREADS, smem, a); break;
        case 128: launch_pdl(ctx, "attention_f16_kernel", attention_f16_kernel<4>, grid, ATTN_THREADS, smem, a); break;
        default: launch_pdl(ctx, "attention_f16_kernel", attention_f16_kernel<8>, grid, ATTN_THREADS, smem, a); break;
        }
        return after_launch(ctx, "attention_f16_kernel");
    }
    launch_pdl(ctx, "attention_kernel", attention_kernel, grid, ATTN_THREADS, smem, a);
    return after_launch(ctx, "attention_kernel");
}

}  // namespace prism
