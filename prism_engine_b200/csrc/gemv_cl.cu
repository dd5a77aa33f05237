// Palettized GEMV for SMALL matrices: the pair-table tensor-core inner loop on a grid where latency,
// not bandwidth, decides (the linears of a sub-billion-parameter model: a 2.3 MB matrix streams in
// well under a microsecond, so what a launch costs is its chain of dependent memory round trips).
//
// y = W x, W as 4-bit palette indices + a 16-entry fp16 palette per row (lut_gemv_cpu,
// src/lut/cpu_fallback.rs:12-35; fused gate/up: engine_impl.rs FusedGateUp).
//
//  * A 64-row block belongs to ONE thread-block cluster of s = 1, 2, 4 or 8 CTAs; CTA r of the
//    cluster takes the r-th part of the block's K range.  The 64 sums of the s CTAs meet in
//    distributed shared memory (rank 0 adds them in rank order): no partial sums in global memory,
//    no arrival counters, no fix-up pass.
//  * Every index chunk of a CTA's range (at most 8 per warp) is requested, and the block's pair
//    table is built, BEFORE the kernel waits for its predecessor: weights do not depend on the
//    previous kernel, so under programmatic dependent launch all of that overlaps the predecessor's
//    tail.  What is left after the wait is: stage x (RMSNorm folded in if asked), the lookups and
//    MMAs on indices that are already in registers, the reduction, y.
#include <cooperative_groups.h>

#include "common.cuh"
#include "pair_table.cuh"

namespace cg = cooperative_groups;

namespace prism {

constexpr int CL_WARPS = 8;
constexpr int CL_THREADS = CL_WARPS * 32;
constexpr int CL_PF = 8;                              // index chunks a warp holds in registers
constexpr int CL_MAX_CHUNKS = CL_WARPS * CL_PF;       // chunks of one CTA's K part (2048 weights per row)
constexpr int CL_X_BYTES = CL_MAX_CHUNKS * 64;
constexpr int CL_MAX_S = 8;                           // largest cluster
constexpr size_t CL_SMEM_BYTES = SK_TBL_BYTES + CL_X_BYTES + CL_WARPS * 64 * 4 + CL_MAX_S * 64 * 4 + 32;

struct ClArgs {
    const uint8_t *idx1, *idx2;   // index arrays the two half-blocks of a block come from
    const uint16_t *pal1, *pal2;
    uint32_t n_chunks;            // chunks per row
    uint32_t hb_mul, hb_add2;     // block b = half-blocks hb_mul*b (rows "1") and hb_mul*b+hb_add2 (rows "2")
    uint32_t m;                   // valid output rows (per tensor)
    uint32_t s;                   // CTAs per block (cluster size)
    const uint16_t *x; uint32_t x_stride;
    uint16_t *y; uint32_t y_stride;
    const uint16_t *resid;
    unsigned int *err;
    uint32_t norm_n;              // > 0: stage rms_norm(x) (row of norm_n values) instead of x
    float norm_eps;
    TpPush tp;                    // GEMV_TP only: where the all-reduce of the block sums goes
};

// The table base is added at run time (SBASE = -1 of the lookup helpers): in a cluster launch the offset
// of a CTA's dynamic shared memory inside its shared window is not the same for every CTA, so the
// compile-time base the other pair-table kernels use does not exist here.
template <int MODE>
__global__ void __launch_bounds__(CL_THREADS) lut_gemv_cl_kernel(const ClArgs a) {
    constexpr int SBASE = -1;
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
    pdl_launch_dependents();
    cg::cluster_group cluster = cg::this_cluster();
    if (cluster.dim_blocks().x != a.s || a.n_chunks > a.s * (uint32_t)CL_MAX_CHUNKS) {  // not launched the way the host meant to
        if (threadIdx.x == 0) atomicExch(a.err, 6u);
        return;  // the same decision in every CTA of the cluster: nobody is left at a cluster barrier
    }
    uint32_t *tbl = reinterpret_cast<uint32_t *>(smem);
    uint16_t *xs = reinterpret_cast<uint16_t *>(smem + SK_TBL_BYTES);
    float *red = reinterpret_cast<float *>(smem + SK_TBL_BYTES + CL_X_BYTES);  // [CL_WARPS][64]
    float *cpush = red + CL_WARPS * 64;   // [CL_MAX_S][64]: on rank 0 the sums of every CTA of the cluster, stored there by their owners
    float &s_inv = *(cpush + CL_MAX_S * 64);
    // First half of a cluster barrier whose only purpose is that every CTA of the cluster has started before
    // anyone stores into rank 0's shared memory; its second half sits right before those stores and has long
    // completed by then.
    if (a.s > 1) asm volatile("barrier.cluster.arrive.relaxed.aligned;\n" ::: "memory");

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t s = a.s, rank = blockIdx.x % s, blk = blockIdx.x / s, bat = blockIdx.y;
    const uint32_t nc = a.n_chunks;
    const uint32_t cb = (uint32_t)((uint64_t)nc * rank / s), ce = (uint32_t)((uint64_t)nc * (rank + 1) / s);
    const uint32_t span = ce - cb;                       // <= CL_MAX_CHUNKS (checked on the host)
    const uint32_t hb1 = a.hb_mul * blk, hb2 = hb1 + a.hb_add2;
    const uint32_t nj = span > warp ? (span - warp + CL_WARPS - 1) / CL_WARPS : 0;  // this warp: chunks cb + warp + 8j

    // ---- every index chunk of this warp, in flight at once ------------------------------------------
    uint4 q1[CL_PF], q2[CL_PF];
    {
        const uint8_t *p1 = a.idx1 + ((size_t)hb1 * nc + cb + warp) * 512 + lane * 16;
        const uint8_t *p2 = a.idx2 + ((size_t)hb2 * nc + cb + warp) * 512 + lane * 16;
#pragma unroll
        for (int j = 0; j < CL_PF; j++) {
            if ((uint32_t)j < nj) {
                q1[j] = sk_ldg<0>(p1 + (size_t)j * CL_WARPS * 512);
                q2[j] = sk_ldg<0>(p2 + (size_t)j * CL_WARPS * 512);
            }
        }
    }
    // ---- pair tables: entry e = lo | hi<<4 -> half2{pal[lo], pal[hi]}; warp w writes hi = w, w + 8 ----
#pragma unroll
    for (int t = 0; t < 2; t++) {
        const uint32_t row = (t == 0 ? hb1 : hb2) * 32 + lane;
        const uint16_t *prow = (t == 0 ? a.pal1 : a.pal2) + (size_t)row * 16;
        const uint4 p0 = *reinterpret_cast<const uint4 *>(prow);
        const uint4 pp = *reinterpret_cast<const uint4 *>(prow + 8);
        const uint32_t cbp[8] = {p0.x, p0.y, p0.z, p0.w, pp.x, pp.y, pp.z, pp.w};
#pragma unroll
        for (int hh = 0; hh < 16 / CL_WARPS; hh++) {
            const uint32_t hi = warp + hh * CL_WARPS;
            const uint32_t hi_pair = hi < 2 ? cbp[0] : hi < 4 ? cbp[1] : hi < 6 ? cbp[2] : hi < 8 ? cbp[3]
                                   : hi < 10 ? cbp[4] : hi < 12 ? cbp[5] : hi < 14 ? cbp[6] : cbp[7];  // {pal[hi&~1], pal[hi|1]}
            const uint32_t hsel = (hi & 1) ? 0x7600u : 0x5400u;
#pragma unroll
            for (int lo = 0; lo < 16; lo++) {
                const uint32_t v = __byte_perm(cbp[lo >> 1], hi_pair, hsel | ((lo & 1) ? 0x32u : 0x10u));
                tbl[((uint32_t)lo + 16u * hi) * 64 + t * 32 + lane] = v;
            }
        }
    }

    // Everything above reads only weights.  x and y belong to the stream order.
    pdl_wait();
    const uint16_t *xrow = a.x + (size_t)bat * a.x_stride;
    float inv = 1.0f;
    if (a.norm_n) {
        // RMSNorm folded into the staging (rms_norm_inplace, src/lut/cpu_fallback.rs:39-54): every CTA sums
        // the squares of the whole row in a fixed order (the same value everywhere), then scales its slice
        const uint4 *xr = reinterpret_cast<const uint4 *>(xrow);
        float ss = 0.0f;
        for (uint32_t i = tid; i < a.norm_n / 8; i += CL_THREADS) {
            const uint4 v = xr[i];
            const __half2 *hp = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float2 f = __half22float2(hp[e]);
                ss += f.x * f.x + f.y * f.y;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        if (tid == 0) {
            float tot = 0.0f;
            for (int w = 0; w < CL_WARPS; w++) tot += red[w];
            s_inv = 1.0f / sqrtf(tot / (float)a.norm_n + a.norm_eps);
        }
        __syncthreads();
        inv = s_inv;
    }
    {
        const uint32_t n16 = span * 4;  // 16-byte units of this CTA's slice of x
        const uint4 *xg = reinterpret_cast<const uint4 *>(xrow + (size_t)cb * 32);
        uint4 *xd = reinterpret_cast<uint4 *>(xs);
        for (uint32_t i = tid; i < n16; i += CL_THREADS) {
            uint4 v = xg[i];
            if (a.norm_n) {
                __half2 *hp = reinterpret_cast<__half2 *>(&v);
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float2 f = __half22float2(hp[e]);
                    hp[e] = __floats2half2_rn(f.x * inv, f.y * inv);
                }
            }
            xd[i] = v;
        }
    }
    __syncthreads();  // table and x are in place

    // ---- lookups and tensor-core steps on the chunks held in registers --------------------------------
    const uint32_t lane_off = lane * 4;
    const uint32_t diag = ((lane >> 2) == (lane & 3)) ? 1u : 0u;  // lanes 0, 5, 10, 15 carry x in the B operand
    uint4 xb[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
    float acc[SK_NACC][4];
#pragma unroll
    for (int i = 0; i < SK_NACC; i++) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    const SkNoNext none;
#pragma unroll
    for (int j = 0; j < CL_PF; j++) {
        if ((uint32_t)j < nj)
            sk_chunk<SBASE, 0>(acc, q1[j], q2[j], xb, lane_off, (warp + j * CL_WARPS) * 64, diag, smem_base, none, false);
    }
    // accumulator column n = 2q, 2q+1 (q = lane%4) of MMA row g = lane/4 (and g+8): column n is the dot
    // product of the lane (g, n); only n < 4 is populated
    if ((lane & 3) < 2) {
        const uint32_t r = (lane >> 2) * 4 + (lane & 3) * 2;
        float *rw = red + warp * 64;
        rw[r] = acc[0][0] + acc[1][0];
        rw[r + 1] = acc[0][1] + acc[1][1];
        rw[32 + r] = acc[0][2] + acc[1][2];
        rw[32 + r + 1] = acc[0][3] + acc[1][3];
    }
    __syncthreads();
    float sum = 0.0f;  // thread tid < 64: rows "1" (tid < 32) or "2", lane tid & 31
    if (tid < 64) {
#pragma unroll
        for (int w = 0; w < CL_WARPS; w++) sum += red[w * 64 + tid];
    }
    if (s > 1) {
        // every CTA stores its 64 sums into slot [rank] of rank 0's shared memory; after one cluster barrier
        // rank 0 adds the slots in rank order from its own memory, and nobody reads a peer's memory after it
        asm volatile("barrier.cluster.wait.aligned;\n" ::: "memory");
        if (tid < 64) *cluster.map_shared_rank(cpush + rank * 64 + tid, 0) = sum;
        cluster.sync();
        if (rank == 0 && tid < 64) {
            sum = 0.0f;
            for (uint32_t r = 0; r < s; r++) sum += cpush[r * 64 + tid];  // rank order
        }
    }
    if (rank == 0) {
        if (MODE == GEMV_SWIGLU) {
            // rows "1" are gate rows, rows "2" the up rows of the same output index
            __syncthreads();
            if (tid < 64) red[tid] = sum;
            __syncthreads();
            if (tid < 32) {
                const uint32_t row = blk * 32 + tid;
                if (row < a.m) {
                    const float gv = __half2float(__float2half_rn(red[tid]));
                    const float uv = __half2float(__float2half_rn(red[32 + tid]));
                    const float sv = __half2float(__float2half_rn(gv / (1.0f + expf(-gv))));
                    a.y[(size_t)bat * a.y_stride + row] = __half_as_ushort(__float2half_rn(sv * uv));
                }
            }
        } else if (MODE == GEMV_TP) {
            if (tid < 64) {  // this CTA has only this block: deliver and finish at once
                const unsigned int e = tp_epoch(a.tp);
                const uint32_t hb = (tid >> 5) ? hb2 : hb1;
                uint16_t *lst = reinterpret_cast<uint16_t *>(&s_inv + 1) + (tid >> 5) * 2;  // spare words behind the norm factor
                tp_deliver(a.tp, e, hb, lane, sum);
                if (lane == 0 && !a.tp.deliver_only) lst[0] = (uint16_t)hb;
                __syncwarp();
                tp_finish(a.tp, e, lst, 1, lane, a.m, a.y + (size_t)bat * a.y_stride, a.err);
            }
        } else if (tid < 64) {
            const uint32_t row = ((tid >> 5) ? hb2 : hb1) * 32 + (tid & 31);
            if (MODE == GEMV_F32) {
                if (row < a.m) reinterpret_cast<float *>(a.y)[(size_t)bat * a.y_stride + row] = sum;
            } else if (row < a.m) {
                __half hv = __float2half_rn(sum);
                if (MODE == GEMV_RESID) {
                    const float r = __half2float(__ushort_as_half(a.resid[(size_t)bat * a.y_stride + row]));
                    hv = __float2half_rn(__half2float(hv) + r);
                }
                a.y[(size_t)bat * a.y_stride + row] = __half_as_ushort(hv);
            }
        }
    }
}

template <int MODE>
static int launch_cl(prism_cuda_ctx *ctx, const ClArgs &a, dim3 grid) {
    static bool configured[PRISM_MAX_DEVICES] = {false};
    if (!configured[ctx->device]) {
        PRISM_CUDA_TRY(ctx, cudaFuncSetAttribute(lut_gemv_cl_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)CL_SMEM_BYTES));
        configured[ctx->device] = true;
    }
    launch_cluster_pdl(ctx, lut_gemv_cl_kernel<MODE>, grid, dim3(CL_THREADS), CL_SMEM_BYTES, a.s, a);
    return after_launch(ctx, "lut_gemv_cl_kernel");
}

// CTAs per block for a matrix of n_blocks x n_chunks units, 0 when this kernel is not the one to use:
// the K part of a CTA must fit its registers (64 chunks), and the whole matrix must be small enough
// that one wave of CTAs holds it (otherwise the persistent kernels stream it better).
uint32_t cl_cluster_size(prism_cuda_ctx *ctx, const LutTensor &t, bool swiglu, uint32_t batch) {
    if (t.bits != 4 || t.k % 32 != 0 || t.k < 32 || batch == 0) return 0;
    const uint32_t n_blocks = swiglu ? t.n_hb : t.n_hb / 2, nc = t.n_chunks;
    if ((uint64_t)n_blocks * nc > (uint64_t)ctx->cl_max_units) return 0;
    uint32_t s = 1;
    while (s < 8 && (nc + s - 1) / s > (uint32_t)CL_MAX_CHUNKS) s *= 2;
    if ((nc + s - 1) / s > (uint32_t)CL_MAX_CHUNKS) return 0;
    // spread a block over more CTAs while they all stay in one wave and keep at least two chunks per warp pair
    // (measured on 896x4864: clusters of 8 take 1 us less per launch than clusters of 4 -- the cluster barrier
    // and the remote reads of the reduction cost less than the longer lookup loop)
    const uint32_t wave = (uint32_t)ctx->sm_count;
    while (s < 8 && n_blocks * batch * (s * 2) <= wave && nc / (s * 2) >= 4) s *= 2;
    if (n_blocks * s * batch > 3 * wave) return 0;
    return s;
}

int launch_gemv_cl(prism_cuda_ctx *ctx, GemvMode mode, const LutTensor &t, const LutTensor *t2, const uint16_t *x,
                   uint32_t x_stride, void *y, uint32_t y_stride, const uint16_t *resid, uint32_t batch, float norm_eps,
                   uint32_t s) {
    ClArgs a{};
    a.n_chunks = t.n_chunks;
    a.m = t.m;
    a.s = s;
    a.x = x; a.x_stride = x_stride; a.y = static_cast<uint16_t *>(y); a.y_stride = y_stride; a.resid = resid;
    a.err = ctx->dev_err;
    a.norm_n = norm_eps >= 0.0f ? t.k : 0;
    a.norm_eps = norm_eps >= 0.0f ? norm_eps : 0.0f;
    uint32_t n_blocks;
    if (mode == GEMV_SWIGLU) {
        a.idx1 = t.idx; a.pal1 = t.pal; a.idx2 = t2->idx; a.pal2 = t2->pal;
        a.hb_mul = 1; a.hb_add2 = 0;
        n_blocks = t.n_hb;
    } else {
        a.idx1 = a.idx2 = t.idx; a.pal1 = a.pal2 = t.pal;
        a.hb_mul = 2; a.hb_add2 = 1;
        n_blocks = t.n_hb / 2;
    }
    const dim3 grid(n_blocks * s, batch);
    switch (mode) {
    case GEMV_PLAIN: return launch_cl<GEMV_PLAIN>(ctx, a, grid);
    case GEMV_RESID: return launch_cl<GEMV_RESID>(ctx, a, grid);
    case GEMV_F32: return launch_cl<GEMV_F32>(ctx, a, grid);
    case GEMV_TP:
        PRISM_TRY(tp_fill_push(ctx, t, &a.tp));
        return launch_cl<GEMV_TP>(ctx, a, grid);
    default: return launch_cl<GEMV_SWIGLU>(ctx, a, grid);
    }
}

}  // namespace prism
