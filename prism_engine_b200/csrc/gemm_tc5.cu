// Prefill palettized GEMM on tcgen05 / TMEM:  Y[t][r] = f16( sum_k f32(X[t][k]) * f32(W[r][k]) )
// -- one lut_gemv_cpu per activation row (prefill_cpu, src/lut/engine_impl.rs:1046-1053; the
// reference's never-dispatched kernel for the same job is templates/palettized_gemm.metal:16-117).
//
// One persistent CTA per SM computes tiles of 128 weight rows x 256 tokens over the whole K:
//  * weights: 16 warps dequantise with the lane-private pair tables of gemv.cu / gemv_tc5.cu
//    (one row per lane = one TMEM lane) and store 32 k at a time into a ring of TMEM stages --
//    the A operand never touches shared memory;
//  * activations: X is re-laid once per call into 16-byte units [k/8][token][8] so that a
//    256-token x 32-k stage is four contiguous 4 KB runs, fetched by one thread with 1-D bulk
//    copies that complete on an mbarrier; in shared memory the runs are exactly the K-major,
//    no-swizzle core-matrix layout the B operand descriptor addresses;
//  * one thread issues two tcgen05.mma (M = 128, N = 256, K = 16) per 32-k chunk; the fp32
//    accumulators (256 TMEM columns) are read back with tcgen05.ld, rounded to fp16 and stored.
// 2-bit tensors (4-entry palettes; BITS = 2) run the same pipeline: a 16-byte index chunk then holds
// 64 weights of a row and expands into two 32-k chunks of the A operand through a 16-entry pair table
// indexed by nibbles (sk_expand2, pair_table.cuh).
// Every mbarrier wait is bounded; a wait that gives up raises the context's device error word.
#include <algorithm>

#include "common.cuh"
#include "pair_table.cuh"
#include "tc5_ptx.cuh"

namespace prism {

constexpr int GM_DEQ_WARPS = 16;
constexpr int GM_MMA_WARP = 16, GM_X_WARP = 17;
constexpr int GM_THREADS = 18 * 32;
constexpr int GM_NT_MAX = 256;                // largest token tile = N of the MMA (template parameter NT <= 256)
constexpr int GM_TBL_BYTES = 2 * 65536;
// A pipeline stage is CPS index chunks (32 k each): the hand-over between the dequantising warps,
// the MMA thread and the activation loader costs a few hundred cycles of single-thread control
// whatever the stage holds, so a weight stage is four chunks (the A operand occupies 256 TMEM
// columns, 16 per chunk); an activation stage is four chunks too, two for 256-token tiles.
constexpr int GM_SA = 8;                      // most A stages (two chunks each)
constexpr int GM_D_COL = 256;                 // accumulator: up to 256 columns after the A stages
constexpr int GM_X_BYTES = 6 * GM_NT_MAX * 32 * 2;   // activation staging area: 96 KB (three 32 KB stages at 128- and 256-token tiles)
constexpr int GM_SX_MAX = 32;                 // most X stages (small token tiles): a stage is NT tokens x 32 k fp16 = NT*64 bytes
// X stages for a token tile of NT: as many as fit the staging area, at most GM_SX_MAX.  Small tiles
// need the depth: a stage is refilled by a bulk copy whose latency is the same whatever its size.
template <int NT>
struct GmX {
    static constexpr int CPS = 4;                             // chunks per A (weight) stage
    static constexpr int XC = NT <= 128 ? 4 : 2;              // chunks per X (activation) stage: at most 32 KB
    static constexpr int SA = GM_D_COL / (16 * CPS);          // A stages: 4
    static constexpr int STAGE_BYTES = NT * 64 * XC;
    static constexpr int SX = (GM_X_BYTES / STAGE_BYTES) < GM_SX_MAX ? (GM_X_BYTES / STAGE_BYTES) : GM_SX_MAX;
};
constexpr int GM_TMEM_COLS = 512;
constexpr int GM_PF = 4;
constexpr int GM_SBASE = 1024;
constexpr int GM_X_OFF = GM_TBL_BYTES;
constexpr int GM_BAR_OFF = GM_X_OFF + GM_X_BYTES;
// barriers (8 B each): afull[SA], aempty[SA], xfull[SX], xempty[SX], dfull, dempty
constexpr int GM_STATE_OFF = GM_BAR_OFF + 8 * (2 * GM_SA + 2 * GM_SX_MAX + 2);
constexpr size_t GM_SMEM_BYTES = GM_STATE_OFF + 64;

struct GemmArgs {
    const uint8_t *idx;
    const uint16_t *pal;
    uint32_t n_chunks, n_hb, m;       // 32-k chunks per row (K/32), half-blocks, valid weight rows
    uint32_t n_ichunks;               // 16-byte index chunks per row (K/32 at 4 bit, K/64 at 2 bit)
    uint32_t n_rt, n_tt;              // row tiles (128 rows), token tiles (256 tokens)
    uint32_t m_tok, m_tok_pad;
    const uint8_t *xc;                // [token tile][K/8][NT][16 B]
    uint16_t *y;                      // [m_tok][m]
    unsigned int *err;
};

// X [m_tok][k] fp16 -> Xc [token tile][k/8][nt][8]: the 32 k of one chunk for the nt tokens of one
// tile are one contiguous run of nt*64 bytes, already in the order the shared-memory B operand
// wants (k-blocks of 8, then tokens), so a stage is filled by ONE bulk copy.  Padded token rows are
// zero.
__global__ void gemm_relay_x_kernel(const uint16_t *__restrict__ x, uint32_t m_tok, uint32_t m_tok_pad, uint32_t k,
                                    uint32_t nt, uint4 *__restrict__ xc) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // index into the output
    const size_t k8n = k / 8;
    if (i >= k8n * m_tok_pad) return;
    const uint32_t tin = (uint32_t)(i % nt);
    const size_t rest = i / nt;
    const uint32_t k8 = (uint32_t)(rest % k8n), tt = (uint32_t)(rest / k8n);
    const uint32_t t = tt * nt + tin;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (t < m_tok) v = *reinterpret_cast<const uint4 *>(x + (size_t)t * k + (size_t)k8 * 8);
    xc[i] = v;
}

__device__ __forceinline__ uint32_t gm_lds(uint32_t off, int slot) {
    uint32_t v;
    if (slot == 0) asm volatile("ld.shared.u32 %0, [%1+%2];\n" : "=r"(v) : "r"(off), "n"(GM_SBASE));
    else asm volatile("ld.shared.u32 %0, [%1+%2];\n" : "=r"(v) : "r"(off), "n"(GM_SBASE + 128));
    return v;
}

// The 16 table lookups of one 32-k chunk of a row: bytes of the index words -> half2 entries.
__device__ __forceinline__ void gm_lookup16(uint32_t (&A)[16], const uint4 &wv, uint32_t laneq, uint32_t slot) {
    const uint32_t aw[4] = {wv.x, wv.y, wv.z, wv.w};
    if (slot == 0) {
#pragma unroll
        for (int hh = 0; hh < 4; hh++) {
            A[4 * hh + 0] = gm_lds(__byte_perm(aw[hh], laneq, 0x7604), 0);
            A[4 * hh + 1] = gm_lds(__byte_perm(aw[hh], laneq, 0x7614), 0);
            A[4 * hh + 2] = gm_lds(__byte_perm(aw[hh], laneq, 0x7624), 0);
            A[4 * hh + 3] = gm_lds(__byte_perm(aw[hh], laneq, 0x7634), 0);
        }
    } else {
#pragma unroll
        for (int hh = 0; hh < 4; hh++) {
            A[4 * hh + 0] = gm_lds(__byte_perm(aw[hh], laneq, 0x7604), 1);
            A[4 * hh + 1] = gm_lds(__byte_perm(aw[hh], laneq, 0x7614), 1);
            A[4 * hh + 2] = gm_lds(__byte_perm(aw[hh], laneq, 0x7624), 1);
            A[4 * hh + 3] = gm_lds(__byte_perm(aw[hh], laneq, 0x7634), 1);
        }
    }
}

template <int NT, int BITS>
__global__ void __launch_bounds__(GM_THREADS, 1) lut_gemm_tc5_kernel(const GemmArgs a) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
    if (smem_base != (uint32_t)GM_SBASE) {  // layout assumption broken: refuse to compute
        if (threadIdx.x == 0) atomicExch(a.err, 1u);
        return;
    }
    // Tables, barriers and TMEM are set up from weights alone while the previous kernel drains; the
    // loader thread waits for it before the first activation copy, and everything that reads or
    // writes activations (MMAs, epilogue) follows that copy through the mbarriers.
    pdl_launch_dependents();
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t bar = smem_base + GM_BAR_OFF;
    const uint32_t b_afull = bar, b_aempty = bar + 8 * GM_SA, b_xfull = bar + 16 * GM_SA,
                   b_xempty = b_xfull + 8 * GM_SX_MAX, b_dfull = b_xempty + 8 * GM_SX_MAX, b_dempty = b_dfull + 8;
    constexpr int SX = GmX<NT>::SX, XSTAGE = GmX<NT>::STAGE_BYTES, CPS = GmX<NT>::CPS, SA = GmX<NT>::SA, XC = GmX<NT>::XC;
    constexpr int ICPS = BITS == 4 ? CPS : CPS / 2;  // 16-byte index chunks per weight stage
    constexpr int NSI = GM_PF / ICPS;                // stages whose index chunks a warp keeps in flight
    volatile uint32_t *err_flag = reinterpret_cast<volatile uint32_t *>(smem + GM_STATE_OFF);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + GM_STATE_OFF + 8);
    const uint32_t nch = a.n_chunks;
    const uint32_t n_items = a.n_rt * a.n_tt;  // item w: row tile w % n_rt, token tile w / n_rt

    if (tid == 0) {
        for (int s = 0; s < SA; s++) { t5::mbar_init(b_afull + 8 * s, 4); t5::mbar_init(b_aempty + 8 * s, 1); }
        for (int s = 0; s < SX; s++) { t5::mbar_init(b_xfull + 8 * s, 1); t5::mbar_init(b_xempty + 8 * s, 1); }
        t5::mbar_init(b_dfull, 1);
        t5::mbar_init(b_dempty, GM_DEQ_WARPS);
        *err_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == GM_MMA_WARP) t5::tmem_alloc(smem_base + GM_STATE_OFF + 8, GM_TMEM_COLS);
    t5::fence_before();
    __syncthreads();
    t5::fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < GM_DEQ_WARPS) {
        // =============================== dequantising warps ===============================
        const uint32_t q = warp & 3, j = warp >> 2;      // TMEM lane quarter, slot within the quarter
        const uint32_t pair = q & 1, slot = q >> 1;      // table area, row slot inside its entries
        const uint32_t laneq = (pair << 16) | (lane * 4);
        const uint32_t tmem_lane = tmem_base + ((q * 32) << 16);
        uint32_t n_base = 0, ti = 0, cur_rt = 0xFFFFFFFFu;
        for (uint32_t w = blockIdx.x; w < n_items; w += gridDim.x, ti++) {
            const uint32_t rt = w % a.n_rt, tt = w / a.n_rt;
            const uint32_t hb = 4 * rt + q;
            const bool ok = hb < a.n_hb;
            const uint32_t h = ok ? hb : a.n_hb - 1;
            const uint32_t nich = a.n_ichunks;
            const uint8_t *sp = a.idx + (size_t)h * nich * 512 + lane * 16;
            uint4 r[GM_PF];
#pragma unroll
            for (int i = 0; i < GM_PF; i++) {  // r[i]: index chunk (i % ICPS) of this warp's stage number i / ICPS
                const uint32_t c = (j + 4 * (i / ICPS)) * ICPS + (i % ICPS);
                if (c < nich) r[i] = t5::ldg128_nc(sp + (size_t)c * 512);
            }
            if (rt != cur_rt) {  // same decision in all warps: they walk the same item list
                cur_rt = rt;
                asm volatile("bar.sync %0, 256;\n" ::"r"(1 + pair) : "memory");  // lookups of the previous tile are done
                if (BITS == 4) {
                    const uint16_t *prow = a.pal + ((size_t)h * 32 + lane) * 16;
                    const uint4 p0 = *reinterpret_cast<const uint4 *>(prow);
                    const uint4 p1 = *reinterpret_cast<const uint4 *>(prow + 8);
                    const uint32_t cbp[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
                    const uint32_t hp0 = reinterpret_cast<const uint32_t *>(prow)[2 * j];
                    const uint32_t hp1 = reinterpret_cast<const uint32_t *>(prow)[2 * j + 1];
                    uint8_t *tb = smem + pair * 65536 + j * 16384 + lane * 4 + slot * 128;
#pragma unroll
                    for (int lo = 0; lo < 16; lo++) {
#pragma unroll
                        for (int hs = 0; hs < 4; hs++) {
                            const uint32_t sel = (((hs & 1) ? 0x76u : 0x54u) << 8) | ((lo & 1) ? 0x32u : 0x10u);
                            *reinterpret_cast<uint32_t *>(tb + lo * 256 + hs * 4096) =
                                __byte_perm(cbp[lo >> 1], (hs & 2) ? hp1 : hp0, sel);
                        }
                    }
                } else {
                    // 16-entry nibble table: entry e = i0 | i1 << 2 -> half2{pal[i0], pal[i1]}; slot j writes e = 4j..4j+3
                    const uint2 pp = *reinterpret_cast<const uint2 *>(a.pal + ((size_t)h * 32 + lane) * 4);
                    const uint32_t v1 = ((j & 2) ? pp.y : pp.x) >> ((j & 1) * 16) & 0xFFFFu;  // pal[i1], i1 = j
                    uint8_t *tb = smem + pair * 65536 + lane * 4 + slot * 128;
#pragma unroll
                    for (uint32_t i0 = 0; i0 < 4; i0++) {
                        const uint32_t v0 = ((i0 & 2) ? pp.y : pp.x) >> ((i0 & 1) * 16) & 0xFFFFu;
                        *reinterpret_cast<uint32_t *>(tb + (4 * j + i0) * 256) = v0 | (v1 << 16);
                    }
                }
                asm volatile("bar.sync %0, 256;\n" ::"r"(1 + pair) : "memory");
            }
            // Everything so far read weights only.  The waits below depend on the activations, which come after the
            // loader's dependency wait: wait for the same dependency first, so that no bounded wait runs while the
            // kernel before this one (under tensor parallelism: a late peer) is still at work.
            if (w == blockIdx.x) pdl_wait();
            // ---- K loop: lookups -> TMEM stage -> signal the MMA thread ----
            // a stage is CPS consecutive chunks; warp slot j takes the stages j, j+4, ...
            const uint32_t nst = nch / CPS;
            for (uint32_t s0 = j; s0 < nst; s0 += 4 * NSI) {
#pragma unroll
                for (int i = 0; i < NSI; i++) {
                    const uint32_t su = s0 + 4 * i;
                    if (su < nst) {
                        uint32_t A[CPS][16];
#pragma unroll
                        for (int cc = 0; cc < ICPS; cc++) {
                            const uint32_t c = su * ICPS + cc;
                            const uint4 wv = r[i * ICPS + cc];
                            const uint32_t nc = c + 4 * GM_PF;
                            if (nc < nich) r[i * ICPS + cc] = t5::ldg128_nc(sp + (size_t)nc * 512);
                            if (BITS == 4) {
                                gm_lookup16(A[cc], wv, laneq, slot);
                            } else {
                                uint4 pa, pb;
                                sk_expand2(pa, pb, wv);
                                gm_lookup16(A[2 * cc], pa, laneq, slot);
                                gm_lookup16(A[2 * cc + 1], pb, laneq, slot);
                            }
                        }
                        const uint32_t n = n_base + su, stage = n % SA, ph = (n / SA) & 1;
                        t5::mbar_wait_warp(b_aempty + 8 * stage, ph ^ 1, err_flag);
                        t5::fence_after();
#pragma unroll
                        for (int cc = 0; cc < CPS; cc++) t5::st16(tmem_lane + stage * 16 * CPS + cc * 16, A[cc]);
                        t5::wait_st();
                        t5::fence_before();
                        if (lane == 0) t5::mbar_arrive(b_afull + 8 * stage);
                    }
                }
            }
            n_base += nst;
            // ---- epilogue: warp (q, j) converts token columns [64j, 64j+64) of its 32 rows ----
            t5::mbar_wait_warp(b_dfull, ti & 1, err_flag);
            t5::fence_after();
            const uint32_t row = hb * 32 + lane;
            const bool row_ok = ok && row < a.m;
            constexpr int CW = NT / 4 > 16 ? NT / 4 : 16;  // accumulator columns (tokens) per warp of a quarter
            if ((int)j * CW < NT) {
#pragma unroll 1
                for (int g = 0; g < CW / 16; g++) {
                    uint32_t v[16];
                    t5::ld16(tmem_lane + GM_D_COL + j * CW + g * 16, v);
                    t5::wait_ld();
                    const uint32_t t0 = tt * NT + j * CW + g * 16;
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        const uint32_t t = t0 + i;
                        if (row_ok && t < a.m_tok)
                            a.y[(size_t)t * a.m + row] = __half_as_ushort(__float2half_rn(__uint_as_float(v[i])));
                    }
                }
            }
            t5::fence_before();
            if (lane == 0) t5::mbar_arrive(b_dempty);
        }
    } else if (warp == GM_MMA_WARP && lane == 0) {
        // =============================== MMA issuing thread ===============================
        const uint32_t idesc = t5::idesc_f16(128, NT);
        const uint32_t x_addr = smem_base + GM_X_OFF;
        uint32_t n = 0, nx = 0, ti = 0;
        pdl_wait();  // see the dequantising warps: no bounded wait before the dependency is met
        for (uint32_t w = blockIdx.x; w < n_items; w += gridDim.x, ti++) {
            t5::mbar_wait_bounded(b_dempty, (ti & 1) ^ 1, err_flag);  // epilogue of the previous tile has read D
            t5::fence_after();
            const uint32_t dcol = tmem_base + GM_D_COL;
            for (uint32_t su = 0; su < nch / CPS; su++, n++) {
                const uint32_t sa = n % SA, pa = (n / SA) & 1;
                t5::mbar_wait_bounded(b_afull + 8 * sa, pa, err_flag);
                const uint32_t acol = tmem_base + sa * 16 * CPS;
#pragma unroll
                for (int xi = 0; xi < CPS / XC; xi++, nx++) {
                    const uint32_t sx = nx % SX, px = (nx / SX) & 1;
                    t5::mbar_wait_bounded(b_xfull + 8 * sx, px, err_flag);
                    t5::fence_after();
                    const uint32_t xs = x_addr + sx * XSTAGE;
                    // B: NT tokens x 16 k; core matrices of 8 tokens are 128 B apart, k-blocks of 8 are NT*16 B apart
#pragma unroll
                    for (int cc = 0; cc < XC; cc++) {
                        const uint32_t ac = acol + (xi * XC + cc) * 16;
                        t5::mma_ts(dcol, ac, t5::smem_desc(xs + cc * NT * 64, NT * 16, 128), idesc, (su | xi | cc) != 0);
                        t5::mma_ts(dcol, ac + 8, t5::smem_desc(xs + cc * NT * 64 + 2 * NT * 16, NT * 16, 128), idesc, 1);
                    }
                    t5::commit(b_xempty + 8 * sx);
                }
                t5::commit(b_aempty + 8 * sa);
            }
            t5::commit(b_dfull);
        }
    } else if (warp == GM_X_WARP && lane == 0) {
        // =============================== activation loader ===============================
        const uint32_t x_addr = smem_base + GM_X_OFF;
        uint32_t n = 0;
        pdl_wait();
        for (uint32_t w = blockIdx.x; w < n_items; w += gridDim.x) {
            const uint32_t tt = w / a.n_rt;
            const uint8_t *src0 = a.xc + (size_t)tt * nch * NT * 64;
            for (uint32_t su = 0; su < nch / XC; su++, n++) {
                const uint32_t sx = n % SX, px = (n / SX) & 1;
                t5::mbar_wait_bounded(b_xempty + 8 * sx, px ^ 1, err_flag);
                t5::mbar_arrive_expect_tx(b_xfull + 8 * sx, XSTAGE);
                t5::bulk_g2s(x_addr + sx * XSTAGE, src0 + (size_t)su * XSTAGE, XSTAGE, b_xfull + 8 * sx);
            }
        }
    }
    t5::fence_before();
    __syncthreads();
    if (warp == GM_MMA_WARP) t5::tmem_dealloc(tmem_base, GM_TMEM_COLS);
    if (tid == 0 && *err_flag) atomicExch(a.err, 5u);
}

// ---- host side ---------------------------------------------------------------------------------

bool gemm_tc5_eligible(prism_cuda_ctx *ctx, const LutTensor &t, uint32_t m_tok) {
    // whole weight stages of 128 k (four 32-k chunks: four index chunks at 4 bit, two at 2 bit)
    return ctx->smem_base == GM_SBASE && (t.bits == 4 || t.bits == 2) && t.k % 128 == 0 && m_tok >= 8;
}

template <int NT, int BITS>
static int launch_gemm_nt(prism_cuda_ctx *ctx, GemmArgs &a, const LutTensor &t, const uint16_t *X) {
    static bool configured[PRISM_MAX_DEVICES] = {false};
    if (!configured[ctx->device]) {
        PRISM_CUDA_TRY(ctx, cudaFuncSetAttribute(lut_gemm_tc5_kernel<NT, BITS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)GM_SMEM_BYTES));
        configured[ctx->device] = true;
    }
    a.m_tok_pad = round_up_u32(a.m_tok, NT);
    a.n_tt = a.m_tok_pad / NT;
    // X -> [token tile][k/8][NT][8] (context scratch)
    const size_t xc_halfs = (size_t)t.k * a.m_tok_pad;
    PRISM_TRY(ensure_tmp(ctx, xc_halfs));
    const size_t units = xc_halfs / 8;
    if (!ctx->gemm_reuse_x) {
        launch_pdl(ctx, "gemm_relay_x_kernel", gemm_relay_x_kernel, dim3((unsigned)((units + 255) / 256)), dim3(256), 0, X, a.m_tok,
                   a.m_tok_pad, t.k, (uint32_t)NT, reinterpret_cast<uint4 *>(ctx->tmp_scratch));
        PRISM_TRY(after_launch(ctx, "gemm_relay_x_kernel"));
    }
    a.xc = reinterpret_cast<const uint8_t *>(ctx->tmp_scratch);
    // one row tile per CTA when possible, so its tables are built once
    const uint32_t G = (uint32_t)ctx->sm_count;
    uint32_t grid;
    if (a.n_rt <= G) grid = a.n_rt * std::max(1u, std::min(G / a.n_rt, a.n_tt));
    else grid = G;
    launch_pdl(ctx, "lut_gemm_tc5_kernel", lut_gemm_tc5_kernel<NT, BITS>, dim3(grid), dim3(GM_THREADS), GM_SMEM_BYTES, a);
    return after_launch(ctx, "lut_gemm_tc5_kernel");
}

int launch_gemm_tc5(prism_cuda_ctx *ctx, const LutTensor &t, const uint16_t *X, uint32_t m_tok, uint16_t *Y) {
    if (reinterpret_cast<uintptr_t>(X) & 15) return fail(ctx, PRISM_E_ARG, "gemm: X must be 16-byte aligned");
    GemmArgs a{};
    a.idx = t.idx; a.pal = t.pal;
    a.n_chunks = t.k / 32; a.n_ichunks = t.n_chunks; a.n_hb = t.n_hb; a.m = t.m;
    a.n_rt = (t.n_hb + 3) / 4;
    a.m_tok = m_tok;
    a.y = Y; a.err = ctx->dev_err;
    // token tile = N of the MMA: as small as the batch allows (the activation tile is the operand
    // that has to come through L2 for every 32-k chunk)
    if (t.bits == 2) {
        if (m_tok <= 32) return launch_gemm_nt<32, 2>(ctx, a, t, X);
        if (m_tok <= 64) return launch_gemm_nt<64, 2>(ctx, a, t, X);
        if (m_tok <= 128) return launch_gemm_nt<128, 2>(ctx, a, t, X);
        return launch_gemm_nt<256, 2>(ctx, a, t, X);
    }
    if (m_tok <= 32) return launch_gemm_nt<32, 4>(ctx, a, t, X);
    if (m_tok <= 64) return launch_gemm_nt<64, 4>(ctx, a, t, X);
    if (m_tok <= 128) return launch_gemm_nt<128, 4>(ctx, a, t, X);
    return launch_gemm_nt<256, 4>(ctx, a, t, X);
}

}  // namespace prism
