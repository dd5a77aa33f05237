// Palettized GEMV on the 5th-generation tensor cores: dequantised weights go to TMEM.
//
//   y[r] = f16( sum_k f32(x[k]) * f32(palette[r][idx[r,k]]) )      (lut_gemv_cpu,
//                                                    src/lut/cpu_fallback.rs:12-35)
//
// One persistent CTA per SM works on tiles of 128 output rows x one K slice (<= 4096):
//
//  * Dequantisation is the pair-table lookup of gemv.cu: every index byte (two weights) is
//    looked up in a 256-entry table of half2{pal[lo], pal[hi]}; the tables of the two rows a
//    lane works on live in that lane's own shared-memory bank (entry stride 256 B), so a
//    warp's 32 lookups never conflict, and the offset is one byte-permute of the index word.
//  * The looked-up half2 values are not multiplied in the thread at all: 16 of them (32
//    consecutive k of one row) are written with one tcgen05.st into the lane's own TMEM
//    lane, where they are the A operand (128 rows x 16 k per instruction) of
//    tcgen05.mma.kind::f16.  x is the B operand, read by the tensor core straight from
//    shared memory (K-major core matrices whose row 0 holds x, rows 1..7 zero), and the
//    fp32 accumulators stay in TMEM until a tile is finished.  Per 1 KB of index bytes a
//    warp issues 32 byte-permutes, 32 lookups, 2 global loads and 2 TMEM stores.
//  * Sixteen dequantising warps (four per TMEM lane quarter, one row per lane; quarters q and
//    q+2 share one 64 KB table area, as its two row slots) feed a ring of TMEM stages; one
//    thread of a seventeenth warp issues two MMAs per 128-row x 32-k chunk; mbarriers carry
//    the full/empty hand-offs.  Every wait is bounded: a wait that gives up sets an error word,
//    all later waits fall through, and the kernel still frees its TMEM and returns.
//
// Epilogues are those of gemv.cu (fp16 rounding points of the reference's step()).
#include <algorithm>
#include <cstdio>

#include "common.cuh"

namespace prism {

constexpr int T5_DEQ_WARPS = 16;             // dequant warps 0..15: quarter = warp % 4, slot in quarter = warp / 4
constexpr int T5_WARPS = T5_DEQ_WARPS + 1;   // warp 16 allocates TMEM and issues the MMAs
constexpr int T5_THREADS = T5_WARPS * 32;
constexpr int T5_TBL_BYTES = 2 * 65536;      // two lane quarters x (256 entries x 256 B)
constexpr int T5_KSLICE = 4096;              // k per CTA slice (x staged as 64 KB of core matrices)
constexpr int T5_XB_BYTES = T5_KSLICE / 8 * 128;
constexpr int T5_STAGES = 16;                // A stages of 16 TMEM columns (32 k of 128 rows)
constexpr int T5_GROUP = 1;                  // stages released by one tcgen05.commit
constexpr int T5_TMEM_COLS = 512;
constexpr int T5_NACC = 4;                   // independent accumulators per tile (MMAs into one are serialised)
constexpr int T5_D_COL = T5_STAGES * 16;     // accumulators: 2 buffers x T5_NACC x 16 columns
constexpr int T5_PF = 4;                     // index chunks in flight per warp
constexpr int T5_SBASE = 1024;               // dynamic shared memory offset in the shared window
constexpr uint32_t T5_SPIN_LIMIT = 64u << 20;
constexpr int T5_BAR_OFF = T5_TBL_BYTES + T5_XB_BYTES;  // barriers and small state
constexpr int T5_STATE_OFF = T5_BAR_OFF + 16 * T5_STAGES + 32;  // after full[S], empty[S], dfull[2], dempty[2]
constexpr size_t T5_SMEM_BYTES = T5_STATE_OFF + 64 + 512;       // state words, then 128 floats of epilogue exchange

struct Tc5Args {
    const uint8_t *idx1, *idx2;
    const uint16_t *pal1, *pal2;
    uint32_t n_chunks;          // chunks per row
    uint32_t n_hb1;             // half-blocks available in idx1 (and idx2)
    uint32_t mode;              // GemvMode
    uint32_t m;                 // valid output rows
    uint32_t n_tiles;           // row tiles (128 rows)
    uint32_t chunks_per_split, ksplit;
    const uint16_t *x;
    void *y;
    const uint16_t *resid;
    float *partials;            // [ksplit][n_tiles*128]
    unsigned int *counters;     // [n_tiles]
    unsigned int *err;
};


// ---- PTX wrappers ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t addr, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(addr), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t addr) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(addr) : "memory");
}
// Non-blocking probe: a blocking try_wait parks the thread for a coarse time slice when the phase
// is not complete yet, which serialised the stage ring.
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t addr, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    return ok;
}
// Bounded wait.  Gives up after T5_SPIN_LIMIT polls (or as soon as another thread gave up): the
// error flag in shared memory makes every later wait of the CTA fall through.
__device__ __forceinline__ void mbar_wait(uint32_t addr, uint32_t parity, volatile uint32_t *err_flag) {
    for (uint32_t i = 0; i < T5_SPIN_LIMIT; i++) {
        if (mbar_try_wait(addr, parity)) return;
        if ((i & 63) == 63 && *err_flag) return;
    }
    *err_flag = 1;
}
// Whole-warp wait: lane 0 polls (with a short back-off), the other lanes park at the warp barrier.
__device__ __forceinline__ void mbar_wait_warp(uint32_t addr, uint32_t parity, volatile uint32_t *err_flag) {
    if ((threadIdx.x & 31) == 0) {
        for (uint32_t i = 0; i < (16u << 20); i++) {
            if (mbar_try_wait(addr, parity)) break;
            if ((i & 63) == 63 && *err_flag) break;
            if (i + 1 == (16u << 20)) *err_flag = 1;
            __nanosleep(32);
        }
    }
    __syncwarp();
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t mbar_addr) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(mbar_addr) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem descriptor]; M = 128, N = 16, K = 16, fp16 in, fp32 accumulate.
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ uint32_t tc_ld1(uint32_t taddr) {
    uint32_t v;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];\n" : "=r"(v) : "r"(taddr) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t lds_tbl(uint32_t off, int imm_sel) {
    uint32_t v;
    if (imm_sel == 0) asm volatile("ld.shared.u32 %0, [%1+%2];\n" : "=r"(v) : "r"(off), "n"(T5_SBASE));
    else asm volatile("ld.shared.u32 %0, [%1+%2];\n" : "=r"(v) : "r"(off), "n"(T5_SBASE + 128));
    return v;
}
__device__ __forceinline__ uint4 ldg128_nc(const uint8_t *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// K-major, no-swizzle shared-memory descriptor of a 16(n) x 16(k) fp16 operand whose 8x8 core
// matrices (128 B, row r at +16r) for consecutive k follow each other (LBO = 128 B).  The second
// group of eight n rows re-reads the first (SBO = 0): accumulator columns 8..15 duplicate 0..7.
__device__ __forceinline__ uint64_t make_b_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(128u >> 4) << 16;   // leading-dimension byte offset: next core matrix along K
    d |= (uint64_t)0 << 32;             // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;             // descriptor version for sm_100
    return d;                           // layout type 0: no swizzle
}

__global__ void __launch_bounds__(T5_THREADS, 1) lut_gemv_tc5_kernel(const Tc5Args a) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
    if (smem_base != (uint32_t)T5_SBASE) {  // layout assumption broken: refuse to compute
        if (threadIdx.x == 0) atomicExch(a.err, 1u);
        return;
    }
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t bar_base = smem_base + T5_BAR_OFF;
    // barrier map (8 B each): full[S], empty[S], dfull[2], dempty[2]; then state words
    const uint32_t bar_full = bar_base, bar_empty = bar_base + 8 * T5_STAGES, bar_dfull = bar_base + 16 * T5_STAGES,
                   bar_dempty = bar_base + 16 * T5_STAGES + 16;
    volatile uint32_t *err_flag = reinterpret_cast<volatile uint32_t *>(smem + T5_STATE_OFF);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + T5_STATE_OFF + 8);

    const uint32_t ks = blockIdx.x % a.ksplit;
    const uint32_t tile0 = blockIdx.x / a.ksplit, tile_step = gridDim.x / a.ksplit;
    const uint32_t c_begin = ks * a.chunks_per_split;
    const uint32_t c_end = min(a.n_chunks, c_begin + a.chunks_per_split);
    const uint32_t nch = c_end - c_begin;

    // ---- set-up -----------------------------------------------------------------------------------
    if (tid == 0) {
        for (int s = 0; s < T5_STAGES; s++) {
            mbar_init(bar_full + 8 * s, 4);   // one arrival per lane quarter
            mbar_init(bar_empty + 8 * s, 1);  // tcgen05.commit
        }
        for (int d = 0; d < 2; d++) {
            mbar_init(bar_dfull + 8 * d, 1);
            mbar_init(bar_dempty + 8 * d, 4);
        }
        *err_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == T5_DEQ_WARPS) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                         smem_base + T5_STATE_OFF + 8),
                     "r"((uint32_t)T5_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    {   // x slice as B core matrices: block i (8 consecutive k) = 128 B, row 0 = x, rows 1..7 = 0
        uint4 *xb = reinterpret_cast<uint4 *>(smem + T5_TBL_BYTES);
        const uint4 z = make_uint4(0, 0, 0, 0);
        const uint32_t nblk = nch * 4;
        const uint4 *xg = reinterpret_cast<const uint4 *>(a.x + (size_t)c_begin * 32);
        for (uint32_t i = tid; i < nblk * 8; i += T5_THREADS) xb[i] = ((i & 7) == 0) ? xg[i >> 3] : z;
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < T5_DEQ_WARPS) {
        // =============================== dequantising warps ===============================
        const uint32_t q = warp & 3, j = warp >> 2;   // TMEM lane quarter, slot within the quarter
        const uint32_t pair = q & 1, slot = q >> 1;   // table area, row slot inside its entries
        const uint32_t laneq = (pair << 16) | (lane * 4);  // PRMT source: table area, this lane's bank
        const uint32_t tmem_lane = tmem_base + ((q * 32) << 16);
        float *ep = reinterpret_cast<float *>(smem + T5_STATE_OFF + 64);
        volatile uint32_t *s_last = reinterpret_cast<volatile uint32_t *>(smem + T5_STATE_OFF + 16);
        uint32_t n_base = 0;  // chunks of earlier tiles (position in the stage ring)
        uint32_t ti = 0;
        for (uint32_t tile = tile0; tile < a.n_tiles; tile += tile_step, ti++) {
            // the row of this lane
            const uint32_t hb = (a.mode == GEMV_SWIGLU) ? 2 * tile + pair : 4 * tile + q;
            const bool second = (a.mode == GEMV_SWIGLU) && slot == 1;  // quarters 2,3 read the up tensor
            const bool ok = hb < a.n_hb1;
            const uint32_t h = ok ? hb : a.n_hb1 - 1;
            // ---- index stream: start the first loads before building the table ----
            const uint8_t *sp = (second ? a.idx2 : a.idx1) + ((size_t)h * a.n_chunks + c_begin) * 512 + lane * 16;
            uint4 r[T5_PF];
#pragma unroll
            for (int i = 0; i < T5_PF; i++) {
                const uint32_t c = j + 4 * i;
                if (c < nch) r[i] = ldg128_nc(sp + (size_t)c * 512);
            }
            // ---- pair table of this row: warp j writes the entries whose high nibble is 4j..4j+3 ----
            asm volatile("bar.sync %0, 256;\n" ::"r"(1 + pair) : "memory");  // lookups of the previous tile are done
            {
                const uint16_t *prow = (second ? a.pal2 : a.pal1) + ((size_t)h * 32 + lane) * 16;
                const uint4 p0 = *reinterpret_cast<const uint4 *>(prow);
                const uint4 p1 = *reinterpret_cast<const uint4 *>(prow + 8);
                const uint32_t cbp[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
                const uint32_t hp0 = reinterpret_cast<const uint32_t *>(prow)[2 * j];      // pal[4j], pal[4j+1]
                const uint32_t hp1 = reinterpret_cast<const uint32_t *>(prow)[2 * j + 1];  // pal[4j+2], pal[4j+3]
                uint8_t *tb = smem + pair * 65536 + j * 16384 + lane * 4 + slot * 128;
#pragma unroll
                for (int lo = 0; lo < 16; lo++) {
#pragma unroll
                    for (int hs = 0; hs < 4; hs++) {
                        const uint32_t sel = (((hs & 1) ? 0x76u : 0x54u) << 8) | ((lo & 1) ? 0x32u : 0x10u);
                        const uint32_t v = __byte_perm(cbp[lo >> 1], (hs & 2) ? hp1 : hp0, sel);
                        // entry e = lo + 16*(4j + hs) sits at byte e*256 of the table area
                        *reinterpret_cast<uint32_t *>(tb + lo * 256 + hs * 4096) = v;
                    }
                }
            }
            asm volatile("bar.sync %0, 256;\n" ::"r"(1 + pair) : "memory");
            // ---- stream: lookups -> TMEM stage -> signal the MMA thread ----
            for (uint32_t c0 = j; c0 < nch; c0 += 4 * T5_PF) {
#pragma unroll
                for (int i = 0; i < T5_PF; i++) {
                    const uint32_t c = c0 + 4 * i;
                    if (c < nch) {
                        uint4 w;
                        w = r[i];
                        const uint32_t nc = c + 4 * T5_PF;
                        if (nc < nch) r[i] = ldg128_nc(sp + (size_t)nc * 512);
                        const uint32_t aw[4] = {w.x, w.y, w.z, w.w};
                        uint32_t A[16];
                        if (slot == 0) {
#pragma unroll
                            for (int hh = 0; hh < 4; hh++) {
                                // byte b of the word -> pair*65536 + (byte << 8) + lane*4
                                A[4 * hh + 0] = lds_tbl(__byte_perm(aw[hh], laneq, 0x7604), 0);
                                A[4 * hh + 1] = lds_tbl(__byte_perm(aw[hh], laneq, 0x7614), 0);
                                A[4 * hh + 2] = lds_tbl(__byte_perm(aw[hh], laneq, 0x7624), 0);
                                A[4 * hh + 3] = lds_tbl(__byte_perm(aw[hh], laneq, 0x7634), 0);
                            }
                        } else {
#pragma unroll
                            for (int hh = 0; hh < 4; hh++) {
                                A[4 * hh + 0] = lds_tbl(__byte_perm(aw[hh], laneq, 0x7604), 1);
                                A[4 * hh + 1] = lds_tbl(__byte_perm(aw[hh], laneq, 0x7614), 1);
                                A[4 * hh + 2] = lds_tbl(__byte_perm(aw[hh], laneq, 0x7624), 1);
                                A[4 * hh + 3] = lds_tbl(__byte_perm(aw[hh], laneq, 0x7634), 1);
                            }
                        }
                        const uint32_t n = n_base + c, stage = n % T5_STAGES, ph = (n / T5_STAGES) & 1;
                        mbar_wait_warp(bar_empty + 8 * (stage / T5_GROUP), ph ^ 1, err_flag);  // MMAs that read this stage group are done
                        tc_fence_after();
                        tc_st16(tmem_lane + stage * 16, A);
                        asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
                        tc_fence_before();
                        if (lane == 0) mbar_arrive(bar_full + 8 * stage);
                    }
                }
            }
            n_base += nch;
            if (j != 0) continue;
            // ---- epilogue (warps 0..3 = the 128 rows of the tile): accumulator column 0 ----
            const uint32_t d = ti & 1;
            const uint32_t te = q * 32 + lane;  // row inside the tile
            mbar_wait_warp(bar_dfull + 8 * d, (ti >> 1) & 1, err_flag);
            tc_fence_after();
            // consecutive MMAs went to T5_NACC accumulators in turn; add the ones that were used
            const uint32_t n_used = min((uint32_t)T5_NACC, 2 * nch);
            uint32_t accv[T5_NACC];
#pragma unroll
            for (int ai = 0; ai < T5_NACC; ai++)
                accv[ai] = (uint32_t)ai < n_used ? tc_ld1(tmem_lane + T5_D_COL + d * (T5_NACC * 16) + ai * 16) : 0u;
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            float sum = 0.0f;
#pragma unroll
            for (int ai = 0; ai < T5_NACC; ai++) sum += __uint_as_float(accv[ai]);
            tc_fence_before();
            if (lane == 0) mbar_arrive(bar_dempty + 8 * d);
            if (a.ksplit > 1) {
                // deterministic split-K: store the partials, the last CTA to arrive adds them in split order
                const size_t pslot = (size_t)tile * 128 + te;
                a.partials[(size_t)ks * a.n_tiles * 128 + pslot] = sum;
                __threadfence();
                asm volatile("bar.sync 3, 128;\n" ::: "memory");
                if (te == 0) {
                    unsigned int *ctr = a.counters + tile;
                    const uint32_t last = (atomicAdd(ctr, 1u) + 1 == a.ksplit) ? 1u : 0u;
                    if (last) *ctr = 0;  // ready for the next launch on this stream
                    *s_last = last;
                }
                asm volatile("bar.sync 3, 128;\n" ::: "memory");
                if (!*s_last) continue;
                __threadfence();
                sum = 0.0f;
                for (uint32_t sp2 = 0; sp2 < a.ksplit; sp2++)
                    sum += __ldcg(a.partials + (size_t)sp2 * a.n_tiles * 128 + pslot);
            }
            if (a.mode == GEMV_SWIGLU) {
                // quarters 0,1 hold gate rows, quarters 2,3 the up rows of the same output index
                asm volatile("bar.sync 3, 128;\n" ::: "memory");  // ep of the previous tile has been read
                ep[te] = sum;
                asm volatile("bar.sync 3, 128;\n" ::: "memory");
                if (te < 64) {
                    const uint32_t row = hb * 32 + lane;
                    if (ok && row < a.m) {
                        const float g = __half2float(__float2half_rn(ep[te]));
                        const float u = __half2float(__float2half_rn(ep[te + 64]));
                        const float sv = __half2float(__float2half_rn(g / (1.0f + expf(-g))));
                        reinterpret_cast<uint16_t *>(a.y)[row] = __half_as_ushort(__float2half_rn(sv * u));
                    }
                }
            } else {
                const uint32_t row = hb * 32 + lane;
                if (ok && row < a.m) {
                    if (a.mode == GEMV_F32) {
                        reinterpret_cast<float *>(a.y)[row] = sum;
                    } else {
                        __half hv = __float2half_rn(sum);
                        if (a.mode == GEMV_RESID)
                            hv = __float2half_rn(__half2float(hv) + __half2float(__ushort_as_half(a.resid[row])));
                        reinterpret_cast<uint16_t *>(a.y)[row] = __half_as_ushort(hv);
                    }
                }
            }
        }
    } else if (lane == 0) {
        // =============================== MMA issuing thread ===============================
        // instruction descriptor: D fp32, A/B fp16, both K-major, N = 16, M = 128
        const uint32_t idesc = (1u << 4) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
        const uint32_t xb_addr = smem_base + T5_TBL_BYTES;
        uint32_t n = 0, ti = 0;
        for (uint32_t tile = tile0; tile < a.n_tiles; tile += tile_step, ti++) {
            const uint32_t d = ti & 1;
            mbar_wait(bar_dempty + 8 * d, ((ti >> 1) & 1) ^ 1, err_flag);  // epilogue of tile ti-2 has read D
            tc_fence_after();
            const uint32_t dcol = tmem_base + T5_D_COL + d * (T5_NACC * 16);
            for (uint32_t c = 0; c < nch; c++, n++) {
                const uint32_t stage = n % T5_STAGES, ph = (n / T5_STAGES) & 1;
                mbar_wait(bar_full + 8 * stage, ph, err_flag);
                tc_fence_after();
                const uint32_t acol = tmem_base + stage * 16;
                const uint32_t m0 = 2 * c, m1 = 2 * c + 1;  // MMA number inside the tile
                tc_mma_ts(dcol + (m0 % T5_NACC) * 16, acol, make_b_desc(xb_addr + c * 512), idesc, m0 >= T5_NACC);
                tc_mma_ts(dcol + (m1 % T5_NACC) * 16, acol + 8, make_b_desc(xb_addr + c * 512 + 256), idesc, m1 >= T5_NACC);
                // one commit per group of stages: a tcgen05.commit costs several hundred cycles of the
                // tensor pipe's command stream, far more than the two small MMAs of a chunk
                if (stage % T5_GROUP == T5_GROUP - 1) tc_commit(bar_empty + 8 * (stage / T5_GROUP));
            }
            tc_commit(bar_dfull + 8 * d);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == T5_DEQ_WARPS) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)T5_TMEM_COLS) : "memory");
    }
    if (tid == 0 && *err_flag) atomicExch(a.err, 5u);
}

// ---- host side ---------------------------------------------------------------------------------

bool tc5_eligible(prism_cuda_ctx *ctx, const LutTensor &t, uint32_t batch) {
    return ctx->smem_base == T5_SBASE && t.bits == 4 && t.k % 32 == 0 && t.k >= 256 && batch == 1;
}

int launch_gemv_tc5(prism_cuda_ctx *ctx, GemvMode mode, const LutTensor &t, const LutTensor *t2, const uint16_t *x,
                    void *y, const uint16_t *resid) {
    static bool configured[PRISM_MAX_DEVICES] = {false};
    if (!configured[ctx->device]) {
        PRISM_CUDA_TRY(ctx, cudaFuncSetAttribute(lut_gemv_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)T5_SMEM_BYTES));
        configured[ctx->device] = true;
    }
    Tc5Args a{};
    a.n_chunks = t.n_chunks;
    a.n_hb1 = t.n_hb;
    a.mode = (uint32_t)mode;
    a.m = t.m;
    a.x = x; a.y = y; a.resid = resid; a.err = ctx->dev_err;
    if (mode == GEMV_SWIGLU) {
        a.idx1 = t.idx; a.pal1 = t.pal; a.idx2 = t2->idx; a.pal2 = t2->pal;
        a.n_tiles = t.n_hb / 2;
    } else {
        a.idx1 = a.idx2 = t.idx; a.pal1 = a.pal2 = t.pal;
        a.n_tiles = (t.n_hb + 3) / 4;
    }
    // K split: a slice of x must fit its staging area; beyond that pick the split with the best
    // estimated efficiency = (fill of the last wave of tiles) x (1 - table-build share of a slice)
    const uint32_t G = (uint32_t)ctx->sm_count;
    const uint32_t min_split = (t.n_chunks + T5_KSLICE / 32 - 1) / (T5_KSLICE / 32);
    uint32_t best = min_split;
    double best_eff = -1.0;
    for (uint32_t sp = min_split; sp <= 64 && t.n_chunks / sp >= 8; sp++) {
        const uint32_t cps = (t.n_chunks + sp - 1) / sp;
        const uint32_t real = (t.n_chunks + cps - 1) / cps;
        if (real != sp) continue;
        const uint64_t tiles = (uint64_t)a.n_tiles * sp;
        const uint32_t grid = (uint32_t)std::min<uint64_t>(tiles, G / sp * sp ? G / sp * sp : sp);
        const uint64_t waves = (tiles + grid - 1) / grid;
        const double fill = (double)tiles / (double)(waves * grid) * ((double)grid / G);
        const double build = 8.0 / (8.0 + cps);  // a table build costs about as much as 8 chunks of lookups
        const double eff = fill * (1.0 - build);
        if (eff > best_eff + 1e-9) { best_eff = eff; best = sp; }
    }
    const uint32_t ksplit0 = best;
    a.chunks_per_split = (t.n_chunks + ksplit0 - 1) / ksplit0;
    a.ksplit = (t.n_chunks + a.chunks_per_split - 1) / a.chunks_per_split;
    if (a.ksplit > 1) {
        PRISM_TRY(ensure_splitk(ctx, (size_t)a.ksplit * a.n_tiles * 128, (size_t)a.n_tiles));
        a.partials = ctx->splitk_partials;
        a.counters = ctx->splitk_counters;
    }
    uint32_t grid = G / a.ksplit * a.ksplit;
    if (grid == 0) grid = a.ksplit;
    const uint64_t tiles = (uint64_t)a.n_tiles * a.ksplit;
    if (grid > tiles) grid = (uint32_t)tiles;
    lut_gemv_tc5_kernel<<<grid, T5_THREADS, T5_SMEM_BYTES, ctx->stream>>>(a);
    return after_launch(ctx, "lut_gemv_tc5_kernel");
}

}  // namespace prism
