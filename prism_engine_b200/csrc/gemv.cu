// Palettized GEMV kernels for sm_100a.
//
//   y[r] = f16( sum_k f32(x[k]) * f32(palette[r][idx[r,k]]) )      (fp32 accumulate)
//
// the sum of lut_gemv_cpu (src/lut/cpu_fallback.rs:12-35).  Two kernels:
//
//  * lut_gemv_simple_kernel: one lane per output row, palette in shared
//    memory, CUDA-core FMAs.  Handles 2- and 4-bit palettes and any K with
//    K*bits % 32 == 0.  The plain, easy-to-audit path.
//
//  * lut_gemv_mma_kernel (4-bit): the bandwidth kernel.  A weight costs half a
//    shared-memory lookup and half an integer instruction:
//      - every index BYTE (two weights) is looked up in a 256-entry table of
//        half2 {palette[lo nibble], palette[hi nibble]} built per row;
//      - the table of the row a lane works on lives entirely in that lane's own
//        shared-memory bank (entry stride 256 B), so the 32 lookups of a warp
//        never conflict whatever the indices are;
//      - the looked-up half2 is directly a register of the A fragment of
//        mma.sync.m16n8k16: each lane feeds two rows x four k.  The B fragment
//        holds x only on the four "diagonal" lanes (column n = lane%4), so
//        column n of the accumulator collects exactly the products of the
//        lanes with lane%4 == n.  The tensor pipe does the fp32 multiply-
//        accumulate; no cvt/FMA instructions are spent per weight.
//    Epilogues fuse the fp16 rounding points of the reference's step():
//    residual add (engine_impl.rs:1158-1162,1196-1203) and gate/up SwiGLU
//    (engine_impl.rs:1163-1195,1349-1367).
#include "common.cuh"

namespace prism {

// ---------------------------------------------------------------------------
// Simple kernel
// ---------------------------------------------------------------------------
constexpr int SIMPLE_WARPS = 4;

template <int BITS>
__global__ void __launch_bounds__(SIMPLE_WARPS * 32)
lut_gemv_simple_kernel(const uint8_t *__restrict__ idx, const uint16_t *__restrict__ pal, uint32_t m,
                       uint32_t k, uint32_t n_chunks, const uint16_t *__restrict__ x, uint32_t x_stride,
                       uint16_t *__restrict__ y, uint32_t y_stride) {
    constexpr uint32_t NE = 1u << BITS, PER_WORD = 32 / BITS, MASK = NE - 1;
    __shared__ float pal_s[NE * 32];               // [entry][lane]: lane-private bank
    __shared__ float red[SIMPLE_WARPS * 32];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t hb = blockIdx.x, b = blockIdx.y;
    const uint32_t row = hb * 32 + lane;
    if (warp == 0) {
#pragma unroll
        for (uint32_t e = 0; e < NE; e++)
            pal_s[e * 32 + lane] = __half2float(__ushort_as_half(pal[(size_t)row * NE + e]));
    }
    __syncthreads();
    const uint16_t *xb = x + (size_t)b * x_stride;
    float acc = 0.0f;
    for (uint32_t c = warp; c < n_chunks; c += SIMPLE_WARPS) {
        uint4 v = *reinterpret_cast<const uint4 *>(idx + lut_idx_offset(n_chunks, hb, c, lane));
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t k0 = c * (128 / BITS);
#pragma unroll
        for (uint32_t wi = 0; wi < 4; wi++) {
            uint32_t kw = k0 + wi * PER_WORD;
            if (kw < k) {  // K*BITS % 32 == 0, so a word is entirely inside or outside
#pragma unroll
                for (uint32_t j = 0; j < PER_WORD; j++) {
                    float xv = __half2float(__ushort_as_half(__ldg(xb + kw + j)));
                    acc = fmaf(xv, pal_s[((w[wi] >> (j * BITS)) & MASK) * 32 + lane], acc);
                }
            }
        }
    }
    red[warp * 32 + lane] = acc;
    __syncthreads();
    if (warp == 0 && row < m) {
        float s = 0.0f;
#pragma unroll
        for (int wv = 0; wv < SIMPLE_WARPS; wv++) s += red[wv * 32 + lane];
        y[(size_t)b * y_stride + row] = __half_as_ushort(__float2half_rn(s));
    }
}

// ---------------------------------------------------------------------------
// Pair-table tensor-core kernel
// ---------------------------------------------------------------------------
constexpr int MMA_WARPS = 8;
constexpr int MMA_THREADS = MMA_WARPS * 32;
constexpr int MMA_TBL_BYTES = 256 * 256;  // 256 entries x (2 rows x 32 lanes x 4 B)
constexpr int MMA_MAX_KSLICE = 4096;      // halves of x staged per CTA
constexpr int MMA_PF = 4;                 // index chunks in flight per warp

struct MmaGemvArgs {
    const uint8_t *idx1, *idx2;   // index arrays the two half-blocks of a CTA come from
    const uint16_t *pal1, *pal2;
    uint32_t n_chunks;            // chunks per row
    uint32_t hb_mul, hb_add2;     // CTA b reads half-blocks hb_mul*b (rows "1") and hb_mul*b+hb_add2 ("2")
    uint32_t m;                   // valid output rows (per tensor)
    uint32_t chunks_per_split, ksplit;
    const uint16_t *x; uint32_t x_stride;
    uint16_t *y; uint32_t y_stride;
    const uint16_t *resid;
    float *partials;              // [batch][ksplit][n_blocks*64]
    unsigned int *counters;       // [batch][n_blocks]
    unsigned int *err;            // device error word (set when a layout assumption does not hold)
    uint32_t norm_n;              // > 0: x is an un-normalised row of norm_n values; stage rms_norm(x) instead
    float norm_eps;
};

__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                             uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg128_stream(const uint8_t *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Shared-memory loads whose address is `register + immediate`.  SBASE is the offset of the
// kernel's dynamic shared memory inside the shared window when it is known at compile time
// (probed once per context): the table base then rides in the instruction's immediate field and a
// lookup needs no address arithmetic beyond the byte-permute that forms the offset.  SBASE < 0
// is the portable variant (base added at run time).
template <int SBASE, int IMM>
__device__ __forceinline__ uint32_t lds_u32(uint32_t off, uint32_t base) {
    uint32_t v;
    if (SBASE >= 0) asm volatile("ld.shared.u32 %0, [%1+%2];\n" : "=r"(v) : "r"(off), "n"(SBASE >= 0 ? SBASE + IMM : 0));
    else asm volatile("ld.shared.u32 %0, [%1+%2];\n" : "=r"(v) : "r"(off + base), "n"(IMM));
    return v;
}
template <int SBASE, int IMM>
__device__ __forceinline__ uint4 lds_u128(uint32_t off, uint32_t base) {
    uint4 v;
    if (SBASE >= 0)
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                     : "r"(off), "n"(SBASE >= 0 ? SBASE + IMM : 0));
    else
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                     : "r"(off + base), "n"(IMM));
    return v;
}

// The eight table lookups of one 32-bit index word per row (= two tensor-core steps).
// byte j of the word -> (byte << 8) | lane*4: offset of table entry `byte` in this lane's bank.
template <int SBASE>
__device__ __forceinline__ void lookup_word(uint32_t (&A)[8], uint32_t w1, uint32_t w2, uint32_t lane_off,
                                            uint32_t base) {
    const uint32_t o10 = __byte_perm(w1, lane_off, 0x7704), o11 = __byte_perm(w1, lane_off, 0x7714);
    const uint32_t o12 = __byte_perm(w1, lane_off, 0x7724), o13 = __byte_perm(w1, lane_off, 0x7734);
    const uint32_t o20 = __byte_perm(w2, lane_off, 0x7704), o21 = __byte_perm(w2, lane_off, 0x7714);
    const uint32_t o22 = __byte_perm(w2, lane_off, 0x7724), o23 = __byte_perm(w2, lane_off, 0x7734);
    A[0] = lds_u32<SBASE, 0>(o10, base);   A[1] = lds_u32<SBASE, 128>(o20, base);
    A[2] = lds_u32<SBASE, 0>(o11, base);   A[3] = lds_u32<SBASE, 128>(o21, base);
    A[4] = lds_u32<SBASE, 0>(o12, base);   A[5] = lds_u32<SBASE, 128>(o22, base);
    A[6] = lds_u32<SBASE, 0>(o13, base);   A[7] = lds_u32<SBASE, 128>(o23, base);
}

// One 32-weight chunk of two rows: 8 tensor-core steps of 4 k each.  x_off is the byte offset of
// the chunk's 64 bytes of x inside the staged slice.  Every lane reads the same x words (a
// broadcast); `dmask` keeps them only on the diagonal lanes.  Lookups of word h+1 are issued
// before the tensor-core steps of word h.
template <int SBASE>
__device__ __forceinline__ void mma_chunk(float (&acc)[2][4], const uint4 &w1, const uint4 &w2,
                                          uint32_t lane_off, uint32_t x_off, uint32_t dmask, uint32_t base) {
    const uint32_t a1w[4] = {w1.x, w1.y, w1.z, w1.w};
    const uint32_t a2w[4] = {w2.x, w2.y, w2.z, w2.w};
    uint4 xb[4];
    xb[0] = lds_u128<SBASE, MMA_TBL_BYTES + 0>(x_off, base);
    xb[1] = lds_u128<SBASE, MMA_TBL_BYTES + 16>(x_off, base);
    xb[2] = lds_u128<SBASE, MMA_TBL_BYTES + 32>(x_off, base);
    xb[3] = lds_u128<SBASE, MMA_TBL_BYTES + 48>(x_off, base);
    uint32_t A[2][8];
    lookup_word<SBASE>(A[0], a1w[0], a2w[0], lane_off, base);
#pragma unroll
    for (int h = 0; h < 4; h++) {
        if (h < 3) lookup_word<SBASE>(A[(h + 1) & 1], a1w[h + 1], a2w[h + 1], lane_off, base);
        const uint32_t(&a)[8] = A[h & 1];
        // step 2h: bytes 0,1 (k0+8h .. +3); step 2h+1: bytes 2,3 (k0+8h+4 .. +7)
        mma_m16n8k16(acc[0], a[0], a[1], a[2], a[3], xb[h].x & dmask, xb[h].y & dmask);
        mma_m16n8k16(acc[1], a[4], a[5], a[6], a[7], xb[h].z & dmask, xb[h].w & dmask);
    }
}

template <int MODE, int SBASE>
__global__ void __launch_bounds__(MMA_THREADS, 3) lut_gemv_mma_kernel(const MmaGemvArgs a) {
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
    if (SBASE >= 0 && smem_base != (uint32_t)SBASE) {  // layout assumption broken: refuse to compute
        if (threadIdx.x == 0) atomicExch(a.err, 1u);
        return;
    }
    uint32_t *tbl = reinterpret_cast<uint32_t *>(smem);
    uint16_t *xs = reinterpret_cast<uint16_t *>(smem + MMA_TBL_BYTES);
    float *red = reinterpret_cast<float *>(smem + MMA_TBL_BYTES + MMA_MAX_KSLICE * 2);  // [MMA_WARPS][64]
    unsigned int &s_last = *reinterpret_cast<unsigned int *>(red + MMA_WARPS * 64);

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t blk = blockIdx.x, ks = blockIdx.y, bat = blockIdx.z;
    const uint32_t n_blocks = gridDim.x;
    const uint32_t c_begin = ks * a.chunks_per_split;
    const uint32_t c_end = min(a.n_chunks, c_begin + a.chunks_per_split);
    const uint32_t hb1 = a.hb_mul * blk, hb2 = hb1 + a.hb_add2;

    // ---- stage the x slice (fp16) -----------------------------------------------------------
    {
        const uint32_t n16 = (c_end - c_begin) * 4;  // 16-byte units: 32 halves per chunk
        const uint4 *xg = reinterpret_cast<const uint4 *>(a.x + (size_t)bat * a.x_stride + (size_t)c_begin * 32);
        uint4 *xd = reinterpret_cast<uint4 *>(xs);
        if (a.norm_n == 0) {
            for (uint32_t i = tid; i < n16; i += MMA_THREADS) xd[i] = xg[i];
        } else {
            // RMSNorm folded into the staging (rms_norm_inplace, src/lut/cpu_fallback.rs:39-54): every CTA
            // sums the squares of the whole row (a few KB from L2), then scales only its own K slice.
            const uint4 *xrow = reinterpret_cast<const uint4 *>(a.x + (size_t)bat * a.x_stride);
            float ss = 0.0f;
            for (uint32_t i = tid; i < a.norm_n / 8; i += MMA_THREADS) {
                const uint4 v = xrow[i];
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
            float tot = 0.0f;
#pragma unroll
            for (int w = 0; w < MMA_WARPS; w++) tot += red[w];  // fixed order: the same value in every CTA
            const float inv = 1.0f / sqrtf(tot / (float)a.norm_n + a.norm_eps);
            for (uint32_t i = tid; i < n16; i += MMA_THREADS) {
                uint4 v = xg[i];
                __half2 *hp = reinterpret_cast<__half2 *>(&v);
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float2 f = __half22float2(hp[e]);
                    hp[e] = __floats2half2_rn(f.x * inv, f.y * inv);
                }
                xd[i] = v;
            }
        }
    }
    // ---- build the pair tables: entry e = lo | hi<<4 -> half2{pal[lo], pal[hi]} -----------
    // warp w writes the entries with hi in {2w, 2w+1}; lane L writes its own bank.
#pragma unroll
    for (int t = 0; t < 2; t++) {
        const uint32_t row = (t == 0 ? hb1 : hb2) * 32 + lane;
        const uint16_t *prow = (t == 0 ? a.pal1 : a.pal2) + (size_t)row * 16;
        const uint4 p0 = *reinterpret_cast<const uint4 *>(prow);
        const uint4 p1 = *reinterpret_cast<const uint4 *>(prow + 8);
        const uint32_t cbp[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
        const uint32_t hi_pair = reinterpret_cast<const uint32_t *>(prow)[warp];  // {pal[2w], pal[2w+1]}
#pragma unroll
        for (int lo = 0; lo < 16; lo++) {
#pragma unroll
            for (int hs = 0; hs < 2; hs++) {
                const uint32_t sel = ((hs ? 0x76u : 0x54u) << 8) | ((lo & 1) ? 0x32u : 0x10u);
                const uint32_t v = __byte_perm(cbp[lo >> 1], hi_pair, sel);
                const uint32_t e = (uint32_t)lo + 16u * (2u * warp + (uint32_t)hs);
                tbl[e * 64 + t * 32 + lane] = v;
            }
        }
    }
    __syncthreads();

    // ---- stream the index chunks ------------------------------------------------------------
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    {
        const uint8_t *s1 = a.idx1 + (size_t)hb1 * a.n_chunks * 512 + lane * 16;
        const uint8_t *s2 = a.idx2 + (size_t)hb2 * a.n_chunks * 512 + lane * 16;
        const uint32_t lane_off = lane * 4;
        const uint32_t dmask = ((lane >> 2) == (lane & 3)) ? 0xFFFFFFFFu : 0u;  // lanes 0, 5, 10, 15

        uint4 q1[MMA_PF], q2[MMA_PF];
        uint32_t c = c_begin + warp;
#pragma unroll
        for (int i = 0; i < MMA_PF; i++) {
            const uint32_t cc = c + i * MMA_WARPS;
            if (cc < c_end) {
                q1[i] = ldg128_stream(s1 + (size_t)cc * 512);
                q2[i] = ldg128_stream(s2 + (size_t)cc * 512);
            }
        }
        for (; c < c_end; c += MMA_WARPS * MMA_PF) {
#pragma unroll
            for (int i = 0; i < MMA_PF; i++) {
                const uint32_t cc = c + i * MMA_WARPS;
                if (cc < c_end) {
                    const uint4 w1 = q1[i], w2 = q2[i];
                    const uint32_t nc = cc + MMA_WARPS * MMA_PF;
                    if (nc < c_end) {
                        q1[i] = ldg128_stream(s1 + (size_t)nc * 512);
                        q2[i] = ldg128_stream(s2 + (size_t)nc * 512);
                    }
                    mma_chunk<SBASE>(acc, w1, w2, lane_off, (cc - c_begin) * 64, dmask, smem_base);
                }
            }
        }
    }

    // ---- reduce across warps ---------------------------------------------------------------
    // accumulator column n = 2j, 2j+1 (j = lane%4) of MMA row g = lane/4 (and g+8):
    // column n is the dot product of the lane (g, n); only n < 4 is populated.
    if ((lane & 3) < 2) {
        const uint32_t r = (lane >> 2) * 4 + (lane & 3) * 2;  // lane index the column belongs to
        float *rw = red + warp * 64;
        rw[r] = acc[0][0] + acc[1][0];
        rw[r + 1] = acc[0][1] + acc[1][1];
        rw[32 + r] = acc[0][2] + acc[1][2];
        rw[32 + r + 1] = acc[0][3] + acc[1][3];
    }
    __syncthreads();

    float sum = 0.0f;  // thread tid < 64: row (tid>>5 ? "2" : "1"), lane tid&31
    if (tid < 64) {
#pragma unroll
        for (int w = 0; w < MMA_WARPS; w++) sum += red[w * 64 + tid];
    }
    if (a.ksplit > 1) {
        // deterministic split-K: every CTA stores its partial, the last one to arrive adds
        // them in split order.
        float *part = a.partials + ((size_t)bat * a.ksplit) * n_blocks * 64;
        if (tid < 64) part[((size_t)ks * n_blocks + blk) * 64 + tid] = sum;
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            unsigned int *ctr = a.counters + (size_t)bat * n_blocks + blk;
            const unsigned int prev = atomicAdd(ctr, 1u);
            s_last = (prev + 1 == a.ksplit) ? 1u : 0u;
            if (s_last) *ctr = 0;  // ready for the next launch on this stream
        }
        __syncthreads();
        if (!s_last) return;
        __threadfence();
        if (tid < 64) {
            sum = 0.0f;
            for (uint32_t s = 0; s < a.ksplit; s++)
                sum += __ldcg(part + ((size_t)s * n_blocks + blk) * 64 + tid);
        }
    }

    // ---- epilogue ---------------------------------------------------------------------------
    if (MODE == GEMV_SWIGLU) {
        // rows "1" are gate rows, rows "2" the up rows of the same output index
        __syncthreads();
        if (tid < 64) red[tid] = sum;
        __syncthreads();
        if (tid < 32) {
            const uint32_t row = blk * 32 + tid;
            if (row < a.m) {
                const float g = __half2float(__float2half_rn(red[tid]));
                const float u = __half2float(__float2half_rn(red[32 + tid]));
                const float s = __half2float(__float2half_rn(g / (1.0f + expf(-g))));
                a.y[(size_t)bat * a.y_stride + row] = __half_as_ushort(__float2half_rn(s * u));
            }
        }
    } else {
        if (tid < 64) {
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

constexpr size_t MMA_SMEM_BYTES = MMA_TBL_BYTES + MMA_MAX_KSLICE * 2 + MMA_WARPS * 64 * 4 + 16;

constexpr int MMA_KNOWN_SBASE = 1024;  // dynamic shared memory starts after the 1 KB the driver reserves

template <int MODE, int SBASE>
static int launch_mma_v(prism_cuda_ctx *ctx, const MmaGemvArgs &a, dim3 grid) {
    static bool configured[PRISM_MAX_DEVICES] = {false};
    if (!configured[ctx->device]) {
        PRISM_CUDA_TRY(ctx, cudaFuncSetAttribute(lut_gemv_mma_kernel<MODE, SBASE>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)MMA_SMEM_BYTES));
        configured[ctx->device] = true;
    }
    lut_gemv_mma_kernel<MODE, SBASE><<<grid, MMA_THREADS, MMA_SMEM_BYTES, ctx->stream>>>(a);
    return after_launch(ctx, "lut_gemv_mma_kernel");
}

template <int MODE>
static int launch_mma(prism_cuda_ctx *ctx, const MmaGemvArgs &a, dim3 grid) {
    if (ctx->smem_base == MMA_KNOWN_SBASE) return launch_mma_v<MODE, MMA_KNOWN_SBASE>(ctx, a, grid);
    return launch_mma_v<MODE, -1>(ctx, a, grid);
}

// Reports where dynamic shared memory starts inside the shared window for a kernel without
// static shared memory (run once per context).
__global__ void probe_smem_base_kernel(unsigned int *out) {
    extern __shared__ __align__(16) uint8_t smem[];
    if (threadIdx.x == 0) *out = (unsigned int)__cvta_generic_to_shared(smem);
}

int probe_smem_base(prism_cuda_ctx *ctx) {
    PRISM_CUDA_TRY(ctx, cudaMemsetAsync(ctx->dev_err, 0, 8, ctx->stream));
    probe_smem_base_kernel<<<1, 32, 4096, ctx->stream>>>(ctx->dev_err + 1);
    PRISM_TRY(after_launch(ctx, "probe_smem_base_kernel"));
    unsigned int v = 0;
    PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(&v, ctx->dev_err + 1, 4, cudaMemcpyDeviceToHost, ctx->stream));
    PRISM_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    ctx->smem_base = (int)v;
    return PRISM_OK;
}

static bool mma_eligible(const LutTensor &t) {
    return t.bits == 4 && t.k % 32 == 0 && t.k >= 32;
}

int launch_gemv(prism_cuda_ctx *ctx, GemvMode mode, const LutTensor &t, const LutTensor *t2,
                const uint16_t *x, uint32_t x_stride, uint16_t *y, uint32_t y_stride,
                const uint16_t *resid, uint32_t batch) {
    if (batch == 0) return PRISM_OK;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || ((size_t)x_stride * 2) % 16)
        return fail(ctx, PRISM_E_ARG, "gemv: activation must be 16-byte aligned");
    if (mode == GEMV_SWIGLU) {
        if (!t2 || t2->m != t.m || t2->k != t.k || t2->bits != t.bits)
            return fail(ctx, PRISM_E_ARG, "fused_gate_up: gate and up must have identical shape");
    }
    // a caller may ask for RMSNorm of x to be folded in (engine: the Norm node in front of a matmul)
    const float norm_eps = ctx->pending_norm_eps;
    ctx->pending_norm_eps = -1.0f;
    // variant 1 (default): the warp-specialised persistent kernel for large matrices, the stream-K
    // kernel for small ones; 2: tcgen05 kernel where eligible, else as 1; 3: the same tensor-core
    // inner loop on a (block, K split) grid; 4: warp-specialised kernel for every shape;
    // 5: stream-K kernel for every shape; 0: plain kernel
    const int v = ctx->gemv_variant;
    // 2..8 activation rows: one pass over the weights for all of them (larger batches in groups of 8)
    if (mode == GEMV_TP && batch != 1) return fail(ctx, PRISM_E_ARG, "the in-kernel all-reduce takes one activation row");
    const bool use_wsb = (v == 1 || v == 2) && batch >= 2 && wsb_eligible(t, batch < 8 ? batch : 8);
    const bool use_tc5 = !use_wsb && v == 2 && tc5_eligible(ctx, t, batch);
    const uint32_t cl_s = (!use_wsb && !use_tc5 && v == 1 && batch == 1) ? cl_cluster_size(ctx, t, mode == GEMV_SWIGLU, batch) : 0;
    if (cl_s && t.k % 8 == 0 && x_stride >= t.k)
        return launch_gemv_cl(ctx, mode, t, t2, x, x_stride, y, y_stride, resid, batch, norm_eps, cl_s);
    const bool use_ws = !use_wsb && !use_tc5 && ((v == 4 && ws_eligible(t)) ||
                                                 ((v == 1 || v == 2) && ws_preferred(ctx, t, mode == GEMV_SWIGLU, batch)));
    const bool use_sk = !use_wsb && !use_tc5 && !use_ws && (v == 1 || v == 2 || v == 5) && sk_eligible(t);
    const bool use_mma = !use_tc5 && ctx->gemv_variant == 3 && mma_eligible(t);
    if (norm_eps >= 0.0f && !((use_mma || use_sk || use_ws) && t.k % 8 == 0 && x_stride >= t.k)) {
        // this kernel choice cannot fold the norm: run it as its own kernel into scratch
        PRISM_TRY(ensure_act(ctx, (size_t)batch * x_stride + 64));
        uint16_t *xn = ctx->act_scratch;
        for (uint32_t b = 0; b < batch; b++)
            PRISM_TRY(launch_rms_norm(ctx, x + (size_t)b * x_stride, xn + (size_t)b * x_stride, t.k, norm_eps, 1));
        return launch_gemv(ctx, mode, t, t2, xn, x_stride, y, y_stride, resid, batch);
    }
    if (use_wsb) {
        for (uint32_t g0 = 0; g0 < batch; g0 += 8) {
            const uint32_t nb = batch - g0 < 8 ? batch - g0 : 8;
            const uint16_t *xg = x + (size_t)g0 * x_stride;
            void *yg = mode == GEMV_F32 ? (void *)(reinterpret_cast<float *>(y) + (size_t)g0 * y_stride)
                                        : (void *)(y + (size_t)g0 * y_stride);
            const uint16_t *rg = resid ? resid + (size_t)g0 * y_stride : nullptr;
            if (nb == 1) PRISM_TRY(launch_gemv(ctx, mode, t, t2, xg, x_stride, static_cast<uint16_t *>(yg), y_stride, rg, 1));
            else PRISM_TRY(launch_gemv_wsb(ctx, mode, t, t2, xg, x_stride, yg, y_stride, rg, nb));
        }
        return PRISM_OK;
    }
    if (mode == GEMV_TP && !(use_ws || use_sk) )
        return fail(ctx, PRISM_E_ARG, "the in-kernel all-reduce needs the pair-table GEMV (4-bit, K % 32 == 0, gemv_variant 1, one row)");
    if (use_tc5) return launch_gemv_tc5(ctx, mode, t, t2, x, y, resid);
    if (use_ws) return launch_gemv_ws(ctx, mode, t, t2, x, x_stride, y, y_stride, resid, batch, norm_eps);
    if (use_sk) return launch_gemv_sk(ctx, mode, t, t2, x, x_stride, y, y_stride, resid, batch, norm_eps);
    if (!use_mma) {
        // plain kernel + separate elementwise kernels keep the same rounding points
        if (mode == GEMV_SWIGLU) {
            const size_t st = t.m_pad;
            PRISM_TRY(ensure_tmp(ctx, 2 * (size_t)batch * st));
            uint16_t *g = ctx->tmp_scratch, *u = g + (size_t)batch * st;
            PRISM_TRY(launch_gemv(ctx, GEMV_PLAIN, t, nullptr, x, x_stride, g, (uint32_t)st, nullptr, batch));
            PRISM_TRY(launch_gemv(ctx, GEMV_PLAIN, *t2, nullptr, x, x_stride, u, (uint32_t)st, nullptr, batch));
            for (uint32_t b = 0; b < batch; b++)
                PRISM_TRY(launch_silu_mul(ctx, y + (size_t)b * y_stride, g + b * st, u + b * st, t.m));
            return PRISM_OK;
        }
        if (mode == GEMV_F32) return fail(ctx, PRISM_E_ARG, "fp32 partial output needs the tensor-core GEMV (4-bit, K % 32 == 0)");
        if (mode == GEMV_RESID && y == resid) {
            // in place (y is the residual stream): the product goes to scratch first, then y = f16(y + W x)
            const size_t st = t.m_pad;
            PRISM_TRY(ensure_tmp(ctx, (size_t)batch * st));
            uint16_t *p = ctx->tmp_scratch;
            PRISM_TRY(launch_gemv(ctx, GEMV_PLAIN, t, nullptr, x, x_stride, p, (uint32_t)st, nullptr, batch));
            for (uint32_t b = 0; b < batch; b++)
                PRISM_TRY(launch_vec_add(ctx, y + (size_t)b * y_stride, p + b * st, t.m));
            return PRISM_OK;
        }
        dim3 grid(t.n_hb, batch);
        if (t.bits == 4)
            lut_gemv_simple_kernel<4><<<grid, SIMPLE_WARPS * 32, 0, ctx->stream>>>(
                t.idx, t.pal, t.m, t.k, t.n_chunks, x, x_stride, y, y_stride);
        else
            lut_gemv_simple_kernel<2><<<grid, SIMPLE_WARPS * 32, 0, ctx->stream>>>(
                t.idx, t.pal, t.m, t.k, t.n_chunks, x, x_stride, y, y_stride);
        PRISM_TRY(after_launch(ctx, "lut_gemv_simple_kernel"));
        if (mode == GEMV_RESID) {
            for (uint32_t b = 0; b < batch; b++)
                PRISM_TRY(launch_vec_add(ctx, y + (size_t)b * y_stride, resid + (size_t)b * y_stride, t.m));
        }
        return PRISM_OK;
    }

    MmaGemvArgs a{};
    a.n_chunks = t.n_chunks;
    a.m = t.m;
    a.x = x; a.x_stride = x_stride; a.y = y; a.y_stride = y_stride; a.resid = resid;
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
    // split K so that (a) a slice of x fits the staging buffer, (b) the grid fills the GPU
    const uint32_t max_chunks = MMA_MAX_KSLICE / 32;
    uint32_t ksplit = (t.n_chunks + max_chunks - 1) / max_chunks;
    const uint32_t target = (uint32_t)ctx->sm_count * 3;
    while (n_blocks * batch * ksplit < target && t.n_chunks / (ksplit * 2) >= 8) ksplit *= 2;
    uint32_t cps = (t.n_chunks + ksplit - 1) / ksplit;
    ksplit = (t.n_chunks + cps - 1) / cps;
    a.chunks_per_split = cps;
    a.ksplit = ksplit;
    if (ksplit > 1) {
        PRISM_TRY(ensure_splitk(ctx, (size_t)batch * ksplit * n_blocks * 64, (size_t)batch * n_blocks));
        a.partials = ctx->splitk_partials;
        a.counters = ctx->splitk_counters;
    }
    dim3 grid(n_blocks, ksplit, batch);
    switch (mode) {
    case GEMV_PLAIN: return launch_mma<GEMV_PLAIN>(ctx, a, grid);
    case GEMV_RESID: return launch_mma<GEMV_RESID>(ctx, a, grid);
    case GEMV_F32: return launch_mma<GEMV_F32>(ctx, a, grid);
    default: return launch_mma<GEMV_SWIGLU>(ctx, a, grid);
    }
}

// ---------------------------------------------------------------------------
// GEMV for callers that must not allocate
// ---------------------------------------------------------------------------
// Some hosts of this library cannot tolerate a device allocation on the GEMV path: an
// inference server that has already handed every free byte of HBM to its own weight and
// KV-cache pools (so a later cudaMalloc can fail, or stall the whole device while it
// runs), or a real-time decode loop with a fixed memory budget.  prism_cuda_gemv_dev may
// grow the context's split-K scratch with cudaMalloc the first time a shape needs it;
// prism_cuda_gemv_static_dev below never does.  Its split-K partial sums and arrival
// counters live in the fixed array that follows, which every GPU that loads this library
// holds (2 MiB + 16 KiB) until the process exits.
//
//  * All calls on a device share the array; it keeps whatever the previous call left.
//    The arrival counters are cleared on the stream before every launch; partial sums are
//    always fully written before they are read, so they need no clearing.
//  * Two calls whose kernels overlap on the GPU (different streams / contexts of the same
//    device) race on the array.  Calls on one context are stream-ordered and safe.
//  * The first call on a device resolves the array's device address (cudaGetSymbolAddress);
//    make that first call outside any stream capture.
//  * Shapes whose split-K scratch would exceed the array are rejected with PRISM_E_ARG.
constexpr size_t STATIC_PARTIAL_FLOATS = 512 * 1024;  // 2 MiB of fp32 partial sums
constexpr size_t STATIC_COUNTERS = 4096;              // one arrival counter per 64-row block
static __device__ __align__(256) float g_static_splitk[STATIC_PARTIAL_FLOATS + STATIC_COUNTERS];

// In host code `g_static_splitk` is only a stand-in for the symbol; the device address has to be
// asked for, once per device, with that device current.
static float *g_static_splitk_dev[PRISM_MAX_DEVICES] = {nullptr};

static int static_scratch_ptr(prism_cuda_ctx *ctx, float **out) {
    // every call: the launch and the memset below must go to the context's device whatever the
    // calling thread had current
    PRISM_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    if (!g_static_splitk_dev[ctx->device]) {
        void *p = nullptr;
        PRISM_CUDA_TRY(ctx, cudaGetSymbolAddress(&p, g_static_splitk));
        g_static_splitk_dev[ctx->device] = static_cast<float *>(p);
    }
    *out = g_static_splitk_dev[ctx->device];
    return PRISM_OK;
}

}  // namespace prism

using namespace prism;

extern "C" int prism_cuda_gemv_static_dev(prism_cuda_ctx *ctx, int32_t handle, const void *x_dev, void *y_dev) {
    LutTensor *tp = get_tensor(ctx, handle);
    if (!tp) return ctx ? PRISM_E_NOTFOUND : PRISM_E_NULL;
    if (!x_dev || !y_dev) return fail(ctx, PRISM_E_NULL, "null vector");
    const LutTensor &t = *tp;
    if (!mma_eligible(t))
        return fail(ctx, PRISM_E_ARG, "gemv_static: needs a 4-bit tensor with dim_n a multiple of 32");
    if (reinterpret_cast<uintptr_t>(x_dev) & 15) return fail(ctx, PRISM_E_ARG, "gemv_static: x must be 16-byte aligned");
    float *scratch = nullptr;
    PRISM_TRY(static_scratch_ptr(ctx, &scratch));
    MmaGemvArgs a{};
    a.n_chunks = t.n_chunks;
    a.m = t.m;
    a.x = static_cast<const uint16_t *>(x_dev); a.x_stride = round_up_u32(t.k, 8);
    a.y = static_cast<uint16_t *>(y_dev); a.y_stride = t.m;
    a.err = ctx->dev_err;
    a.idx1 = a.idx2 = t.idx; a.pal1 = a.pal2 = t.pal;
    a.hb_mul = 2; a.hb_add2 = 1;
    const uint32_t n_blocks = t.n_hb / 2;
    // same split rule as the allocating path: x slice fits its staging buffer, grid fills the GPU
    const uint32_t max_chunks = MMA_MAX_KSLICE / 32;
    uint32_t ksplit = (t.n_chunks + max_chunks - 1) / max_chunks;
    const uint32_t target = (uint32_t)ctx->sm_count * 3;
    while (n_blocks * ksplit < target && t.n_chunks / (ksplit * 2) >= 8) ksplit *= 2;
    const uint32_t cps = (t.n_chunks + ksplit - 1) / ksplit;
    ksplit = (t.n_chunks + cps - 1) / cps;
    a.chunks_per_split = cps;
    a.ksplit = ksplit;
    if (ksplit > 1) {
        const size_t need = (size_t)ksplit * n_blocks * 64;
        if (need > STATIC_PARTIAL_FLOATS || n_blocks > STATIC_COUNTERS)
            return fail(ctx, PRISM_E_ARG,
                        "gemv_static: this shape needs " + std::to_string(need) + " partial sums and " +
                            std::to_string(n_blocks) + " counters; the fixed scratch holds " +
                            std::to_string(STATIC_PARTIAL_FLOATS) + " and " + std::to_string(STATIC_COUNTERS));
        a.partials = scratch;
        a.counters = reinterpret_cast<unsigned int *>(scratch + STATIC_PARTIAL_FLOATS);
        PRISM_CUDA_TRY(ctx, cudaMemsetAsync(a.counters, 0, (size_t)n_blocks * sizeof(unsigned int), ctx->stream));
    }
    return launch_mma<GEMV_PLAIN>(ctx, a, dim3(n_blocks, ksplit, 1));
}
