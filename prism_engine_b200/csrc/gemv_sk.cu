// Palettized GEMV, persistent "stream-K" form of the pair-table tensor-core kernel.
//
// y = W x with W stored as 4-bit palette indices + a 16-entry fp16 palette per row
// (lut_gemv_cpu, src/lut/cpu_fallback.rs:12-35; fused gate/up: engine_impl.rs FusedGateUp), or as
// 2-bit indices + a 4-entry palette (BITS = 2; no such format in the reference).  At 2 bits a
// 16-byte chunk holds 64 weights of a row; every NIBBLE (two weights) is looked up in a 16-entry pair
// table, through the same lookup and mma.sync code as the 4-bit bytes: the two nibble planes of an
// index word are separated and re-interleaved into two "pseudo-words" whose bytes are table indices.
//
// Work is counted in units of (block, chunk): a block is two half-blocks of 32 rows (64 output
// rows, or 32 gate + 32 up rows), a chunk is 32 weights (16 index bytes) of every row of the block,
// i.e. 1 KB of indices.  The U = n_blocks * n_chunks units are laid out block-major and cut into G
// contiguous, nearly equal ranges, one per CTA, with G = 3 CTAs x SM count: every CTA streams the
// same number of bytes, so there is no partial last wave.  A range is walked as segments (one
// block, a run of chunks).  For each segment the CTA builds the block's pair tables in shared
// memory, stages the matching slice of x, streams the chunks through mma.sync.m16n8k16 and
// reduces to 64 sums.  A segment that covers a whole block writes its outputs; otherwise the sums
// go to a partial slot and the CTA that completes the block (arrival counter in chunks) adds the
// partials in range order, so results do not depend on scheduling.
#include "common.cuh"
#include "pair_table.cuh"

namespace prism {

constexpr int SK_WARPS = 8;
constexpr int SK_CTAS_PER_SM = 3;
constexpr int SK_THREADS = SK_WARPS * 32;
constexpr int SK_PIECE_BYTES = SK_WARPS * 16 * 64;  // x staged at a time: 4096 halves, 8 KB (128 chunks at 4 bit, 64 at 2 bit)
constexpr int SK_PF = 2;                 // index chunks in flight per warp (1, 2 or 4)
constexpr int SK_KNOWN_SBASE = 1024;      // dynamic shared memory starts after the 1 KB the driver reserves
constexpr size_t SK_SMEM_BYTES = SK_TBL_BYTES + SK_PIECE_BYTES + SK_WARPS * 64 * 4 + 32 + 2 * TP_LIST_MAX * 2;


// A 2-bit chunk (64 weights per row) as two pseudo 4-bit chunks of 32 weights each.
template <int SBASE, int NEXT_IMM, typename SRC>
__device__ __forceinline__ void sk_chunk2(float (&acc)[SK_NACC][4], uint4 &w1, uint4 &w2, uint4 (&xb)[2], uint32_t lane_off,
                                          uint32_t x_off, uint32_t diag, uint32_t base, const SRC &next, bool more) {
    uint4 a1, b1, a2, b2;
    sk_expand2(a1, b1, w1);
    sk_expand2(a2, b2, w2);
    if (more) {  // the index words are dead once expanded: the chunk PF steps ahead goes into them
        w1 = next.template load1<NEXT_IMM>();
        w2 = next.template load2<NEXT_IMM>();
    }
    const SkNoNext none;
    sk_chunk<SBASE, 0>(acc, a1, a2, xb, lane_off, x_off, diag, base, none, false);
    sk_chunk<SBASE, 0>(acc, b1, b2, xb, lane_off, x_off + 64, diag, base, none, false);
}

template <int MODE, int SBASE, int BITS>
__global__ void __launch_bounds__(SK_THREADS, SK_CTAS_PER_SM) lut_gemv_sk_kernel(const SkArgs a) {
    constexpr uint32_t XB = BITS == 4 ? 64 : 128;               // bytes of x per chunk (32 or 64 halves)
    constexpr uint32_t SK_PIECE_CHUNKS = SK_PIECE_BYTES / XB;   // chunks of x staged at a time
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
    if (SBASE >= 0 && smem_base != (uint32_t)SBASE) {  // layout assumption broken: refuse to compute
        if (threadIdx.x == 0) atomicExch(a.err, 1u);
        return;
    }
    uint32_t *tbl = reinterpret_cast<uint32_t *>(smem);
    uint16_t *xs = reinterpret_cast<uint16_t *>(smem + SK_TBL_BYTES);
    float *red = reinterpret_cast<float *>(smem + SK_TBL_BYTES + SK_PIECE_BYTES);  // [SK_WARPS][64]
    unsigned int &s_last = *reinterpret_cast<unsigned int *>(red + SK_WARPS * 64);
    float &s_inv = *reinterpret_cast<float *>(red + SK_WARPS * 64 + 1);

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t cta = blockIdx.x, G = gridDim.x, bat = blockIdx.y;
    const uint32_t nc = a.n_chunks;
    const uint32_t u_begin = sk_boundary(a.part, cta);
    const uint32_t u_end = sk_boundary(a.part, cta + 1);
    pdl_launch_dependents();
    if (u_begin >= u_end) return;
    const uint16_t *xrow = a.x + (size_t)bat * a.x_stride;
    const uint32_t lane_off = lane * 4;
    const uint32_t diag = ((lane >> 2) == (lane & 3)) ? 1u : 0u;  // lanes 0, 5, 10, 15
    uint4 xb[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};

    float inv = 1.0f;
    bool waited = false;
    // GEMV_TP: what warps 0 and 1 have delivered to the peers, finished when the CTA has nothing left to stream
    TpWarpList wl{reinterpret_cast<uint16_t *>(red + SK_WARPS * 64 + 8) + (warp & 1) * TP_LIST_MAX, 0};

    for (uint32_t u = u_begin; u < u_end;) {
        const uint32_t blk = u / nc;
        const uint32_t cb = u - blk * nc;
        const uint32_t ce = min(nc, cb + (u_end - u));
        u += ce - cb;
        const uint32_t hb1 = a.hb_mul * blk, hb2 = hb1 + a.hb_add2;

        // ---- first index chunks of this warp: in flight while the tables are built ---------------
        // warp w handles chunks cb + w + 8j, j < nj
        const uint32_t span = ce - cb;
        const uint32_t nj = span > warp ? (span - warp + SK_WARPS - 1) / SK_WARPS : 0;
        SkSrcPtr src;
        src.p = a.idx1 + ((size_t)hb1 * nc + cb + warp) * 512 + lane * 16;
        src.d2 = (uint64_t)(reinterpret_cast<uintptr_t>(a.idx2 + ((size_t)hb2 * nc + cb + warp) * 512 + lane * 16) -
                            reinterpret_cast<uintptr_t>(src.p));
        uint4 q1[SK_PF], q2[SK_PF];
        if (0 < nj) { q1[0] = src.template load1<0>(); q2[0] = src.template load2<0>(); }
        if (SK_PF > 1 && 1 < nj) { q1[1 % SK_PF] = src.template load1<1 * SK_WARPS * 512>(); q2[1 % SK_PF] = src.template load2<1 * SK_WARPS * 512>(); }
        if (SK_PF > 2 && 2 < nj) { q1[2 % SK_PF] = src.template load1<2 * SK_WARPS * 512>(); q2[2 % SK_PF] = src.template load2<2 * SK_WARPS * 512>(); }
        if (SK_PF > 3 && 3 < nj) { q1[3 % SK_PF] = src.template load1<3 * SK_WARPS * 512>(); q2[3 % SK_PF] = src.template load2<3 * SK_WARPS * 512>(); }
        src.advance(SK_PF * SK_WARPS * 512);  // from here on: the chunk SK_PF steps ahead

        __syncthreads();  // the previous segment is done with the tables, x and the reduction buffer
        // ---- pair tables: entry e = lo | hi<<4 -> half2{pal[lo], pal[hi]} ------------------------
        // warp w writes the entries with hi = w, w + SK_WARPS, ...; lane L writes its own bank.
        if (BITS == 4) {
#pragma unroll
            for (int t = 0; t < 2; t++) {
                const uint32_t row = (t == 0 ? hb1 : hb2) * 32 + lane;
                const uint16_t *prow = (t == 0 ? a.pal1 : a.pal2) + (size_t)row * 16;
                const uint4 p0 = *reinterpret_cast<const uint4 *>(prow);
                const uint4 pp = *reinterpret_cast<const uint4 *>(prow + 8);
                const uint32_t cbp[8] = {p0.x, p0.y, p0.z, p0.w, pp.x, pp.y, pp.z, pp.w};
                for (uint32_t hi = warp; hi < 16; hi += SK_WARPS) {
                    const uint32_t hi_pair = reinterpret_cast<const uint32_t *>(prow)[hi >> 1];  // {pal[hi&~1], pal[hi|1]}
                    const uint32_t hsel = (hi & 1) ? 0x7600u : 0x5400u;
#pragma unroll
                    for (int lo = 0; lo < 16; lo++) {
                        const uint32_t v = __byte_perm(cbp[lo >> 1], hi_pair, hsel | ((lo & 1) ? 0x32u : 0x10u));
                        tbl[((uint32_t)lo + 16u * hi) * 64 + t * 32 + lane] = v;
                    }
                }
            }
        } else {
            sk_build_table2(tbl, a.pal1, a.pal2, hb1, hb2, lane, warp, SK_WARPS);
        }

        if (!waited) {
            // Everything above reads only weights.  x, the partial sums, the counters and y belong to
            // the stream order: wait for the kernels before this one.
            pdl_wait();
            waited = true;
            // RMSNorm folded into the staging (rms_norm_inplace, src/lut/cpu_fallback.rs:39-54): every CTA
            // sums the squares of the whole row once (a few KB from L2) and scales the slices it stages.
            if (a.norm_n) {
                const uint4 *xr = reinterpret_cast<const uint4 *>(xrow);
                float ss = 0.0f;
                for (uint32_t i = tid; i < a.norm_n / 8; i += SK_THREADS) {
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
                    for (int w = 0; w < SK_WARPS; w++) tot += red[w];  // fixed order: the same value in every CTA
                    s_inv = 1.0f / sqrtf(tot / (float)a.norm_n + a.norm_eps);
                }
                __syncthreads();
                inv = s_inv;
            }
        }

        float acc[SK_NACC][4];
#pragma unroll
        for (int i = 0; i < SK_NACC; i++) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
        uint32_t j = 0;
        for (uint32_t pb = cb; pb < ce; pb += SK_PIECE_CHUNKS) {
            // ---- stage this piece of x (fp16, normalised on the way if asked) --------------------
            if (pb != cb) __syncthreads();  // every warp has finished reading the previous piece
            {
                const uint32_t n16 = (min(ce, pb + SK_PIECE_CHUNKS) - pb) * (XB / 16);  // 16-byte units
                const uint4 *xg = reinterpret_cast<const uint4 *>(xrow + (size_t)pb * (XB / 2));
                uint4 *xd = reinterpret_cast<uint4 *>(xs);
                if (a.norm_n == 0) {
                    for (uint32_t i = tid; i < n16; i += SK_THREADS) xd[i] = xg[i];
                } else {
                    for (uint32_t i = tid; i < n16; i += SK_THREADS) {
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
            __syncthreads();
            // ---- stream this warp's chunks of the piece: 16 per full piece ------------------------
            const uint32_t j_end = min(nj, j + SK_PIECE_CHUNKS / SK_WARPS);
            uint32_t x_off = warp * XB;
#define SK_STEP(I)                                                                                              \
    if ((I) < SK_PF && ((I) == 0 || j + (I) < j_end)) {                                                         \
        if (BITS == 4)                                                                                          \
            sk_chunk<SBASE, (I) * SK_WARPS * 512>(acc, q1[(I) % SK_PF], q2[(I) % SK_PF], xb, lane_off,              \
                                                  x_off + (I) * SK_WARPS * XB, diag, smem_base, src,             \
                                                  j + (I) + SK_PF < nj);                                        \
        else                                                                                                    \
            sk_chunk2<SBASE, (I) * SK_WARPS * 512>(acc, q1[(I) % SK_PF], q2[(I) % SK_PF], xb, lane_off,             \
                                                   x_off + (I) * SK_WARPS * XB, diag, smem_base, src,            \
                                                   j + (I) + SK_PF < nj);                                       \
    }
            for (; j < j_end; j += SK_PF) {
                SK_STEP(0) SK_STEP(1) SK_STEP(2) SK_STEP(3)
                x_off += SK_PF * SK_WARPS * XB;
                src.advance(SK_PF * SK_WARPS * 512);
            }
#undef SK_STEP
            j = j_end;
        }

        // ---- reduce across warps ---------------------------------------------------------------
        // accumulator column n = 2q, 2q+1 (q = lane%4) of MMA row g = lane/4 (and g+8): column n is
        // the dot product of the lane (g, n); only n < 4 is populated.
        if ((lane & 3) < 2) {
            const uint32_t r = (lane >> 2) * 4 + (lane & 3) * 2;  // lane index the column belongs to
            float *rw = red + warp * 64;
            float c0 = acc[0][0] + acc[1][0], c1 = acc[0][1] + acc[1][1];
            float c2 = acc[0][2] + acc[1][2], c3 = acc[0][3] + acc[1][3];
            if (SK_NACC == 4) {
                c0 += acc[SK_NACC - 2][0] + acc[SK_NACC - 1][0]; c1 += acc[SK_NACC - 2][1] + acc[SK_NACC - 1][1];
                c2 += acc[SK_NACC - 2][2] + acc[SK_NACC - 1][2]; c3 += acc[SK_NACC - 2][3] + acc[SK_NACC - 1][3];
            }
            rw[r] = c0;
            rw[r + 1] = c1;
            rw[32 + r] = c2;
            rw[32 + r + 1] = c3;
        }
        __syncthreads();
        float sum = 0.0f;  // thread tid < 64: rows "1" (tid < 32) or "2", lane tid & 31
        if (tid < 64) {
#pragma unroll
            for (int w = 0; w < SK_WARPS; w++) sum += red[w * 64 + tid];
        }

        if (span != nc) {
            // part of a block: leave the sums in this CTA's slot (0: the range starts inside the
            // block, 1: it starts with the block); whoever completes the block adds the slots in
            // range order.
            float *part = a.partials + (size_t)bat * G * 128;
            if (tid < 64) part[((size_t)cta * 2 + (cb > 0 ? 0 : 1)) * 64 + tid] = sum;
            __syncthreads();
            if (tid == 0) {
                unsigned int *ctr = a.counters + (size_t)bat * a.n_blocks + blk;
                const unsigned int prev = sk_arrive(ctr, span);
                s_last = (prev + span == nc) ? 1u : 0u;
                if (s_last) *ctr = 0;  // ready for the next launch on this stream
            }
            __syncthreads();
            if (!s_last) continue;
            // The contributors of the block are consecutive CTAs.  Thread k works out what CTA
            // c0 + k left (slot 0: its range starts inside the block, slot 1: it starts with the
            // block); then 64 threads add the slots in that order, four loads in flight.
            {
                const uint32_t b0 = blk * nc, b1 = b0 + nc;
                const SkPart &p = a.part;
                // first contributor: the CTA whose unsnapped range holds b0, unless its snapped range ends there
                uint32_t c0;
                if (p.s) {
                    c0 = blk * p.s;
                } else {
                    c0 = (b0 < p.r * (p.q + 1)) ? b0 / (p.q + 1) : p.r + (b0 - p.r * (p.q + 1)) / p.q;
                    if (sk_boundary_in_block(p, c0 + 1, b0) <= b0) c0 += 1;
                }
                const uint32_t c = c0 + tid;
                const uint32_t r0 = c < G ? sk_boundary_in_block(p, c, b0) : b1;
                const uint32_t r1 = c < G ? sk_boundary_in_block(p, c + 1, b0) : b1;
                uint32_t *list = reinterpret_cast<uint32_t *>(xs);  // x is not needed any more
                list[tid] = (r1 > r0) ? (c * 2 + (r0 > b0 ? 0u : 1u)) : 0xFFFFFFFFu;
                const uint32_t n = (uint32_t)__syncthreads_count(c < G && r0 < b1);
                // thread (g, t): contributors g, g+NG, ... of output t, four loads in flight
                constexpr uint32_t NG = SK_THREADS / 64;
                const uint32_t g = tid >> 6, t = tid & 63;
                if (g < NG) {
                    float ps = 0.0f;
                    for (uint32_t k = g; k < n; k += 4 * NG) {
                        float v[4];
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const uint32_t slot = (k + NG * e < n) ? list[k + NG * e] : 0xFFFFFFFFu;
                            v[e] = (slot != 0xFFFFFFFFu) ? __ldcg(part + (size_t)slot * 64 + t) : 0.0f;
                        }
#pragma unroll
                        for (int e = 0; e < 4; e++) ps += v[e];
                    }
                    red[g * 64 + t] = ps;
                }
                __syncthreads();
                if (tid < 64) {
                    sum = red[tid];
#pragma unroll
                    for (uint32_t gg = 1; gg < NG; gg++) sum += red[gg * 64 + tid];
                }
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
                    const float uu = __half2float(__float2half_rn(red[32 + tid]));
                    const float s = __half2float(__float2half_rn(g / (1.0f + expf(-g))));
                    a.y[(size_t)bat * a.y_stride + row] = __half_as_ushort(__float2half_rn(s * uu));
                }
            }
        } else if (MODE == GEMV_TP) {
            if (tid < 64) tp_deliver_listed(a.tp, wl, (tid >> 5) ? hb2 : hb1, lane, sum, a.m, a.y + (size_t)bat * a.y_stride, a.err);
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
    if (MODE == GEMV_TP && tid < 64) tp_finish(a.tp, tp_epoch(a.tp), wl.list, wl.n, lane, a.m, a.y + (size_t)bat * a.y_stride, a.err);
}

template <int MODE, int SBASE, int BITS>
static int launch_sk_v(prism_cuda_ctx *ctx, const SkArgs &a, dim3 grid) {
    static bool configured[PRISM_MAX_DEVICES] = {false};
    if (!configured[ctx->device]) {
        PRISM_CUDA_TRY(ctx, cudaFuncSetAttribute(lut_gemv_sk_kernel<MODE, SBASE, BITS>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SK_SMEM_BYTES));
        configured[ctx->device] = true;
    }
    launch_pdl(ctx, "lut_gemv_sk_kernel", lut_gemv_sk_kernel<MODE, SBASE, BITS>, grid, SK_THREADS, SK_SMEM_BYTES, a);
    return after_launch(ctx, "lut_gemv_sk_kernel");
}

template <int MODE>
static int launch_sk(prism_cuda_ctx *ctx, const SkArgs &a, dim3 grid, uint32_t bits) {
    if (bits == 2) {
        if (ctx->smem_base == SK_KNOWN_SBASE) return launch_sk_v<MODE, SK_KNOWN_SBASE, 2>(ctx, a, grid);
        return launch_sk_v<MODE, -1, 2>(ctx, a, grid);
    }
    if (ctx->smem_base == SK_KNOWN_SBASE) return launch_sk_v<MODE, SK_KNOWN_SBASE, 4>(ctx, a, grid);
    return launch_sk_v<MODE, -1, 4>(ctx, a, grid);
}

// 4 bit: whole 32-weight chunks; 2 bit: whole 64-weight chunks
bool sk_eligible(const LutTensor &t) {
    return (t.bits == 4 && t.k % 32 == 0 && t.k >= 32) || (t.bits == 2 && t.k % 64 == 0 && t.k >= 64);
}

// Chooses the partition (see SkPart) for one activation vector of a batch.
SkPart sk_partition(prism_cuda_ctx *ctx, uint32_t n_blocks, uint32_t n_chunks, uint32_t batch) {
    const uint32_t slots = (uint32_t)ctx->sm_count * SK_CTAS_PER_SM / (batch ? batch : 1);
    return sk_choose_partition(n_blocks, n_chunks, slots, (uint32_t)ctx->sk_stream_chunks, (uint32_t)ctx->sk_min_chunks, 128);
}

int launch_gemv_sk(prism_cuda_ctx *ctx, GemvMode mode, const LutTensor &t, const LutTensor *t2, const uint16_t *x,
                   uint32_t x_stride, void *y, uint32_t y_stride, const uint16_t *resid, uint32_t batch,
                   float norm_eps) {
    SkArgs a{};
    a.n_chunks = t.n_chunks;
    a.m = t.m;
    a.x = x; a.x_stride = x_stride; a.y = static_cast<uint16_t *>(y); a.y_stride = y_stride; a.resid = resid;
    a.err = ctx->dev_err;
    a.norm_n = norm_eps >= 0.0f ? t.k : 0;
    a.norm_eps = norm_eps >= 0.0f ? norm_eps : 0.0f;
    if (mode == GEMV_SWIGLU) {
        a.idx1 = t.idx; a.pal1 = t.pal; a.idx2 = t2->idx; a.pal2 = t2->pal;
        a.hb_mul = 1; a.hb_add2 = 0;
        a.n_blocks = t.n_hb;
    } else {
        a.idx1 = a.idx2 = t.idx; a.pal1 = a.pal2 = t.pal;
        a.hb_mul = 2; a.hb_add2 = 1;
        a.n_blocks = t.n_hb / 2;
    }
    a.part = sk_partition(ctx, a.n_blocks, a.n_chunks, batch);
    const uint32_t G = a.part.G;
    PRISM_TRY(ensure_splitk(ctx, (size_t)batch * G * 128, (size_t)batch * a.n_blocks));
    a.partials = ctx->splitk_partials;
    a.counters = ctx->splitk_counters;
    const dim3 grid(G, batch);
    switch (mode) {
    case GEMV_PLAIN: return launch_sk<GEMV_PLAIN>(ctx, a, grid, t.bits);
    case GEMV_RESID: return launch_sk<GEMV_RESID>(ctx, a, grid, t.bits);
    case GEMV_F32: return launch_sk<GEMV_F32>(ctx, a, grid, t.bits);
    case GEMV_TP:
        PRISM_TRY(tp_fill_push(ctx, t, &a.tp));
        return launch_sk<GEMV_TP>(ctx, a, grid, t.bits);
    default: return launch_sk<GEMV_SWIGLU>(ctx, a, grid, t.bits);
    }
}

}  // namespace prism
