// Palettized GEMV, warp-specialised persistent form of the pair-table tensor-core kernel.
//
// y = W x with W stored as 4-bit palette indices + a 16-entry fp16 palette per row
// (lut_gemv_cpu, src/lut/cpu_fallback.rs:12-35; fused gate/up: engine_impl.rs FusedGateUp).
//
// One CTA per SM.  The (block, chunk) units of the matrix are dealt to the CTAs as in the
// stream-K kernel (SkPart); a CTA walks its range as stages: (block, run of at most
// WS_STAGE_CHUNKS chunks).  Two groups of warps work on the stages as a pipeline:
//   * builder warps prepare a stage: the block's pair tables (when the stage opens a new block) in
//     one of two table buffers, and the stage's slice of x (normalised if asked) in one of two x
//     buffers; they also finish a block: add the compute warps' sums, write y or the partial sums,
//     and run the deterministic fix-up when this CTA completes a block;
//   * compute warps stream the stage's index chunks through table lookups and mma.sync and leave
//     64 sums per warp when a block's run ends.
// While the compute warps stream stage t, the builders prepare stage t+1 and finish stage t-1, so
// the palette loads, table stores, x staging, reductions and global atomics of a stage are off
// the streaming path.  Hand-over is by mbarriers in shared memory (full[buf]: builders -> compute,
// empty[buf]: compute -> builders); every wait is bounded and sets the error word if it gives up.
#include "common.cuh"
#include "pair_table.cuh"
#include "tc5_ptx.cuh"
#include "ws_common.cuh"

namespace prism {

constexpr int WS_NC = 20;                       // compute warps
constexpr int WS_NB = 4;                        // builder warps
static_assert(WS_NB * 32 == WS_COMMON_BTHREADS, "the finish step (scratch sizes, two groups of 64 threads) is written for 128 builder threads");
constexpr int WS_THREADS = (WS_NC + WS_NB) * 32;
constexpr int WS_BTHREADS = WS_NB * 32;
constexpr int WS_PF = 2;                        // index chunks in flight per compute warp (1, 2 or 4)
constexpr int WS_STAGE_CHUNKS = 256;            // chunks of x per stage (8192 halves, 16 KB)
constexpr int WS_TBL_BYTES = 65536;             // one pair-table buffer
constexpr int WS_X_OFF = 2 * WS_TBL_BYTES;      // two x buffers
constexpr int WS_X_BYTES = WS_STAGE_CHUNKS * 64;
constexpr int WS_RED_OFF = WS_X_OFF + 2 * WS_X_BYTES;       // [2][WS_NC][64] floats
constexpr int WS_FIN_OFF = WS_RED_OFF + 2 * WS_NC * 64 * 4; // builder scratch: 256 words
constexpr int WS_BAR_OFF = WS_FIN_OFF + 256 * 4;            // full[2], empty[2], flags
constexpr int WS_TPL_OFF = WS_BAR_OFF + 64;                 // GEMV_TP: two lists of delivered half-blocks
constexpr size_t WS_SMEM_BYTES = WS_TPL_OFF + 2 * TP_LIST_MAX * 2;
constexpr int WS_KNOWN_SBASE = 1024;


// One 32-weight chunk of the two half-blocks (see sk_chunk in gemv_sk.cu for the operand layout);
// compute warps are WS_NC chunks apart.
template <int SBASE, int NEXT_IMM>
__device__ __forceinline__ void ws_chunk(float (&acc)[2][4], uint4 &w1, uint4 &w2, uint4 (&xb)[2], uint32_t lane_off,
                                         uint32_t x_off, uint32_t diag, uint32_t base, const SkSrcPtr &next, bool more) {
    sk_ldx<SBASE, WS_X_OFF + 0>(xb[0], x_off, base, diag);
    sk_ldx<SBASE, WS_X_OFF + 16>(xb[1], x_off, base, diag);
    uint32_t A0[8], A1[8];
    sk_lookup<SBASE>(A0, w1.x, w2.x, lane_off, base);
    sk_lookup<SBASE>(A1, w1.y, w2.y, lane_off, base);
    sk_mma(acc[0], A0[0], A0[1], A0[2], A0[3], xb[0].x, xb[0].y);
    sk_mma(acc[1], A0[4], A0[5], A0[6], A0[7], xb[0].z, xb[0].w);
    sk_ldx<SBASE, WS_X_OFF + 32>(xb[0], x_off, base, diag);
    sk_lookup<SBASE>(A0, w1.z, w2.z, lane_off, base);
    sk_mma(acc[0], A1[0], A1[1], A1[2], A1[3], xb[1].x, xb[1].y);
    sk_mma(acc[1], A1[4], A1[5], A1[6], A1[7], xb[1].z, xb[1].w);
    sk_ldx<SBASE, WS_X_OFF + 48>(xb[1], x_off, base, diag);
    sk_lookup<SBASE>(A1, w1.w, w2.w, lane_off, base);
    if (more) {
        w1 = next.template load1<NEXT_IMM>();
        w2 = next.template load2<NEXT_IMM>();
    }
    sk_mma(acc[0], A0[0], A0[1], A0[2], A0[3], xb[0].x, xb[0].y);
    sk_mma(acc[1], A0[4], A0[5], A0[6], A0[7], xb[0].z, xb[0].w);
    sk_mma(acc[0], A1[0], A1[1], A1[2], A1[3], xb[1].x, xb[1].y);
    sk_mma(acc[1], A1[4], A1[5], A1[6], A1[7], xb[1].z, xb[1].w);
}

// ---- compute warps --------------------------------------------------------------------------------
template <int SBASE>
__device__ __forceinline__ void ws_compute(const SkArgs &a, uint8_t *smem, uint32_t smem_base, uint32_t u_begin,
                                           uint32_t u_end, uint32_t cw, uint32_t lane, volatile uint32_t *err_flag) {
    const uint32_t nc = a.n_chunks;
    const uint32_t bar_full = smem_base + WS_BAR_OFF, bar_empty = bar_full + 16;
    const uint32_t diag = ((lane >> 2) == (lane & 3)) ? 1u : 0u;  // lanes 0, 5, 10, 15 carry x in the B operand
    uint4 xb[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    WsWalk walk;
    walk.init(u_begin, u_end, nc, WS_STAGE_CHUNKS);
    for (uint32_t t = 0; walk.next(); t++) {
        const WsStage &st = walk.cur;
        const uint32_t xbuf = t & 1, par = (t >> 1) & 1, tb = st.seg & 1;
        const uint32_t hb1 = a.hb_mul * st.blk, hb2 = hb1 + a.hb_add2;
        const uint32_t span = st.pe - st.pb;
        const uint32_t nj = span > cw ? (span - cw + WS_NC - 1) / WS_NC : 0;  // this warp: chunks pb + cw + WS_NC*j
        SkSrcPtr src;
        src.p = a.idx1 + ((size_t)hb1 * nc + st.pb + cw) * 512 + lane * 16;
        src.d2 = (uint64_t)(reinterpret_cast<uintptr_t>(a.idx2 + ((size_t)hb2 * nc + st.pb + cw) * 512 + lane * 16) -
                            reinterpret_cast<uintptr_t>(src.p));
        // first chunks in flight before the stage's table and x are waited for
        uint4 q1[WS_PF], q2[WS_PF];
#define WS_LOAD(I)                                                              \
    if ((I) < WS_PF && (I) < nj) {                                              \
        q1[(I) % WS_PF] = src.load1<((I) % WS_PF) * WS_NC * 512>();             \
        q2[(I) % WS_PF] = src.load2<((I) % WS_PF) * WS_NC * 512>();             \
    }
        WS_LOAD(0) WS_LOAD(1) WS_LOAD(2) WS_LOAD(3)
#undef WS_LOAD
        src.advance(WS_PF * WS_NC * 512);  // from here on: the chunk WS_PF steps ahead
        if (t == 0) {  // with the first index chunks in flight: this warp's share of the first pair table
            ws_first_table(a, reinterpret_cast<uint32_t *>(smem + (st.seg & 1) * WS_TBL_BYTES), st.blk, cw, WS_NC, lane);
            asm volatile("bar.sync 2, %0;\n" ::"n"(WS_NC * 32) : "memory");  // the compute warps only: they are the table's readers
        }
        if (st.first) {
#pragma unroll
            for (int i = 0; i < 2; i++) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
        }
        // The first stage's x comes after the builders' dependency wait, which lasts as long as the kernel before
        // this one -- under tensor parallelism as long as a late peer.  The bounded hand-over wait must not run
        // during that time: wait for the same dependency first.
        if (t == 0) pdl_wait();
        ws_wait(bar_full + 8 * xbuf, par, err_flag);
        const uint32_t lane_off = lane * 4 | (tb << 16);
        uint32_t x_off = xbuf * WS_X_BYTES + cw * 64;
#define WS_STEP(I)                                                                                            \
    if ((I) < WS_PF && ((I) == 0 || j + (I) < nj))                                                            \
        ws_chunk<SBASE, ((I) % WS_PF) * WS_NC * 512>(acc, q1[(I) % WS_PF], q2[(I) % WS_PF], xb, lane_off,         \
                                                     x_off + ((I) % WS_PF) * WS_NC * 64, diag, smem_base, src, \
                                                     j + (I) + WS_PF < nj);
        for (uint32_t j = 0; j < nj; j += WS_PF) {
            WS_STEP(0) WS_STEP(1) WS_STEP(2) WS_STEP(3)
            x_off += WS_PF * WS_NC * 64;
            src.advance(WS_PF * WS_NC * 512);
        }
#undef WS_STEP
        if (st.last) {
            // accumulator column n = 2q, 2q+1 (q = lane%4) of MMA row g = lane/4 (and g+8): column n is
            // the dot product of the lane (g, n); only n < 4 is populated.
            if ((lane & 3) < 2) {
                const uint32_t r = (lane >> 2) * 4 + (lane & 3) * 2;  // lane index the column belongs to
                float *rw = reinterpret_cast<float *>(smem + WS_RED_OFF) + (tb * WS_NC + cw) * 64;
                rw[r] = acc[0][0] + acc[1][0];
                rw[r + 1] = acc[0][1] + acc[1][1];
                rw[32 + r] = acc[0][2] + acc[1][2];
                rw[32 + r + 1] = acc[0][3] + acc[1][3];
            }
        }
        t5::mbar_arrive(bar_empty + 8 * xbuf);  // every lane: its reads of the buffers and its sums are done
    }
}

// ---- builder warps ---------------------------------------------------------------------------------
// Adds the compute warps' sums of a finished segment and writes the block's outputs, or leaves the
// partial sums and, when this CTA completes the block, adds every contributor's in range order.
template <int MODE>
__device__ __forceinline__ void ws_finish(const SkArgs &a, uint8_t *smem, const WsStage &st, uint32_t bt, uint32_t cta,
                                          uint32_t G, uint32_t bat, TpWarpList &wl) {
    const uint32_t nc = a.n_chunks, blk = st.blk, tb = st.seg & 1;
    const uint32_t hb1 = a.hb_mul * blk, hb2 = hb1 + a.hb_add2;
    const float *red = reinterpret_cast<const float *>(smem + WS_RED_OFF) + tb * WS_NC * 64;
    float *fin = reinterpret_cast<float *>(smem + WS_FIN_OFF);           // [128] floats
    uint32_t *list = reinterpret_cast<uint32_t *>(smem + WS_FIN_OFF) + 128;  // [128] contributor slots
    unsigned int &s_last = *reinterpret_cast<unsigned int *>(smem + WS_BAR_OFF + 40);
    float sum = 0.0f;  // thread bt < 64: rows "1" (bt < 32) or "2", lane bt & 31
    if (bt < 64) {
#pragma unroll
        for (int w = 0; w < WS_NC; w++) sum += red[w * 64 + bt];
    }
    const uint32_t span = st.ce - st.cb;
    if (span != nc) {
        float *part = a.partials + (size_t)bat * G * 128;
        if (bt < 64) part[((size_t)cta * 2 + (st.cb > 0 ? 0 : 1)) * 64 + bt] = sum;
        ws_bar_builders();
        if (bt == 0) {
            unsigned int *ctr = a.counters + (size_t)bat * a.n_blocks + blk;
            const unsigned int prev = sk_arrive(ctr, span);
            s_last = (prev + span == nc) ? 1u : 0u;
            if (s_last) *ctr = 0;  // ready for the next launch on this stream
        }
        ws_bar_builders();
        if (!s_last) return;
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
        const uint32_t c = c0 + bt;
        const uint32_t r0 = c < G ? sk_boundary_in_block(p, c, b0) : b1;
        const uint32_t r1 = c < G ? sk_boundary_in_block(p, c + 1, b0) : b1;
        list[bt] = (r1 > r0) ? (c * 2 + (r0 > b0 ? 0u : 1u)) : 0xFFFFFFFFu;
        const uint32_t n = ws_bar_builders_count(c < G && r0 < b1);
        // thread (g, t): contributors g, g+2, ... of output t, four loads in flight
        const uint32_t g = bt >> 6, t = bt & 63;
        float ps = 0.0f;
        for (uint32_t k = g; k < n; k += 8) {
            float v[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const uint32_t slot = (k + 2 * e < n) ? list[k + 2 * e] : 0xFFFFFFFFu;
                v[e] = (slot != 0xFFFFFFFFu) ? __ldcg(part + (size_t)slot * 64 + t) : 0.0f;
            }
#pragma unroll
            for (int e = 0; e < 4; e++) ps += v[e];
        }
        fin[g * 64 + t] = ps;
        ws_bar_builders();
        if (bt < 64) sum = fin[bt] + fin[64 + bt];
        ws_bar_builders();  // fin is reused by the epilogue below
    }
    if (MODE == GEMV_SWIGLU) {
        // rows "1" are gate rows, rows "2" the up rows of the same output index
        if (bt < 64) fin[bt] = sum;
        ws_bar_builders();
        if (bt < 32) {
            const uint32_t row = blk * 32 + bt;
            if (row < a.m) {
                const float gv = __half2float(__float2half_rn(fin[bt]));
                const float uv = __half2float(__float2half_rn(fin[32 + bt]));
                const float sv = __half2float(__float2half_rn(gv / (1.0f + expf(-gv))));
                a.y[(size_t)bat * a.y_stride + row] = __half_as_ushort(__float2half_rn(sv * uv));
            }
        }
        ws_bar_builders();  // fin may be rewritten by the next segment's finish
    } else if (MODE == GEMV_TP) {
        if (bt < 64) tp_deliver_listed(a.tp, wl, (bt >> 5) ? hb2 : hb1, bt & 31, sum, a.m, a.y + (size_t)bat * a.y_stride, a.err);
    } else if (bt < 64) {
        const uint32_t row = ((bt >> 5) ? hb2 : hb1) * 32 + (bt & 31);
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

template <int MODE>
__device__ __forceinline__ void ws_build(const SkArgs &a, uint8_t *smem, uint32_t smem_base, uint32_t u_begin,
                                         uint32_t u_end, uint32_t bt, uint32_t cta, uint32_t G, uint32_t bat,
                                         volatile uint32_t *err_flag) {
    const uint32_t nc = a.n_chunks, lane = bt & 31, bw = bt >> 5;
    const uint32_t bar_full = smem_base + WS_BAR_OFF, bar_empty = bar_full + 16;
    float &s_inv = *reinterpret_cast<float *>(smem + WS_BAR_OFF + 36);
    float *fin = reinterpret_cast<float *>(smem + WS_FIN_OFF);
    const uint16_t *xrow = a.x + (size_t)bat * a.x_stride;
    float inv = 1.0f;
    bool waited = false;
    WsStage hist[2];  // the two stages in flight, by buffer
    // GEMV_TP: what builder warps 0 and 1 have delivered to the peers, finished after the CTA's last stage
    TpWarpList wl{reinterpret_cast<uint16_t *>(smem + WS_TPL_OFF) + (bw & 1) * TP_LIST_MAX, 0};
    WsWalk walk;
    walk.init(u_begin, u_end, nc, WS_STAGE_CHUNKS);
    uint32_t t = 0;
    for (; walk.next(); t++) {
        const WsStage st = walk.cur;
        const uint32_t xbuf = t & 1, tb = st.seg & 1;
        if (t >= 2) {
            // the compute warps are done with stage t-2: its buffers are free, its sums (if it
            // closed a segment) are in place
            ws_wait(bar_empty + 8 * xbuf, ((t - 2) >> 1) & 1, err_flag);
            if (hist[xbuf].last) ws_finish<MODE>(a, smem, hist[xbuf], bt, cta, G, bat, wl);
        }
        hist[xbuf] = st;
        bool staged = false;
        if (t == 0) {
            // the first block's table is the compute warps' job (ws_first_table)
        } else if (st.first) {
            // pair tables: entry e = lo | hi<<4 -> half2{pal[lo], pal[hi]}; builder warp w writes the
            // entries with hi = w, w + WS_NB, ...; lane L writes its own bank.
            const uint32_t hb1 = a.hb_mul * st.blk, hb2 = hb1 + a.hb_add2;
            uint32_t *tbl = reinterpret_cast<uint32_t *>(smem + tb * WS_TBL_BYTES);
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const uint32_t row = (h == 0 ? hb1 : hb2) * 32 + lane;
                const uint16_t *prow = (h == 0 ? a.pal1 : a.pal2) + (size_t)row * 16;
                const uint4 p0 = *reinterpret_cast<const uint4 *>(prow);
                const uint4 pp = *reinterpret_cast<const uint4 *>(prow + 8);
                const uint32_t cbp[8] = {p0.x, p0.y, p0.z, p0.w, pp.x, pp.y, pp.z, pp.w};
                for (uint32_t hi = bw; hi < 16; hi += WS_NB) {
                    const uint32_t hi_pair = reinterpret_cast<const uint32_t *>(prow)[hi >> 1];  // {pal[hi&~1], pal[hi|1]}
                    const uint32_t hsel = (hi & 1) ? 0x7600u : 0x5400u;
#pragma unroll
                    for (int lo = 0; lo < 16; lo++) {
                        const uint32_t v = __byte_perm(cbp[lo >> 1], hi_pair, hsel | ((lo & 1) ? 0x32u : 0x10u));
                        tbl[((uint32_t)lo + 16u * hi) * 64 + h * 32 + lane] = v;
                    }
                }
            }
        }
        if (!waited) {
            // Everything above reads only weights.  x, the partial sums, the counters and y belong to
            // the stream order: wait for the kernels before this one.
            pdl_wait();
            waited = true;
            // RMSNorm folded into the staging (rms_norm_inplace, src/lut/cpu_fallback.rs:39-54): every CTA
            // sums the squares of the whole row once (a few KB from L2) and scales the slices it stages.
            if (a.norm_n) {
                // rows of up to 8192 values are read once: kept in registers between the sum of
                // squares and the scaling of this first stage's slice
                const uint4 *xr = reinterpret_cast<const uint4 *>(xrow);
                const uint32_t n16row = a.norm_n / 8;
                const bool one_pass = n16row <= 8 * WS_BTHREADS;
                uint4 keep[8];
                float ss = 0.0f;
                if (one_pass) {
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        const uint32_t i = bt + e * WS_BTHREADS;
                        keep[e] = i < n16row ? xr[i] : make_uint4(0, 0, 0, 0);
                    }
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        const __half2 *hp = reinterpret_cast<const __half2 *>(&keep[e]);
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            const float2 f = __half22float2(hp[q]);
                            ss += f.x * f.x + f.y * f.y;
                        }
                    }
                } else {
                    for (uint32_t i = bt; i < n16row; i += WS_BTHREADS) {
                        const uint4 v = xr[i];
                        const __half2 *hp = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            const float2 f = __half22float2(hp[q]);
                            ss += f.x * f.x + f.y * f.y;
                        }
                    }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
                if (lane == 0) fin[bw] = ss;
                ws_bar_builders();
                if (bt == 0) {
                    float tot = 0.0f;
                    for (int w = 0; w < WS_NB; w++) tot += fin[w];  // fixed order: the same value in every CTA
                    s_inv = 1.0f / sqrtf(tot / (float)a.norm_n + a.norm_eps);
                }
                ws_bar_builders();
                inv = s_inv;
                if (one_pass) {
                    const uint32_t lo = st.pb * 4, hi = st.pe * 4;  // this stage's slice in 16-byte units of the row
                    uint4 *xd = reinterpret_cast<uint4 *>(smem + WS_X_OFF + xbuf * WS_X_BYTES);
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        const uint32_t i = bt + e * WS_BTHREADS;
                        if (i >= lo && i < hi) {
                            uint4 v = keep[e];
                            __half2 *hp = reinterpret_cast<__half2 *>(&v);
#pragma unroll
                            for (int q = 0; q < 4; q++) {
                                const float2 f = __half22float2(hp[q]);
                                hp[q] = __floats2half2_rn(f.x * inv, f.y * inv);
                            }
                            xd[i - lo] = v;
                        }
                    }
                    staged = true;
                }
            }
        }
        // this stage's slice of x (fp16, normalised on the way if asked)
        if (!staged) {
            const uint32_t n16 = (st.pe - st.pb) * 4;  // 16-byte units
            const uint4 *xg = reinterpret_cast<const uint4 *>(xrow + (size_t)st.pb * 32);
            uint4 *xd = reinterpret_cast<uint4 *>(smem + WS_X_OFF + xbuf * WS_X_BYTES);
            // four 16-byte loads per thread in flight before the first store
            for (uint32_t i0 = bt; i0 < n16; i0 += 4 * WS_BTHREADS) {
                uint4 v[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const uint32_t i = i0 + e * WS_BTHREADS;
                    v[e] = i < n16 ? xg[i] : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const uint32_t i = i0 + e * WS_BTHREADS;
                    if (i >= n16) continue;
                    if (a.norm_n != 0) {
                        __half2 *hp = reinterpret_cast<__half2 *>(&v[e]);
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            const float2 f = __half22float2(hp[q]);
                            hp[q] = __floats2half2_rn(f.x * inv, f.y * inv);
                        }
                    }
                    xd[i] = v[e];
                }
            }
        }
        t5::mbar_arrive(bar_full + 8 * xbuf);  // every builder thread: its table entries and x words are stored
    }
    // retire the last two stages in order
    const uint32_t n_stages = t;
    for (uint32_t r = (n_stages >= 2 ? n_stages - 2 : 0); r < n_stages; r++) {
        const uint32_t xbuf = r & 1;
        ws_wait(bar_empty + 8 * xbuf, (r >> 1) & 1, err_flag);
        if (hist[xbuf].last) ws_finish<MODE>(a, smem, hist[xbuf], bt, cta, G, bat, wl);
    }
    if (MODE == GEMV_TP && bt < 64) tp_finish(a.tp, tp_epoch(a.tp), wl.list, wl.n, bt & 31, a.m, a.y + (size_t)bat * a.y_stride, a.err);
}

template <int MODE, int SBASE>
__global__ void __launch_bounds__(WS_THREADS, 1) lut_gemv_ws_kernel(const SkArgs a) {
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
    if (SBASE >= 0 && smem_base != (uint32_t)SBASE) {  // layout assumption broken: refuse to compute
        if (threadIdx.x == 0) atomicExch(a.err, 1u);
        return;
    }
    pdl_launch_dependents();
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t cta = blockIdx.x, G = gridDim.x, bat = blockIdx.y;
    const uint32_t u_begin = sk_boundary(a.part, cta);
    const uint32_t u_end = sk_boundary(a.part, cta + 1);
    if (u_begin >= u_end) return;
    volatile uint32_t *err_flag = reinterpret_cast<volatile uint32_t *>(smem + WS_BAR_OFF + 32);
    if (tid == 0) {
        const uint32_t bar = smem_base + WS_BAR_OFF;
        t5::mbar_init(bar + 0, WS_BTHREADS);
        t5::mbar_init(bar + 8, WS_BTHREADS);
        t5::mbar_init(bar + 16, WS_NC * 32);
        t5::mbar_init(bar + 24, WS_NC * 32);
        *err_flag = 0;
    }
    __syncthreads();
    if (warp < WS_NC) {
        ws_compute<SBASE>(a, smem, smem_base, u_begin, u_end, warp, lane, err_flag);
    } else {
        ws_build<MODE>(a, smem, smem_base, u_begin, u_end, tid - WS_NC * 32, cta, G, bat, err_flag);
        if (*err_flag && tid == WS_NC * 32) atomicExch(a.err, 2u);  // a hand-over wait gave up
    }
}

template <int MODE, int SBASE>
static int launch_ws_v(prism_cuda_ctx *ctx, const SkArgs &a, dim3 grid) {
    static bool configured[PRISM_MAX_DEVICES] = {false};
    if (!configured[ctx->device]) {
        PRISM_CUDA_TRY(ctx, cudaFuncSetAttribute(lut_gemv_ws_kernel<MODE, SBASE>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)WS_SMEM_BYTES));
        configured[ctx->device] = true;
    }
    launch_pdl(ctx, "lut_gemv_ws_kernel", lut_gemv_ws_kernel<MODE, SBASE>, grid, WS_THREADS, WS_SMEM_BYTES, a);
    return after_launch(ctx, "lut_gemv_ws_kernel");
}

template <int MODE>
static int launch_ws(prism_cuda_ctx *ctx, const SkArgs &a, dim3 grid) {
    if (ctx->smem_base == WS_KNOWN_SBASE) return launch_ws_v<MODE, WS_KNOWN_SBASE>(ctx, a, grid);
    return launch_ws_v<MODE, -1>(ctx, a, grid);
}

bool ws_eligible(const LutTensor &t) { return t.bits == 4 && t.k % 32 == 0 && t.k >= 32; }

// The pipeline pays off when a CTA has several stages of some length: rows of at least 64 chunks
// and enough work for the contiguous, balanced partition.
bool ws_preferred(prism_cuda_ctx *ctx, const LutTensor &t, bool swiglu, uint32_t batch) {
    if (!ws_eligible(t) || t.n_chunks < 64) return false;
    const uint32_t n_blocks = swiglu ? t.n_hb : t.n_hb / 2;
    uint32_t slots = (uint32_t)ctx->sm_count / (batch ? batch : 1);
    if (slots == 0) slots = 1;
    return (uint64_t)n_blocks * t.n_chunks / slots >= (uint64_t)ctx->sk_stream_chunks;
}

// Chooses the partition (see SkPart) for one activation vector of a batch: one CTA per SM.
SkPart ws_partition(prism_cuda_ctx *ctx, uint32_t n_blocks, uint32_t n_chunks, uint32_t batch, uint32_t fill_pct) {
    // Fewer blocks than CTAs, but at least fill_pct per 100, and rows short enough that a block is a few
    // microseconds of streaming: one whole block per CTA on n_blocks CTAs.  The idle SMs cost less than what
    // every CTA otherwise pays for covering parts of two blocks (a second table, partial sums, the arrival and
    // the fix-up at the end): measured down to 54 blocks per 100 SMs for one activation row (10240x8192 cut
    // in two: 11.2 -> 10.9 us; 2 x 3696 x 8192, 78 per 100: 13.6 -> 11.7 us).
    const uint32_t slots = ws_choose_slots(n_blocks, n_chunks, (uint32_t)ctx->sm_count / (batch ? batch : 1),
                                           (uint32_t)ctx->ws_whole_blocks, fill_pct);
    return sk_choose_partition(n_blocks, n_chunks, slots, (uint32_t)ctx->sk_stream_chunks, (uint32_t)ctx->sk_min_chunks, 96);
}

int launch_gemv_ws(prism_cuda_ctx *ctx, GemvMode mode, const LutTensor &t, const LutTensor *t2, const uint16_t *x,
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
    a.part = ws_partition(ctx, a.n_blocks, a.n_chunks, batch, (uint32_t)ctx->ws_whole_fill);
    const uint32_t G = a.part.G;
    PRISM_TRY(ensure_splitk(ctx, (size_t)batch * G * 128, (size_t)batch * a.n_blocks));
    a.partials = ctx->splitk_partials;
    a.counters = ctx->splitk_counters;
    const dim3 grid(G, batch);
    switch (mode) {
    case GEMV_PLAIN: return launch_ws<GEMV_PLAIN>(ctx, a, grid);
    case GEMV_RESID: return launch_ws<GEMV_RESID>(ctx, a, grid);
    case GEMV_F32: return launch_ws<GEMV_F32>(ctx, a, grid);
    case GEMV_TP:
        PRISM_TRY(tp_fill_push(ctx, t, &a.tp));
        return launch_ws<GEMV_TP>(ctx, a, grid);
    default: return launch_ws<GEMV_SWIGLU>(ctx, a, grid);
    }
}

}  // namespace prism

