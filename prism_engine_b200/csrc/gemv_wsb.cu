// Palettized GEMV for a small batch of activation vectors (2..8 sequences decoded together): the
// warp-specialised pair-table kernel of gemv_ws.cu with the batch in the N dimension of the MMA.
//
// Y[b] = W x[b] (lut_gemv_cpu, src/lut/cpu_fallback.rs:12-35, once per sequence; the reference's
// prefill_cpu, engine_impl.rs:1046-1053, is the same loop).  The weights are streamed ONCE for the
// whole batch: the looked-up half2 pairs are the A fragments of mma.sync.m16n8k16 as in the
// single-vector kernel, and each A fragment is multiplied by NBP B fragments.  A B fragment serves
// two sequences: columns 0..3 carry x of sequence 2p on lanes 0, 5, 10, 15, columns 4..7 carry x of
// sequence 2p+1 on lanes 16, 21, 26, 31, so accumulator column n of MMA row g is the dot product of
// lane (g, n % 4) with sequence 2p + n / 4.  Table lookups and index loads per weight are those of
// batch 1; only the x fragments (16 bytes per lane, sequence pair and index word) grow with it.
//
// Pipeline, partition and partial-sum fix-up are those of lut_gemv_ws_kernel (16 or 12 compute warps,
// 4 builder warps, two pair-table buffers, two x buffers).  The per-warp sums of a finished block
// go through one buffer guarded by its own mbarrier.  RMSNorm is not folded in here: the caller
// passes normalised rows.
#include "common.cuh"
#include "pair_table.cuh"
#include "tc5_ptx.cuh"
#include "ws_common.cuh"

namespace prism {


constexpr int WB_NC_MAX = 16;                    // compute warps: 16 for one or two sequence pairs, 12 (more registers) for three or four
constexpr int WB_NB = 4;                         // builder warps
static_assert(WB_NB * 32 == WS_COMMON_BTHREADS, "builder barrier size");
constexpr int WB_PF = 2;                         // index chunks in flight per compute warp
constexpr int WB_TBL_BYTES = 65536;
constexpr int WB_X_OFF = 2 * WB_TBL_BYTES;
constexpr int WB_X_BYTES = 24 * 1024;            // one x buffer: stage chunks x 64 B x padded batch
constexpr int WB_RED_OFF = WB_X_OFF + 2 * WB_X_BYTES;        // [compute warps][padded batch][64] floats
constexpr int WB_RED_BYTES = WB_NC_MAX * 8 * 64 * 4;
constexpr int WB_FIN_OFF = WB_RED_OFF + WB_RED_BYTES;         // builder scratch: 128 floats + 128 slots + 8*64 sums
constexpr int WB_FIN_BYTES = (128 + 128 + 8 * 64) * 4;
constexpr int WB_BAR_OFF = WB_FIN_OFF + WB_FIN_BYTES;         // full[2], empty[2], red_free, flags
constexpr size_t WB_SMEM_BYTES = WB_BAR_OFF + 64;
constexpr int WB_KNOWN_SBASE = 1024;

// chunks of x per stage for NBP sequence pairs: the x buffer holds 2*NBP rows of them
template <int NBP>
struct WbGeom {
    static constexpr int NB = 2 * NBP;                       // padded batch
    static constexpr int NC = NBP <= 2 ? 16 : 12;            // compute warps
    static constexpr int THREADS = (NC + WB_NB) * 32;
    static constexpr int SC = WB_X_BYTES / (64 * NB);        // 192, 96, 64 (3 pairs), 48
    static constexpr int ROW_BYTES = SC * 64;                // bytes of one sequence's slice in an x buffer
};

struct WbArgs {
    SkArgs g;             // the single-vector arguments: x/y are the first sequence's rows, strides apply
    uint32_t batch;       // sequences (<= 2*NBP)
};

// One 32-weight chunk of the two half-blocks against NBP sequence pairs.  The x fragments of index
// word h+1 are requested before the tensor-core steps of word h, the table lookups of the next
// word in between, so neither kind of shared-memory load is waited for right after it is issued.
template <int SBASE, int NBP, int H>
__device__ __forceinline__ void wb_ldx_all(uint4 (&xb)[NBP], uint32_t x_off, uint32_t base, uint32_t diag) {
    constexpr int RB = 2 * WbGeom<NBP>::ROW_BYTES;  // bytes between sequence pairs in the x buffer
#pragma unroll
    for (int p = 0; p < NBP; p++) sk_ldx<SBASE, WB_X_OFF + 16 * H>(xb[p], x_off + p * RB, base, diag);
}
template <int NBP>
__device__ __forceinline__ void wb_mma_all(float (&acc)[NBP][2][4], const uint32_t (&A)[8], const uint4 (&xb)[NBP]) {
#pragma unroll
    for (int p = 0; p < NBP; p++) {
        sk_mma(acc[p][0], A[0], A[1], A[2], A[3], xb[p].x, xb[p].y);
        sk_mma(acc[p][1], A[4], A[5], A[6], A[7], xb[p].z, xb[p].w);
    }
}
// NEXT_IMM >= 0: the chunk two steps ahead inside the same stage is requested from `next` (when
// `more`); NEXT_IMM < 0: the request goes through the cross-stage cursor `pf`.
template <int SBASE, int NBP, int NEXT_IMM>
__device__ __forceinline__ void wb_chunk(float (&acc)[NBP][2][4], uint4 &w1, uint4 &w2, uint4 (&xb)[NBP],
                                         uint32_t lane_off, uint32_t x_off, uint32_t diag, uint32_t base,
                                         WsPrefetch &pf, const SkSrcPtr &next, bool more) {
    uint32_t A0[8], A1[8];
    sk_lookup<SBASE>(A0, w1.x, w2.x, lane_off, base);
    wb_ldx_all<SBASE, NBP, 0>(xb, x_off, base, diag);
    sk_lookup<SBASE>(A1, w1.y, w2.y, lane_off, base);
    wb_mma_all<NBP>(acc, A0, xb);
    wb_ldx_all<SBASE, NBP, 1>(xb, x_off, base, diag);
    sk_lookup<SBASE>(A0, w1.z, w2.z, lane_off, base);
    wb_mma_all<NBP>(acc, A1, xb);
    wb_ldx_all<SBASE, NBP, 2>(xb, x_off, base, diag);
    sk_lookup<SBASE>(A1, w1.w, w2.w, lane_off, base);
    // w1/w2 are dead from here: they take the chunk two steps ahead
    if (NEXT_IMM >= 0) {
        if (more) {
            w1 = next.template load1<(NEXT_IMM >= 0 ? NEXT_IMM : 0)>();
            w2 = next.template load2<(NEXT_IMM >= 0 ? NEXT_IMM : 0)>();
        }
    } else if (pf.valid) {
        w1 = pf.src.load1<0>();
        w2 = pf.src.load2<0>();
    }
    wb_mma_all<NBP>(acc, A0, xb);
    wb_ldx_all<SBASE, NBP, 3>(xb, x_off, base, diag);
    wb_mma_all<NBP>(acc, A1, xb);
    if (NEXT_IMM < 0 && pf.valid) pf.advance();
}

// ---- compute warps --------------------------------------------------------------------------------
template <int SBASE, int NBP>
__device__ __forceinline__ void wb_compute(const SkArgs &a, uint8_t *smem, uint32_t smem_base, uint32_t u_begin,
                                           uint32_t u_end, uint32_t cw, uint32_t lane, volatile uint32_t *err_flag) {
    using Geo = WbGeom<NBP>;
    const uint32_t nc = a.n_chunks;
    const uint32_t bar_full = smem_base + WB_BAR_OFF, bar_empty = bar_full + 16, bar_red = bar_full + 32;
    // lanes whose B-operand slot is non-zero: 0, 5, 10, 15 (first sequence of a pair), 16, 21, 26, 31 (second)
    const uint32_t diag = ((lane & 3) == ((lane >> 2) & 3)) ? 1u : 0u;
    uint4 xb[NBP];
#pragma unroll
    for (int p = 0; p < NBP; p++) xb[p] = make_uint4(0, 0, 0, 0);
    float acc[NBP][2][4];
    static_assert(WB_PF == 2, "the ring below has two slots");
    // Three or four sequence pairs: stages are short (48..64 chunks), so the two chunks in flight are
    // requested continuously over the stages (slot 0 holds the chunk consumed next).  One or two
    // pairs: stages are long and the cheaper per-stage ring is used.
    constexpr bool CONT = NBP > 2;
    WsWalk walk;
    walk.init(u_begin, u_end, nc, Geo::SC);
    WsPrefetch pf;
    pf.valid = false;
    uint4 q1[2], q2[2];
    if (CONT) {
        pf.init(&a, u_begin, u_end, Geo::SC, cw, Geo::NC, lane);
#pragma unroll
        for (int i = 0; i < 2; i++) {
            if (pf.valid) {
                q1[i] = pf.src.load1<0>();
                q2[i] = pf.src.load2<0>();
                pf.advance();
            }
        }
    }
    uint32_t segs_done = 0;
    for (uint32_t t = 0; walk.next(); t++) {
        const WsStage &st = walk.cur;
        const uint32_t xbuf = t & 1, par = (t >> 1) & 1, tb = st.seg & 1;
        const uint32_t span = st.pe - st.pb;
        const uint32_t nj = span > cw ? (span - cw + Geo::NC - 1) / Geo::NC : 0;  // this warp: chunks pb + cw + NC*j
        SkSrcPtr src;
        src.p = nullptr; src.d2 = 0;
        if (!CONT) {
            const uint32_t hb1 = a.hb_mul * st.blk, hb2 = hb1 + a.hb_add2;
            src.p = a.idx1 + ((size_t)hb1 * nc + st.pb + cw) * 512 + lane * 16;
            src.d2 = (uint64_t)(reinterpret_cast<uintptr_t>(a.idx2 + ((size_t)hb2 * nc + st.pb + cw) * 512 + lane * 16) -
                                reinterpret_cast<uintptr_t>(src.p));
            if (0 < nj) { q1[0] = src.load1<0>(); q2[0] = src.load2<0>(); }
            if (1 < nj) { q1[1] = src.load1<Geo::NC * 512>(); q2[1] = src.load2<Geo::NC * 512>(); }
            src.advance(2 * Geo::NC * 512);  // from here on: the chunk two steps ahead
        }
        if (t == 0) {  // with the first index chunks in flight: the first block's pair table (see ws_first_table)
            ws_first_table(a, reinterpret_cast<uint32_t *>(smem + tb * WB_TBL_BYTES), st.blk, cw, Geo::NC, lane);
            asm volatile("bar.sync 2, %0;\n" ::"n"(Geo::NC * 32) : "memory");
        }
        if (st.first) {
#pragma unroll
            for (int p = 0; p < NBP; p++)
#pragma unroll
                for (int i = 0; i < 2; i++) acc[p][i][0] = acc[p][i][1] = acc[p][i][2] = acc[p][i][3] = 0.f;
        }
        // The first stage's x comes after the builders' dependency wait, which lasts as long as the kernel before
        // this one -- under tensor parallelism as long as a late peer.  The bounded hand-over wait must not run
        // during that time: wait for the same dependency first.
        if (t == 0) pdl_wait();
        ws_wait(bar_full + 8 * xbuf, par, err_flag);
        const uint32_t lane_off = lane * 4 | (tb << 16);
        uint32_t x_off = xbuf * WB_X_BYTES + (lane >> 4) * Geo::ROW_BYTES + cw * 64;
        if (CONT) {
            for (uint32_t j = 0; j < nj; j += 2) {
                wb_chunk<SBASE, NBP, -1>(acc, q1[0], q2[0], xb, lane_off, x_off, diag, smem_base, pf, src, false);
                if (j + 1 < nj)
                    wb_chunk<SBASE, NBP, -1>(acc, q1[1], q2[1], xb, lane_off, x_off + Geo::NC * 64, diag, smem_base, pf, src, false);
                x_off += 2 * Geo::NC * 64;
            }
            if (nj & 1) {  // an odd count leaves the next chunk in slot 1: rotate the ring
                const uint4 t1 = q1[0], t2 = q2[0];
                q1[0] = q1[1]; q2[0] = q2[1];
                q1[1] = t1; q2[1] = t2;
            }
        } else {
            for (uint32_t j = 0; j < nj; j += 2) {
                wb_chunk<SBASE, NBP, 0>(acc, q1[0], q2[0], xb, lane_off, x_off, diag, smem_base, pf, src, j + 2 < nj);
                if (j + 1 < nj)
                    wb_chunk<SBASE, NBP, Geo::NC * 512>(acc, q1[1], q2[1], xb, lane_off, x_off + Geo::NC * 64, diag, smem_base,
                                                        pf, src, j + 3 < nj);
                x_off += 2 * Geo::NC * 64;
                src.advance(2 * Geo::NC * 512);
            }
        }
        if (st.last) {
            // the builders have read the sums of the segment before this one
            if (segs_done > 0) ws_wait(bar_red, (segs_done - 1) & 1, err_flag);
            // lane (g, t): accumulator columns 2t, 2t+1 of MMA rows g (half-block 1) and g+8 (half-block 2):
            // column n belongs to lane 4g + n%4 and to sequence 2p + n/4
            const uint32_t r = (lane >> 2) * 4 + (lane & 1) * 2;
            float *red = reinterpret_cast<float *>(smem + WB_RED_OFF) + (size_t)cw * Geo::NB * 64;
#pragma unroll
            for (int p = 0; p < NBP; p++) {
                float *rw = red + (2 * p + ((lane >> 1) & 1)) * 64;
                rw[r] = acc[p][0][0] + acc[p][1][0];
                rw[r + 1] = acc[p][0][1] + acc[p][1][1];
                rw[32 + r] = acc[p][0][2] + acc[p][1][2];
                rw[32 + r + 1] = acc[p][0][3] + acc[p][1][3];
            }
            segs_done++;
        }
        t5::mbar_arrive(bar_empty + 8 * xbuf);  // every lane: its reads of the buffers and its sums are done
    }
}

// ---- builder warps ---------------------------------------------------------------------------------
// Adds the compute warps' sums of a finished segment for every sequence and writes the block's
// outputs, or leaves the partial sums and, when this CTA completes the block, adds every
// contributor's in range order.
template <int MODE, int NBP>
__device__ __forceinline__ void wb_finish(const WbArgs &wa, uint8_t *smem, uint32_t smem_base, const WsStage &st,
                                          uint32_t bt, uint32_t cta, uint32_t G) {
    using Geo = WbGeom<NBP>;
    const SkArgs &a = wa.g;
    const uint32_t nc = a.n_chunks, blk = st.blk, B = wa.batch;
    const uint32_t hb1 = a.hb_mul * blk, hb2 = hb1 + a.hb_add2;
    const float *red = reinterpret_cast<const float *>(smem + WB_RED_OFF);
    float *fin = reinterpret_cast<float *>(smem + WB_FIN_OFF);                  // [128] floats
    uint32_t *list = reinterpret_cast<uint32_t *>(smem + WB_FIN_OFF) + 128;     // [128] contributor slots
    float *sums = reinterpret_cast<float *>(smem + WB_FIN_OFF) + 256;           // [8][64] block sums per sequence
    unsigned int &s_last = *reinterpret_cast<unsigned int *>(smem + WB_BAR_OFF + 48);
    // thread (h, t): sequences h, h+2, ... of output t (rows "1": t < 32, rows "2": t >= 32)
    const uint32_t h = bt >> 6, t = bt & 63;
    for (uint32_t b = h; b < (uint32_t)Geo::NB; b += 2) {
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < Geo::NC; w++) s += red[((size_t)w * Geo::NB + b) * 64 + t];
        sums[b * 64 + t] = s;
    }
    ws_bar_builders();
    t5::mbar_arrive(smem_base + WB_BAR_OFF + 32);  // the sum buffer may be rewritten
    const uint32_t span = st.ce - st.cb;
    if (span != nc) {
        // partial slots: [CTA][leading / trailing][sequence][64]
        float *part = a.partials;
        const size_t my = ((size_t)cta * 2 + (st.cb > 0 ? 0 : 1)) * Geo::NB * 64;
        for (uint32_t i = bt; i < B * 64; i += WS_COMMON_BTHREADS) part[my + i] = sums[i];
        ws_bar_builders();
        if (bt == 0) {
            unsigned int *ctr = a.counters + blk;
            const unsigned int prev = sk_arrive(ctr, span);
            s_last = (prev + span == nc) ? 1u : 0u;
            if (s_last) *ctr = 0;  // ready for the next launch on this stream
        }
        ws_bar_builders();
        if (!s_last) return;
        const uint32_t b0 = blk * nc, b1 = b0 + nc;
        const SkPart &p = a.part;
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
        // every contributor in range order, four loads in flight; thread (h, t) as above
        for (uint32_t b = h; b < B; b += 2) {
            float s = 0.0f;
            for (uint32_t k = 0; k < n; k += 4) {
                float v[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const uint32_t slot = (k + e < n) ? list[k + e] : 0xFFFFFFFFu;
                    v[e] = (slot != 0xFFFFFFFFu) ? __ldcg(part + ((size_t)slot * Geo::NB + b) * 64 + t) : 0.0f;
                }
#pragma unroll
                for (int e = 0; e < 4; e++) s += v[e];
            }
            sums[b * 64 + t] = s;
        }
        ws_bar_builders();
    }
    (void)fin;
    // ---- epilogue, one sequence after the other over the 128 builder threads -----------------------
    if (MODE == GEMV_SWIGLU) {
        // rows "1" are gate rows, rows "2" the up rows of the same output index
        for (uint32_t i = bt; i < B * 32; i += WS_COMMON_BTHREADS) {
            const uint32_t b = i >> 5, rr = i & 31, row = blk * 32 + rr;
            if (row < a.m) {
                const float gv = __half2float(__float2half_rn(sums[b * 64 + rr]));
                const float uv = __half2float(__float2half_rn(sums[b * 64 + 32 + rr]));
                const float sv = __half2float(__float2half_rn(gv / (1.0f + expf(-gv))));
                a.y[(size_t)b * a.y_stride + row] = __half_as_ushort(__float2half_rn(sv * uv));
            }
        }
    } else {
        for (uint32_t i = bt; i < B * 64; i += WS_COMMON_BTHREADS) {
            const uint32_t b = i >> 6, rr = i & 63;
            const uint32_t row = ((rr >> 5) ? hb2 : hb1) * 32 + (rr & 31);
            if (row >= a.m) continue;
            const float sum = sums[b * 64 + rr];
            if (MODE == GEMV_F32) {
                reinterpret_cast<float *>(a.y)[(size_t)b * a.y_stride + row] = sum;
            } else {
                __half hv = __float2half_rn(sum);
                if (MODE == GEMV_RESID) {
                    const float r = __half2float(__ushort_as_half(a.resid[(size_t)b * a.y_stride + row]));
                    hv = __float2half_rn(__half2float(hv) + r);
                }
                a.y[(size_t)b * a.y_stride + row] = __half_as_ushort(hv);
            }
        }
    }
    ws_bar_builders();  // `sums` is rewritten by the next segment's finish
}

template <int MODE, int NBP>
__device__ __forceinline__ void wb_build(const WbArgs &wa, uint8_t *smem, uint32_t smem_base, uint32_t u_begin,
                                         uint32_t u_end, uint32_t bt, uint32_t cta, uint32_t G,
                                         volatile uint32_t *err_flag) {
    using Geo = WbGeom<NBP>;
    const SkArgs &a = wa.g;
    const uint32_t nc = a.n_chunks, lane = bt & 31, bw = bt >> 5;
    const uint32_t bar_full = smem_base + WB_BAR_OFF, bar_empty = bar_full + 16;
    bool waited = false;
    WsStage hist[2];  // the two stages in flight, by buffer
    WsWalk walk;
    walk.init(u_begin, u_end, nc, Geo::SC);
    uint32_t t = 0;
    for (; walk.next(); t++) {
        const WsStage st = walk.cur;
        const uint32_t xbuf = t & 1, tb = st.seg & 1;
        if (t >= 2) {
            ws_wait(bar_empty + 8 * xbuf, ((t - 2) >> 1) & 1, err_flag);
            if (hist[xbuf].last) wb_finish<MODE, NBP>(wa, smem, smem_base, hist[xbuf], bt, cta, G);
        }
        hist[xbuf] = st;
        if (st.first && t != 0) {  // the first block's table is the compute warps' job
            // pair tables: entry e = lo | hi<<4 -> half2{pal[lo], pal[hi]}; builder warp w writes the
            // entries with hi = w, w + WB_NB, ...; lane L writes its own bank.
            const uint32_t hb1 = a.hb_mul * st.blk, hb2 = hb1 + a.hb_add2;
            uint32_t *tbl = reinterpret_cast<uint32_t *>(smem + tb * WB_TBL_BYTES);
#pragma unroll
            for (int hh = 0; hh < 2; hh++) {
                const uint32_t row = (hh == 0 ? hb1 : hb2) * 32 + lane;
                const uint16_t *prow = (hh == 0 ? a.pal1 : a.pal2) + (size_t)row * 16;
                const uint4 p0 = *reinterpret_cast<const uint4 *>(prow);
                const uint4 pp = *reinterpret_cast<const uint4 *>(prow + 8);
                const uint32_t cbp[8] = {p0.x, p0.y, p0.z, p0.w, pp.x, pp.y, pp.z, pp.w};
                for (uint32_t hi = bw; hi < 16; hi += WB_NB) {
                    const uint32_t hi_pair = reinterpret_cast<const uint32_t *>(prow)[hi >> 1];  // {pal[hi&~1], pal[hi|1]}
                    const uint32_t hsel = (hi & 1) ? 0x7600u : 0x5400u;
#pragma unroll
                    for (int lo = 0; lo < 16; lo++) {
                        const uint32_t v = __byte_perm(cbp[lo >> 1], hi_pair, hsel | ((lo & 1) ? 0x32u : 0x10u));
                        tbl[((uint32_t)lo + 16u * hi) * 64 + hh * 32 + lane] = v;
                    }
                }
            }
        }
        if (!waited) {
            // Everything above reads only weights.  x, the partial sums, the counters and y belong to
            // the stream order: wait for the kernels before this one.
            pdl_wait();
            waited = true;
        }
        // this stage's slice of every sequence's x; rows of the padding sequences are zero.  Four
        // 16-byte loads per thread are in flight before the first store.
        {
            const uint32_t n16 = (st.pe - st.pb) * 4;           // 16-byte units per sequence
            const uint32_t total = n16 * (uint32_t)Geo::NB;     // flat index: sequence-major
            uint8_t *xbase = smem + WB_X_OFF + xbuf * WB_X_BYTES;
            for (uint32_t i0 = bt; i0 < total; i0 += 4 * WS_COMMON_BTHREADS) {
                uint4 v[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const uint32_t i = i0 + e * WS_COMMON_BTHREADS;
                    v[e] = make_uint4(0, 0, 0, 0);
                    if (i < total) {
                        const uint32_t b = i / n16, k = i - b * n16;
                        if (b < wa.batch)
                            v[e] = reinterpret_cast<const uint4 *>(a.x + (size_t)b * a.x_stride + (size_t)st.pb * 32)[k];
                    }
                }
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const uint32_t i = i0 + e * WS_COMMON_BTHREADS;
                    if (i < total) {
                        const uint32_t b = i / n16, k = i - b * n16;
                        reinterpret_cast<uint4 *>(xbase + b * Geo::ROW_BYTES)[k] = v[e];
                    }
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
        if (hist[xbuf].last) wb_finish<MODE, NBP>(wa, smem, smem_base, hist[xbuf], bt, cta, G);
    }
}

template <int MODE, int SBASE, int NBP>
__global__ void __launch_bounds__(WbGeom<NBP>::THREADS, 1) lut_gemv_wsb_kernel(const WbArgs wa) {
    constexpr int NC = WbGeom<NBP>::NC;
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
    const SkArgs &a = wa.g;
    if (SBASE >= 0 && smem_base != (uint32_t)SBASE) {  // layout assumption broken: refuse to compute
        if (threadIdx.x == 0) atomicExch(a.err, 1u);
        return;
    }
    pdl_launch_dependents();
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t cta = blockIdx.x, G = gridDim.x;
    const uint32_t u_begin = sk_boundary(a.part, cta);
    const uint32_t u_end = sk_boundary(a.part, cta + 1);
    if (u_begin >= u_end) return;
    volatile uint32_t *err_flag = reinterpret_cast<volatile uint32_t *>(smem + WB_BAR_OFF + 40);
    if (tid == 0) {
        const uint32_t bar = smem_base + WB_BAR_OFF;
        t5::mbar_init(bar + 0, WS_COMMON_BTHREADS);
        t5::mbar_init(bar + 8, WS_COMMON_BTHREADS);
        t5::mbar_init(bar + 16, NC * 32);
        t5::mbar_init(bar + 24, NC * 32);
        t5::mbar_init(bar + 32, WS_COMMON_BTHREADS);  // red_free: the builders have read the sum buffer
        *err_flag = 0;
    }
    __syncthreads();
    if (warp < NC) {
        wb_compute<SBASE, NBP>(a, smem, smem_base, u_begin, u_end, warp, lane, err_flag);
    } else {
        wb_build<MODE, NBP>(wa, smem, smem_base, u_begin, u_end, tid - NC * 32, cta, G, err_flag);
        if (*err_flag && tid == NC * 32) atomicExch(a.err, 2u);  // a hand-over wait gave up
    }
}

template <int MODE, int SBASE, int NBP>
static int launch_wsb_v(prism_cuda_ctx *ctx, const WbArgs &wa, dim3 grid) {
    static bool configured[PRISM_MAX_DEVICES] = {false};
    if (!configured[ctx->device]) {
        PRISM_CUDA_TRY(ctx, cudaFuncSetAttribute(lut_gemv_wsb_kernel<MODE, SBASE, NBP>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)WB_SMEM_BYTES));
        configured[ctx->device] = true;
    }
    launch_pdl(ctx, "lut_gemv_wsb_kernel", lut_gemv_wsb_kernel<MODE, SBASE, NBP>, grid, WbGeom<NBP>::THREADS, WB_SMEM_BYTES, wa);
    return after_launch(ctx, "lut_gemv_wsb_kernel");
}

template <int MODE, int NBP>
static int launch_wsb_m(prism_cuda_ctx *ctx, const WbArgs &wa, dim3 grid) {
    if (ctx->smem_base == WB_KNOWN_SBASE) return launch_wsb_v<MODE, WB_KNOWN_SBASE, NBP>(ctx, wa, grid);
    return launch_wsb_v<MODE, -1, NBP>(ctx, wa, grid);
}

template <int NBP>
static int launch_wsb_n(prism_cuda_ctx *ctx, GemvMode mode, const WbArgs &wa, dim3 grid) {
    switch (mode) {
    case GEMV_PLAIN: return launch_wsb_m<GEMV_PLAIN, NBP>(ctx, wa, grid);
    case GEMV_RESID: return launch_wsb_m<GEMV_RESID, NBP>(ctx, wa, grid);
    case GEMV_F32: return launch_wsb_m<GEMV_F32, NBP>(ctx, wa, grid);
    default: return launch_wsb_m<GEMV_SWIGLU, NBP>(ctx, wa, grid);
    }
}

bool wsb_eligible(const LutTensor &t, uint32_t batch) {
    return t.bits == 4 && t.k % 32 == 0 && t.k >= 32 && batch >= 2 && batch <= 8;
}

// Up to 8 rows of x (x_stride halfs apart) against one tensor; rows of y are y_stride apart.
int launch_gemv_wsb(prism_cuda_ctx *ctx, GemvMode mode, const LutTensor &t, const LutTensor *t2, const uint16_t *x,
                    uint32_t x_stride, void *y, uint32_t y_stride, const uint16_t *resid, uint32_t batch) {
    if (!wsb_eligible(t, batch)) return fail(ctx, PRISM_E_ARG, "batched GEMV: 4-bit, K % 32 == 0, 2..8 rows");
    WbArgs wa{};
    SkArgs &a = wa.g;
    wa.batch = batch;
    a.n_chunks = t.n_chunks;
    a.m = t.m;
    a.x = x; a.x_stride = x_stride; a.y = static_cast<uint16_t *>(y); a.y_stride = y_stride; a.resid = resid;
    a.err = ctx->dev_err;
    if (mode == GEMV_SWIGLU) {
        a.idx1 = t.idx; a.pal1 = t.pal; a.idx2 = t2->idx; a.pal2 = t2->pal;
        a.hb_mul = 1; a.hb_add2 = 0;
        a.n_blocks = t.n_hb;
    } else {
        a.idx1 = a.idx2 = t.idx; a.pal1 = a.pal2 = t.pal;
        a.hb_mul = 2; a.hb_add2 = 1;
        a.n_blocks = t.n_hb / 2;
    }
    a.part = ws_partition(ctx, a.n_blocks, a.n_chunks, 1, 85);  // a batch streams longer per block: idle SMs cost more
    const uint32_t G = a.part.G;
    const uint32_t nbp = (batch + 1) / 2;
    PRISM_TRY(ensure_splitk(ctx, (size_t)G * 2 * (2 * nbp) * 64, (size_t)a.n_blocks));
    a.partials = ctx->splitk_partials;
    a.counters = ctx->splitk_counters;
    const dim3 grid(G, 1);
    switch (nbp) {
    case 1: return launch_wsb_n<1>(ctx, mode, wa, grid);
    case 2: return launch_wsb_n<2>(ctx, mode, wa, grid);
    case 3: return launch_wsb_n<3>(ctx, mode, wa, grid);
    default: return launch_wsb_n<4>(ctx, mode, wa, grid);
    }
}

}  // namespace prism

