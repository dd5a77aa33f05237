// Pieces shared by the pair-table tensor-core GEMV kernels: the partition of the work over CTAs,
// and the device helpers of the inner loop (table lookups, x fragments, mma.sync).
#pragma once

#include "common.cuh"
#include "tp_push.cuh"

namespace prism {

constexpr int SK_QUANT = 8;  // segment boundaries fall on multiples of this many chunks

// The partition of the U = n_blocks * n_chunks units over G CTAs, in one of two forms.
//  * stream (s == 0): CTA i starts at i*q + min(i, r) (q = U / G, r = U % G), ranges as equal as
//    integers allow, G = every resident CTA slot.  For work of many chunks per CTA.
//  * uniform (s > 0): every block is cut into s equal parts, CTA b*s + k takes part k of block b,
//    so a CTA never builds more than one table.  For small matrices, where the time is latency.
// A start that falls inside a block is moved down to a multiple of SK_QUANT chunks, or up to the
// next block when fewer than SK_QUANT chunks of the block would be left (no segment is shorter
// than SK_QUANT chunks); with whole_blocks set it is moved down to the start of the block.
struct SkPart {
    uint32_t q, r, G, n_chunks, total, s, whole_blocks;
};
__host__ __device__ inline uint32_t sk_raw_start(const SkPart &p, uint32_t i) {
    if (i >= p.G) return p.total;
    if (p.s) {
        const uint32_t b = i / p.s, k = i - b * p.s;
        return b * p.n_chunks + k * p.n_chunks / p.s;
    }
    return i * p.q + (i < p.r ? i : p.r);
}
// snaps a position given relative to the start of its block (0 <= c < n_chunks)
__host__ __device__ inline uint32_t sk_snap_rel(const SkPart &p, uint32_t c) {
    if (p.whole_blocks) return 0;
    const uint32_t s = c / SK_QUANT * SK_QUANT;
    return (s > 0 && p.n_chunks - s < (uint32_t)SK_QUANT) ? p.n_chunks : s;
}
__host__ __device__ inline uint32_t sk_boundary(const SkPart &p, uint32_t i) {
    const uint32_t u = sk_raw_start(p, i);
    if (u >= p.total) return p.total;
    const uint32_t b = u / p.n_chunks;
    return b * p.n_chunks + sk_snap_rel(p, u - b * p.n_chunks);
}
// Start of CTA i's range clipped to the block [b0, b0 + n_chunks).
__device__ __forceinline__ uint32_t sk_boundary_in_block(const SkPart &p, uint32_t i, uint32_t b0) {
    const uint32_t u = sk_raw_start(p, i);
    if (u <= b0) return b0;                       // starts in an earlier block: snapping never crosses b0
    if (u >= b0 + p.n_chunks) return b0 + p.n_chunks;
    return b0 + sk_snap_rel(p, u - b0);
}

struct SkArgs {
    const uint8_t *idx1, *idx2;   // index arrays the two half-blocks of a block come from
    const uint16_t *pal1, *pal2;
    uint32_t n_chunks;            // chunks per row
    uint32_t hb_mul, hb_add2;     // block b = half-blocks hb_mul*b (rows "1") and hb_mul*b+hb_add2 (rows "2")
    uint32_t m;                   // valid output rows (per tensor)
    uint32_t n_blocks;
    SkPart part;                  // how the (block, chunk) units are dealt to the CTAs
    const uint16_t *x; uint32_t x_stride;
    uint16_t *y; uint32_t y_stride;
    const uint16_t *resid;
    float *partials;              // [batch][G][2][64]
    unsigned int *counters;       // [batch][n_blocks], chunks of the block that have arrived
    unsigned int *err;
    uint32_t norm_n;              // > 0: stage rms_norm(x) (row of norm_n values) instead of x
    float norm_eps;
    TpPush tp;                    // GEMV_TP only: where the all-reduce of the block sums goes
};

// Chooses between the two forms for a matrix of n_blocks x n_chunks units and `slots` resident CTA
// slots: contiguous balanced ranges when a CTA gets at least `stream_chunks` chunks (and no block
// more than `max_contrib` contributors), else every block in s <= 8 equal parts of at least
// `min_chunks` chunks.  Pure host arithmetic.
inline SkPart sk_choose_partition(uint32_t n_blocks, uint32_t n_chunks, uint32_t slots, uint32_t stream_chunks,
                                  uint32_t min_chunks, uint32_t max_contrib) {
    SkPart p{};
    p.n_chunks = n_chunks;
    p.total = n_blocks * n_chunks;
    if (slots == 0) slots = 1;
    if (min_chunks < (uint32_t)SK_QUANT) min_chunks = SK_QUANT;
    if (p.total / slots >= stream_chunks && p.total / slots >= (n_chunks + max_contrib - 1) / max_contrib &&
        p.total / slots >= 1) {
        p.G = slots;
        p.q = p.total / p.G;
        p.r = p.total % p.G;
        // short rows, several blocks per CTA: whole blocks only (no partial sums, no extra table)
        p.whole_blocks = (n_chunks <= 64 && p.q >= 3 * n_chunks) ? 1 : 0;
    } else {
        uint32_t s = n_chunks / min_chunks;
        if (n_blocks && s > slots / n_blocks) s = slots / n_blocks;
        if (s > 8) s = 8;
        if (s < 1) s = 1;
        p.s = s;
        p.G = n_blocks * s;
    }
    return p;
}

// How many CTAs the warp-specialised kernels use for n_blocks blocks of rows n_chunks long when `slots` CTAs can
// be resident: all of them, or -- when the matrix has fewer blocks than that but at least fill_pct per 100, and
// rows of at most whole_max_chunks chunks (0: never) -- one per block, so that every CTA gets one whole block
// (sk_choose_partition then cuts nothing).  Pure host arithmetic.
inline uint32_t ws_choose_slots(uint32_t n_blocks, uint32_t n_chunks, uint32_t slots, uint32_t whole_max_chunks, uint32_t fill_pct) {
    if (slots == 0) slots = 1;
    if (whole_max_chunks && n_blocks < slots && (uint64_t)n_blocks * 100 >= (uint64_t)slots * fill_pct && n_chunks <= whole_max_chunks)
        return n_blocks;
    return slots;
}

// gemv_ws.cu: the partition of the warp-specialised kernels (one CTA per SM)
SkPart ws_partition(prism_cuda_ctx *ctx, uint32_t n_blocks, uint32_t n_chunks, uint32_t batch, uint32_t fill_pct);

// Arrival on a block's counter: an acq_rel add at gpu scope.  Called by one thread after a CTA-level
// barrier that follows the CTA's stores of partial sums (the release then covers those stores) and
// before a CTA-level barrier that precedes the loads of other CTAs' partial sums (the acquire covers
// them), so no separate fences are needed.
__device__ __forceinline__ unsigned int sk_arrive(unsigned int *ctr, unsigned int v) {
    unsigned int prev;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;\n" : "=r"(prev) : "l"(ctr), "r"(v) : "memory");
    return prev;
}

__device__ __forceinline__ void sk_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int IMM>
__device__ __forceinline__ uint4 sk_ldg(const uint8_t *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4+%5];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p), "n"(IMM));
    return v;
}
// Where a warp's index chunks come from: 16 bytes per lane and chunk, lane-contiguous (512 B per
// half-block and chunk).  `OFF` is in bytes from the warp's current chunk.
struct SkSrcPtr {
    const uint8_t *p;   // rows "1", this lane
    uint64_t d2;        // byte distance to the rows "2" array position
    template <int OFF> __device__ __forceinline__ uint4 load1() const { return sk_ldg<OFF>(p); }
    template <int OFF> __device__ __forceinline__ uint4 load2() const { return sk_ldg<OFF>(p + d2); }
    __device__ __forceinline__ void advance(uint32_t bytes) { p += bytes; }
};
// Shared-memory loads whose address is `register + immediate`.  SBASE is the offset of dynamic
// shared memory inside the shared window when it is known at compile time (probed once per
// context): the table base then rides in the immediate field and a lookup costs one byte-permute
// (offset) and one load.  SBASE < 0 is the portable variant (base added at run time).
template <int SBASE, int IMM>
__device__ __forceinline__ uint32_t sk_lds(uint32_t off, uint32_t base) {
    uint32_t v;
    if (SBASE >= 0) asm volatile("ld.shared.u32 %0, [%1+%2];\n" : "=r"(v) : "r"(off), "n"(SBASE >= 0 ? SBASE + IMM : 0));
    else asm volatile("ld.shared.u32 %0, [%1+%2];\n" : "=r"(v) : "r"(off + base), "n"(IMM));
    return v;
}

// 16 bytes of x for the lanes that hold a non-zero part of the B operand; the other lanes keep
// what their registers hold (zero, set once before the first chunk).  Predicated-off lanes issue
// no shared-memory request.
template <int SBASE, int IMM>
__device__ __forceinline__ void sk_ldx(uint4 &v, uint32_t off, uint32_t base, uint32_t diag) {
    if (SBASE >= 0)
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %5, 0;\n\t"
            "@p ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%6];\n\t}\n"
            : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
            : "r"(off), "r"(diag), "n"(SBASE >= 0 ? SBASE + IMM : 0));
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %5, 0;\n\t"
            "@p ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%6];\n\t}\n"
            : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
            : "r"(off + base), "r"(diag), "n"(IMM));
}

// The eight table lookups of one 32-bit index word per half-block (= two tensor-core steps).
// byte j of the word -> (byte << 8) | lane_off: offset of table entry `byte` in this lane's bank;
// lane_off = lane*4, plus a multiple of 65536 to select one of several tables (its byte 2 is kept).
template <int SBASE>
__device__ __forceinline__ void sk_lookup(uint32_t (&A)[8], uint32_t w1, uint32_t w2, uint32_t lane_off, uint32_t base) {
    const uint32_t o10 = __byte_perm(w1, lane_off, 0x7604), o11 = __byte_perm(w1, lane_off, 0x7614);
    const uint32_t o12 = __byte_perm(w1, lane_off, 0x7624), o13 = __byte_perm(w1, lane_off, 0x7634);
    const uint32_t o20 = __byte_perm(w2, lane_off, 0x7604), o21 = __byte_perm(w2, lane_off, 0x7614);
    const uint32_t o22 = __byte_perm(w2, lane_off, 0x7624), o23 = __byte_perm(w2, lane_off, 0x7634);
    A[0] = sk_lds<SBASE, 0>(o10, base);   A[1] = sk_lds<SBASE, 128>(o20, base);
    A[2] = sk_lds<SBASE, 0>(o11, base);   A[3] = sk_lds<SBASE, 128>(o21, base);
    A[4] = sk_lds<SBASE, 0>(o12, base);   A[5] = sk_lds<SBASE, 128>(o22, base);
    A[6] = sk_lds<SBASE, 0>(o13, base);   A[7] = sk_lds<SBASE, 128>(o23, base);
}

constexpr int SK_NACC = 2;                // independent accumulator sets of the chunk routine (2 or 4)
constexpr int SK_TBL_BYTES = 256 * 256;   // one pair table: 256 entries x (2 half-blocks x 32 lanes x 4 B); x is staged right behind it

// Stands for "no further chunk to request" where the chunk routine is used without its prefetch.
struct SkNoNext {
    template <int OFF> __device__ __forceinline__ uint4 load1() const { return make_uint4(0, 0, 0, 0); }
    template <int OFF> __device__ __forceinline__ uint4 load2() const { return make_uint4(0, 0, 0, 0); }
};
// One 32-weight chunk of the two half-blocks: 8 tensor-core steps of 4 k each.  The MMA's 16 x 16
// A operand is read as "row g = lanes 4g..4g+3, each lane two k-pairs of its own weight row"
// (rows g: half-block 1, rows g+8: half-block 2), and B carries x[k..k+3] only where its k-rows
// meet the column of the same lane (lanes 0, 5, 10, 15), so accumulator column n of MMA row g is
// the dot product of lane (g, n).  x_off is the byte offset of the chunk's 64 bytes of x inside
// the staged piece.  Lookups of word h+1 are issued before the tensor-core steps of word h; once
// the last word's lookups are out, w1/w2 are dead and the chunk PF steps ahead is loaded into them.
template <int SBASE, int NEXT_IMM, typename SRC>
__device__ __forceinline__ void sk_chunk(float (&acc)[SK_NACC][4], uint4 &w1, uint4 &w2, uint4 (&xb)[2], uint32_t lane_off,
                                         uint32_t x_off, uint32_t diag, uint32_t base, const SRC &next, bool more) {
    sk_ldx<SBASE, SK_TBL_BYTES + 0>(xb[0], x_off, base, diag);
    sk_ldx<SBASE, SK_TBL_BYTES + 16>(xb[1], x_off, base, diag);
    uint32_t A0[8], A1[8];
    sk_lookup<SBASE>(A0, w1.x, w2.x, lane_off, base);
    sk_lookup<SBASE>(A1, w1.y, w2.y, lane_off, base);
    constexpr int H = SK_NACC == 4 ? 2 : 0;  // second pair of accumulator sets
    sk_mma(acc[0], A0[0], A0[1], A0[2], A0[3], xb[0].x, xb[0].y);
    sk_mma(acc[1], A0[4], A0[5], A0[6], A0[7], xb[0].z, xb[0].w);
    sk_ldx<SBASE, SK_TBL_BYTES + 32>(xb[0], x_off, base, diag);
    sk_lookup<SBASE>(A0, w1.z, w2.z, lane_off, base);
    sk_mma(acc[H + 0], A1[0], A1[1], A1[2], A1[3], xb[1].x, xb[1].y);
    sk_mma(acc[H + 1], A1[4], A1[5], A1[6], A1[7], xb[1].z, xb[1].w);
    sk_ldx<SBASE, SK_TBL_BYTES + 48>(xb[1], x_off, base, diag);
    sk_lookup<SBASE>(A1, w1.w, w2.w, lane_off, base);
    if (more) {
        w1 = next.template load1<NEXT_IMM>();
        w2 = next.template load2<NEXT_IMM>();
    }
    sk_mma(acc[0], A0[0], A0[1], A0[2], A0[3], xb[0].x, xb[0].y);
    sk_mma(acc[1], A0[4], A0[5], A0[6], A0[7], xb[0].z, xb[0].w);
    sk_mma(acc[H + 0], A1[0], A1[1], A1[2], A1[3], xb[1].x, xb[1].y);
    sk_mma(acc[H + 1], A1[4], A1[5], A1[6], A1[7], xb[1].z, xb[1].w);
}

// ---- 2-bit indices (4-entry palette) through the same lookups ------------------------------------
// A 2-bit index word holds 16 weights; a NIBBLE (two weights) indexes a 16-entry pair table laid out
// like the 4-bit one (entry e at byte e*256 + t*128 + lane*4).  The even and odd nibble planes of the
// word are separated and re-interleaved so that the bytes of each resulting word are the table indices
// of four consecutive weight pairs -- exactly what a 4-bit index word is to sk_lookup.
__device__ __forceinline__ void sk_expand2_word(uint32_t &lo, uint32_t &hi, uint32_t w) {
    const uint32_t we = w & 0x0F0F0F0Fu, wo = (w >> 4) & 0x0F0F0F0Fu;  // pairs (0,1),(4,5),.. and (2,3),(6,7),..
    lo = __byte_perm(we, wo, 0x5140);  // weights 0..7
    hi = __byte_perm(we, wo, 0x7362);  // weights 8..15
}
// 16 bytes of 2-bit indices (64 weights) -> two pseudo 4-bit chunks of 32 weights
__device__ __forceinline__ void sk_expand2(uint4 &a, uint4 &b, const uint4 &w) {
    sk_expand2_word(a.x, a.y, w.x);
    sk_expand2_word(a.z, a.w, w.y);
    sk_expand2_word(b.x, b.y, w.z);
    sk_expand2_word(b.z, b.w, w.w);
}
// Pair table of a block of 2-bit rows: entry e = i0 | i1 << 2 -> half2{pal[i0], pal[i1]}, 16 entries per
// row.  `n_warps` warps share the entries; lane L writes its own bank.
__device__ __forceinline__ void sk_build_table2(uint32_t *tbl, const uint16_t *pal1, const uint16_t *pal2, uint32_t hb1,
                                                uint32_t hb2, uint32_t lane, uint32_t warp, uint32_t n_warps) {
#pragma unroll
    for (int t = 0; t < 2; t++) {
        const uint32_t row = (t == 0 ? hb1 : hb2) * 32 + lane;
        const uint2 p = *reinterpret_cast<const uint2 *>((t == 0 ? pal1 : pal2) + (size_t)row * 4);  // 4 fp16
        for (uint32_t e = warp; e < 16; e += n_warps) {
            const uint32_t i0 = e & 3, i1 = e >> 2;
            const uint32_t v0 = ((i0 & 2) ? p.y : p.x) >> ((i0 & 1) * 16) & 0xFFFFu;
            const uint32_t v1 = ((i1 & 2) ? p.y : p.x) >> ((i1 & 1) * 16) & 0xFFFFu;
            tbl[e * 64 + t * 32 + lane] = v0 | (v1 << 16);
        }
    }
}

}  // namespace prism
