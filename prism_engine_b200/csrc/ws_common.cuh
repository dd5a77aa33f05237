// Pieces shared by the warp-specialised GEMV kernels: the walk over a CTA's stages, bounded
// mbarrier waits, and the builder warps' own barrier.
#pragma once

#include "common.cuh"
#include "pair_table.cuh"
#include "tc5_ptx.cuh"

namespace prism {

constexpr int WS_COMMON_BTHREADS = 128;          // builder threads (4 warps) of every warp-specialised kernel
constexpr uint32_t WS_WAIT_LIMIT = 1u << 24;     // polls (with back-off) before a wait gives up

// One stage of a CTA's range: a block and a run of at most `stage_chunks` chunks inside it.
struct WsStage {
    uint32_t blk, pb, pe;   // block, chunk run [pb, pe) inside it
    uint32_t cb, ce;        // the whole run of this CTA inside the block (segment)
    uint32_t seg;           // index of the segment within the CTA (table buffer = seg & 1)
    bool first, last;       // first / last stage of the segment
};
// Walks the stages of a CTA's range [u0, u1).  The two segments that cover only part of a block
// (the head of the range, when it starts inside a block, and its tail, when it ends inside one)
// come first, whole blocks after them: the partial sums of shared blocks are delivered, and fixed up
// by whichever CTA completes the block, while the whole blocks are still being streamed, and the
// kernel ends on a segment that only has to write its outputs.
struct WsWalk {
    uint32_t lo1, hi1, lo2, hi2;  // tail, whole blocks (the head is the first [u, u_end))
    uint32_t phase, u, u_end, nc, seg, pb_next, sc;
    WsStage cur;
    bool in_seg;
    __device__ __forceinline__ void init(uint32_t u0, uint32_t u1, uint32_t n_chunks, uint32_t stage_chunks) {
        nc = n_chunks; sc = stage_chunks; seg = 0; in_seg = false; pb_next = 0;
        cur = WsStage{};
        const uint32_t b0 = u0 / nc;
        uint32_t m0 = u0;                                   // start of what follows the head
        u = u_end = u0;
        if (u0 != b0 * nc) {                                // the range starts inside block b0: head
            u_end = min(u1, (b0 + 1) * nc);
            m0 = u_end;
        }
        const uint32_t t0 = max(m0, (u1 / nc) * nc);        // start of the block the range ends in
        lo1 = t0; hi1 = (t0 < u1 && u1 != (u1 / nc) * nc) ? u1 : t0;  // tail: only if it ends inside a block
        lo2 = m0; hi2 = hi1 > lo1 ? t0 : u1;                // whole blocks between them
        phase = 0;
    }
    // false when the range is exhausted
    __device__ __forceinline__ bool next() {
        if (!in_seg) {
            while (u >= u_end) {
                if (++phase > 2) return false;
                u = phase == 1 ? lo1 : lo2;
                u_end = phase == 1 ? hi1 : hi2;
            }
            cur.blk = u / nc;
            cur.cb = u - cur.blk * nc;
            cur.ce = min(nc, cur.cb + (u_end - u));
            u += cur.ce - cur.cb;
            cur.seg = seg++;
            pb_next = cur.cb;
            in_seg = true;
        }
        cur.pb = pb_next;
        cur.pe = min(cur.ce, cur.pb + sc);
        cur.first = cur.pb == cur.cb;
        cur.last = cur.pe == cur.ce;
        pb_next = cur.pe;
        if (cur.last) in_seg = false;
        return true;
    }
};

// The index chunks one compute warp will consume, in order, over all stages of the CTA's range:
// warp `cw` of `n_warps` takes chunks pb + cw + n_warps*j of every stage.  The cursor runs a fixed
// number of chunks ahead of the warp's consumption, across stage boundaries (index data does not
// depend on the stage hand-over), so the loads of a stage's first chunks are in flight while the
// previous stage is still being streamed.
struct WsPrefetch {
    WsWalk w;
    SkSrcPtr src;       // this lane's pointers for the next chunk to request
    uint32_t left;      // chunks of the cursor's stage still to request
    uint32_t cw, n_warps, lane;
    const SkArgs *a;
    bool valid;
    __device__ __forceinline__ void seek() {
        while (left == 0) {
            if (!w.next()) {
                valid = false;
                return;
            }
            const uint32_t span = w.cur.pe - w.cur.pb;
            left = span > cw ? (span - cw + n_warps - 1) / n_warps : 0;
            if (left) {
                const uint32_t hb1 = a->hb_mul * w.cur.blk, hb2 = hb1 + a->hb_add2;
                src.p = a->idx1 + ((size_t)hb1 * a->n_chunks + w.cur.pb + cw) * 512 + lane * 16;
                src.d2 = (uint64_t)(reinterpret_cast<uintptr_t>(a->idx2 + ((size_t)hb2 * a->n_chunks + w.cur.pb + cw) * 512 +
                                                                lane * 16) -
                                    reinterpret_cast<uintptr_t>(src.p));
            }
        }
    }
    __device__ __forceinline__ void init(const SkArgs *args, uint32_t u0, uint32_t u1, uint32_t stage_chunks,
                                         uint32_t warp, uint32_t warps, uint32_t ln) {
        a = args; cw = warp; n_warps = warps; lane = ln; left = 0; valid = true;
        w.init(u0, u1, args->n_chunks, stage_chunks);
        seek();
    }
    // after the chunk at the cursor has been requested
    __device__ __forceinline__ void advance() {
        src.advance(n_warps * 512);
        left--;
        if (left == 0) seek();
    }
};

// The pair tables of the CTA's FIRST block, built by the compute warps (they would otherwise idle until the
// builders have made it) while the builders wait for the stream dependency and stage the first slice of x:
// the two halves of the prologue run side by side.  Compute warp gw of n_warps takes the (hi nibble,
// half-block) combinations gw, gw + n_warps, ... of the 32; lane L writes its own bank.
// Entry e = lo | hi<<4 -> half2{pal[lo], pal[hi]}.  The callers close it with a barrier of the compute warps.
__device__ __forceinline__ void ws_first_table(const SkArgs &a, uint32_t *tbl, uint32_t blk, uint32_t gw, uint32_t n_warps,
                                               uint32_t lane) {
    const uint32_t hb1 = a.hb_mul * blk, hb2 = hb1 + a.hb_add2;
    for (uint32_t c = gw; c < 32; c += n_warps) {
        const uint32_t hi = c >> 1, h = c & 1;
        const uint32_t row = (h == 0 ? hb1 : hb2) * 32 + lane;
        const uint16_t *prow = (h == 0 ? a.pal1 : a.pal2) + (size_t)row * 16;
        const uint4 p0 = *reinterpret_cast<const uint4 *>(prow);
        const uint4 pp = *reinterpret_cast<const uint4 *>(prow + 8);
        const uint32_t cbp[8] = {p0.x, p0.y, p0.z, p0.w, pp.x, pp.y, pp.z, pp.w};
        const uint32_t hi_pair = reinterpret_cast<const uint32_t *>(prow)[hi >> 1];  // {pal[hi&~1], pal[hi|1]}
        const uint32_t hsel = (hi & 1) ? 0x7600u : 0x5400u;
#pragma unroll
        for (int lo = 0; lo < 16; lo++) {
            const uint32_t v = __byte_perm(cbp[lo >> 1], hi_pair, hsel | ((lo & 1) ? 0x32u : 0x10u));
            tbl[((uint32_t)lo + 16u * hi) * 64 + h * 32 + lane] = v;
        }
    }
}

__device__ __forceinline__ void ws_wait(uint32_t bar, uint32_t parity, volatile uint32_t *err_flag) {
    for (uint32_t i = 0; i < WS_WAIT_LIMIT; i++) {
        if (t5::mbar_test(bar, parity)) return;
        if ((i & 15) == 15) {
            if (*err_flag) return;
            __nanosleep(20);
        }
    }
    *err_flag = 1;
}
__device__ __forceinline__ void ws_bar_builders() { asm volatile("bar.sync 1, %0;\n" ::"n"(WS_COMMON_BTHREADS) : "memory"); }
__device__ __forceinline__ uint32_t ws_bar_builders_count(bool pred) {
    uint32_t n;
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %1, 0;\n\t"
        "bar.red.popc.u32 %0, 1, %2, p;\n\t}\n"
        : "=r"(n)
        : "r"((uint32_t)pred), "n"(WS_COMMON_BTHREADS)
        : "memory");
    return n;
}

}  // namespace prism
