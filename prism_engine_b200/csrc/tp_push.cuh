// All-reduce of a row-parallel matmul's partial sums, done inside the GEMV kernel that produces them
// (tensor-parallel decode, one sequence).  The reference has no collective; this is the exchange step
// of a K-sharded linear: h = f16( f16(sum over ranks of partial) + h ).
//
// The unit is a half-block: 32 output rows, owned by one warp of the CTA that has just completed the
// rank's local sums for them.  That warp
//   1. stores its 32 fp32 sums into slot [epoch & 1][this rank] of EVERY rank's receive area (plain
//      stores over NVLink into peer memory mapped with cudaIpc*) as soon as they are complete, while the
//      CTA goes on streaming;
// and, when the CTA has nothing left to stream, for all the half-blocks it delivered:
//   2. fences at system scope, writes the epoch into flag [this rank][half-block] of every rank, and
//      waits (bounded) until its own flags [0..world)[half-block] hold the epoch -- the peers run the
//      same kernel on their own K shard;
//   3. adds the `world` partial sums in rank order (bit-identical on every rank), rounds to fp16, adds
//      the residual and stores h.
// Nothing waits before it has delivered, so no rank can wait for a rank that waits for it.  Two
// slots are enough: a rank can only start all-reduce e+2 after every peer has delivered e+1, which a
// peer does after it has finished reading e (its kernel e completes before its kernel e+1 starts).
// The epoch lives in device memory and is advanced by the warp that finishes the last half-block, so
// the kernel replays inside a CUDA graph.  No multimem, no TMA, no bulk copies on peer memory.
#pragma once

#include "common.cuh"

namespace prism {

constexpr int TP_AR_MAX_CTAS = 1024;               // flags per rank: CTAs of the stand-alone kernel, or half-blocks
constexpr unsigned int TP_AR_SPIN_LIMIT = 1u << 25;  // polls with back-off: about fifteen seconds (ranks may start seconds apart)
constexpr uint32_t TP_LL_CAP = 65536;              // rows per rank slot of the flagged-word area (longest output vector it takes)

struct TpPush {
    void *const *peer_tab;   // device array: world receive-area pointers, then world flag pointers; nullptr: not in use
    float *recv;             // this rank's receive area [2][world][cap]
    unsigned int *flags;     // this rank's flags [world][TP_AR_MAX_CTAS]
    unsigned int *state;     // {epoch of the last completed all-reduce, half-blocks finished in the current one}
    uint32_t world, rank, cap, spin_limit;
    uint32_t n_units;        // half-blocks of the output vector
    uint32_t deliver_only;   // 1: the kernel only delivers; wait and reduction are a following kernel
    uint32_t ll_off;         // != 0: deliver 8-byte words {sum, epoch} into the flagged-word area, this many bytes into
                             // every rank's receive area ([2][world][TP_LL_CAP] words); the reader polls the words themselves
};

// Host side (tp.cu): fills the kernel argument from the context's peer set-up; fails when the peer path is
// not set up or the tensor has more half-blocks than flags.
int tp_fill_push(prism_cuda_ctx *ctx, const LutTensor &t, TpPush *out);

#ifdef __CUDACC__
constexpr int TP_LIST_MAX = 32;  // half-blocks a warp may have delivered before it must stop and finish them

__device__ __forceinline__ unsigned int tp_epoch(const TpPush &tp) {
    return *reinterpret_cast<volatile unsigned int *>(tp.state) + 1;  // stable while this kernel runs
}

// Step 1 for one half-block, called by one whole warp as soon as the rank's local sums of the 32 rows are
// complete: lane L holds the sum of row hb*32 + L (rows past the tensor carry zeros).  Only stores: a warp
// never waits in the middle of the kernel, where a late peer would stall the CTA's pipeline.
__device__ __forceinline__ void tp_deliver(const TpPush &tp, unsigned int e, uint32_t hb, uint32_t lane, float sum) {
    const uint32_t slot = e & 1, row = hb * 32 + lane;
    if (tp.ll_off) {
        // One 8-byte store carries value and epoch: a reader that sees the epoch sees the value (a scalar 64-bit
        // access is single-copy atomic), so neither a fence nor a separate flag crosses the link.
        const unsigned long long word = ((unsigned long long)e << 32) | (unsigned long long)__float_as_uint(sum);
        for (uint32_t q = 0; q < tp.world; q++) {
            unsigned long long *dst = reinterpret_cast<unsigned long long *>(static_cast<char *>(tp.peer_tab[q]) + tp.ll_off) +
                                      ((size_t)slot * tp.world + tp.rank) * TP_LL_CAP + row;
            asm volatile("st.relaxed.sys.global.u64 [%0], %1;\n" ::"l"(dst), "l"(word) : "memory");
        }
        return;
    }
    for (uint32_t q = 0; q < tp.world; q++) {
        float *dst = static_cast<float *>(tp.peer_tab[q]) + ((size_t)slot * tp.world + tp.rank) * tp.cap + row;
        *dst = sum;
    }
}

// Steps 2 and 3 for the `n` half-blocks list[0..n) this warp has delivered (the same warp, so one fence at
// system scope covers all its stores): publish the flags, then for each half-block wait for every rank's
// flag (bounded: spin_limit polls, then error code 3), add in rank order, round, add the residual into h,
// and count the half-block as finished.  Called at the end of the CTA's work.
__device__ __forceinline__ void tp_finish(const TpPush &tp, unsigned int e, const uint16_t *list, uint32_t n, uint32_t lane,
                                          uint32_t m, uint16_t *h, unsigned int *err) {
    if (n == 0 || tp.deliver_only) return;
    const uint32_t slot = e & 1;
    if (tp.ll_off) {
        // flagged words: nothing to publish; poll the `world` words of each row (bounded), add in rank order
        const unsigned long long *ll = reinterpret_cast<const unsigned long long *>(reinterpret_cast<const char *>(tp.recv) + tp.ll_off) +
                                       (size_t)slot * tp.world * TP_LL_CAP;
        for (uint32_t i = 0; i < n; i++) {
            const uint32_t row = list[i] * 32 + lane;
            float s = 0.0f;
            for (uint32_t r = 0; r < tp.world; r++) {
                const unsigned long long *p = ll + (size_t)r * TP_LL_CAP + row;
                unsigned long long v;
                unsigned int polls = 0;
                for (;;) {
                    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];\n" : "=l"(v) : "l"(p) : "memory");
                    if ((unsigned int)(v >> 32) == e) break;
                    if (++polls > tp.spin_limit) {
                        atomicExch(err, 3u);
                        break;
                    }
                    if (polls > 64) __nanosleep(polls > 4096 ? 500 : 50);
                }
                s += __uint_as_float((unsigned int)v);
            }
            if (row < m) {
                const float o = __half2float(__float2half_rn(s)) + __half2float(__ushort_as_half(h[row]));
                h[row] = __half_as_ushort(__float2half_rn(o));
            }
        }
    } else {
    __threadfence_system();
    __syncwarp();
    if (lane < tp.world) {
        unsigned int *fb = static_cast<unsigned int *>(tp.peer_tab[tp.world + lane]) + (size_t)tp.rank * TP_AR_MAX_CTAS;
        for (uint32_t i = 0; i < n; i++) asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(fb + list[i]), "r"(e) : "memory");
    }
    for (uint32_t i = 0; i < n; i++) {
        const uint32_t hb = list[i], row = hb * 32 + lane;
        if (lane < tp.world) {
            const unsigned int *f = tp.flags + (size_t)lane * TP_AR_MAX_CTAS + hb;
            unsigned int seen = 0, polls = 0;
            for (;;) {
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(seen) : "l"(f) : "memory");
                if ((int)(seen - e) >= 0) break;  // a peer that is already one all-reduce ahead has delivered this one too
                if (++polls > tp.spin_limit) {
                    atomicExch(err, 3u);  // a peer did not deliver: reported by the next synchronising host call
                    break;
                }
                if (polls > 64) __nanosleep(polls > 4096 ? 500 : 50);
            }
        }
        __syncwarp();
        float s = 0.0f;
        for (uint32_t r = 0; r < tp.world; r++) s += __ldcg(tp.recv + ((size_t)slot * tp.world + r) * tp.cap + row);
        if (row < m) {
            const float o = __half2float(__float2half_rn(s)) + __half2float(__ushort_as_half(h[row]));
            h[row] = __half_as_ushort(__float2half_rn(o));
        }
    }
    }
    // ---- the warp that finishes the last half-block advances the epoch ----
    __syncwarp();
    if (lane == 0) {
        __threadfence();
        if (atomicAdd(&tp.state[1], n) + n == tp.n_units) {
            tp.state[1] = 0;
            __threadfence();
            tp.state[0] = e;
        }
    }
}

// A warp's bookkeeping of what it has delivered: deliver, remember, and finish early only when the list is full.
struct TpWarpList {
    uint16_t *list;   // TP_LIST_MAX entries of shared memory owned by this warp
    uint32_t n;
};
__device__ __forceinline__ void tp_deliver_listed(const TpPush &tp, TpWarpList &wl, uint32_t hb, uint32_t lane, float sum,
                                                  uint32_t m, uint16_t *h, unsigned int *err) {
    const unsigned int e = tp_epoch(tp);
    if (tp.deliver_only) {
        tp_deliver(tp, e, hb, lane, sum);
        return;
    }
    if (wl.n == (uint32_t)TP_LIST_MAX) {
        tp_finish(tp, e, wl.list, wl.n, lane, m, h, err);
        wl.n = 0;
    }
    tp_deliver(tp, e, hb, lane, sum);
    if (lane == 0) wl.list[wl.n] = (uint16_t)hb;
    __syncwarp();
    wl.n += 1;
}
#endif

}  // namespace prism
