// Tensor-parallel plumbing: one process per GPU, NCCL over NVLink.  The
// reference has no collective of any kind; this is the exchange step a
// K-sharded (row-parallel) palettized matmul needs.  NCCL is bound at run time
// (dlopen) so a single-GPU user needs no NCCL at all, and a process that
// already loaded NCCL (e.g. through torch) shares that copy.
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <vector>

#include "common.cuh"
#include "tp_push.cuh"

struct prism_nccl_api {
    void *lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                              cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
};

namespace prism {

static prism_nccl_api *load_nccl(std::string &err) {
    static prism_nccl_api api;
    static bool tried = false;
    if (tried) return api.lib ? &api : nullptr;
    tried = true;
    const char *names[] = {"libnccl.so.2", "libnccl.so"};
    void *lib = nullptr;
    for (const char *n : names) {
        lib = dlopen(n, RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);  // a copy the process already holds
        if (lib) break;
    }
    for (int i = 0; !lib && i < 2; i++) lib = dlopen(names[i], RTLD_NOW | RTLD_GLOBAL);
    if (!lib) {
        err = std::string("NCCL not found: ") + dlerror();
        return nullptr;
    }
#define LOAD(field, sym)                                                 \
    api.field = reinterpret_cast<decltype(api.field)>(dlsym(lib, sym)); \
    if (!api.field) {                                                    \
        err = std::string("NCCL symbol missing: ") + sym;                \
        return nullptr;                                                  \
    }
    LOAD(GetUniqueId, "ncclGetUniqueId");
    LOAD(CommInitRank, "ncclCommInitRank");
    LOAD(AllReduce, "ncclAllReduce");
    LOAD(AllGather, "ncclAllGather");
    LOAD(CommDestroy, "ncclCommDestroy");
    LOAD(GetErrorString, "ncclGetErrorString");
#undef LOAD
    api.lib = lib;
    return &api;
}

int tp_all_reduce_f32(prism_cuda_ctx *ctx, float *buf, size_t n) {
    if (ctx->tp_world <= 1) return PRISM_OK;
    if (!ctx->nccl || !ctx->nccl_comm) return fail(ctx, PRISM_E_STATE, "no NCCL communicator on this context");
    ncclResult_t r = ctx->nccl->AllReduce(buf, buf, n, ncclFloat32, ncclSum, (ncclComm_t)ctx->nccl_comm, ctx->stream);
    if (r != ncclSuccess) return fail(ctx, PRISM_E_COMM, std::string("ncclAllReduce: ") + ctx->nccl->GetErrorString(r));
    ctx->launches++;
    return PRISM_OK;
}

int tp_all_gather_bytes(prism_cuda_ctx *ctx, const void *send, void *recv, size_t bytes_per_rank) {
    if (ctx->tp_world <= 1) return PRISM_OK;
    if (!ctx->nccl || !ctx->nccl_comm) return fail(ctx, PRISM_E_STATE, "no NCCL communicator on this context");
    ncclResult_t r = ctx->nccl->AllGather(send, recv, bytes_per_rank, ncclUint8, (ncclComm_t)ctx->nccl_comm, ctx->stream);
    if (r != ncclSuccess) return fail(ctx, PRISM_E_COMM, std::string("ncclAllGather: ") + ctx->nccl->GetErrorString(r));
    ctx->launches++;
    return PRISM_OK;
}

// ---------------------------------------------------------------------------------------------
// All-reduce through peer memory, fused with the residual add that follows a row-parallel matmul.
//
// Every rank owns a receive area [2][world][cap] floats and a flag array [world][TP_AR_MAX_CTAS],
// both mapped by every peer (cudaIpc*).  All-reduce number e (counted on the device, the same on
// every rank because every rank runs the same kernel sequence) works in independent slices, one
// per CTA: CTA c of rank r stores its slice of the partial sums into slot [e & 1][r] of EVERY rank's
// receive area (plain stores over NVLink), makes them visible (fence at system scope) and writes e
// into flag [r][c] of every rank; it then waits until its own flags [0..world)[c] all hold e (or more: a
// peer can be one all-reduce ahead) and adds
// the `world` slices of its own receive area in rank order, so every rank computes bit-identical
// sums.  Two slots are enough: a rank can only start e+2 after every peer has delivered e+1, which a
// peer does only after it finished reading e.  The wait is bounded; when it gives up it sets the
// context's error word and the step goes on with whatever arrived.
// ---------------------------------------------------------------------------------------------
constexpr int TP_AR_THREADS = 256;
constexpr size_t TP_AR_CAP_FLOATS = 256 * 1024;    // largest vector the peer path takes (1 MB per slot: batch 32 x 8192)

__global__ void __launch_bounds__(TP_AR_THREADS) tp_ar_resid_kernel(const float *__restrict__ part, uint16_t *h,
                                                                    uint32_t n, void *const *peer_tab,
                                                                    float *recv, unsigned int *flags,
                                                                    unsigned int *state, uint32_t world,
                                                                    uint32_t rank, uint32_t cap,
                                                                    unsigned int *err, uint32_t spin_limit) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t cta = blockIdx.x, tid = threadIdx.x;
    const unsigned int e = state[0] + 1;  // stable: the previous all-reduce kernel has completed
    const uint32_t slot = e & 1;
    const uint32_t i = (cta * TP_AR_THREADS + tid) * 4;
    // ---- deliver this CTA's slice to every rank ----
    if (i < n) {
        const float4 v = *reinterpret_cast<const float4 *>(part + i);
        for (uint32_t q = 0; q < world; q++) {
            float *dst = static_cast<float *>(peer_tab[q]) + ((size_t)slot * world + rank) * cap + i;
            *reinterpret_cast<float4 *>(dst) = v;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (tid < world) {
        unsigned int *f = static_cast<unsigned int *>(peer_tab[world + tid]) + rank * TP_AR_MAX_CTAS + cta;
        asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(f), "r"(e) : "memory");
    }
    // ---- wait for the same slice of every rank (bounded: spin_limit polls, then error code 3) ----
    if (tid < world) {
        const unsigned int *f = flags + tid * TP_AR_MAX_CTAS + cta;
        unsigned int seen = 0, polls = 0;
        for (;;) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(seen) : "l"(f) : "memory");
            if ((int)(seen - e) >= 0) break;  // a peer that is already one all-reduce ahead has delivered this one too
            if (++polls > spin_limit) {
                atomicExch(err, 3u);  // a peer did not deliver: reported by the next host call
                break;
            }
            if (polls > 64) __nanosleep(polls > 4096 ? 500 : 50);
        }
    }
    __syncthreads();
    // ---- add in rank order, round, add the residual ----
    if (i < n) {
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t r = 0; r < world; r++) {
            const float4 v = __ldcg(reinterpret_cast<const float4 *>(recv + ((size_t)slot * world + r) * cap + i));
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        uint2 hv = *reinterpret_cast<const uint2 *>(h + i);
        const __half2 h01 = *reinterpret_cast<const __half2 *>(&hv.x), h23 = *reinterpret_cast<const __half2 *>(&hv.y);
        const float o0 = __half2float(__float2half_rn(s.x)) + __low2float(h01);
        const float o1 = __half2float(__float2half_rn(s.y)) + __high2float(h01);
        const float o2 = __half2float(__float2half_rn(s.z)) + __low2float(h23);
        const float o3 = __half2float(__float2half_rn(s.w)) + __high2float(h23);
        const __half2 r01 = __floats2half2_rn(o0, o1), r23 = __floats2half2_rn(o2, o3);
        hv.x = *reinterpret_cast<const unsigned int *>(&r01);
        hv.y = *reinterpret_cast<const unsigned int *>(&r23);
        *reinterpret_cast<uint2 *>(h + i) = hv;
    }
    // ---- the last CTA to finish advances the epoch ----
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(&state[1], 1u) == gridDim.x - 1) {
            state[1] = 0;
            state[0] = e;
        }
    }
}

// The flagged-word area follows the float slots inside the same allocation (one IPC handle covers both).
static size_t tp_ll_offset(int world) { return 2ull * world * TP_AR_CAP_FLOATS * sizeof(float); }

int tp_fill_push(prism_cuda_ctx *ctx, const LutTensor &t, TpPush *out) {
    if (ctx->tp_world <= 1 || ctx->tp_cap == 0 || !ctx->tp_peer_tab)
        return fail(ctx, PRISM_E_STATE, "fused all-reduce: the peer-memory path is not set up" +
                                            (ctx->tp_peer_reason.empty() ? std::string() : ": " + ctx->tp_peer_reason));
    if (t.n_hb > (uint32_t)TP_AR_MAX_CTAS || t.m_pad > ctx->tp_cap)
        return fail(ctx, PRISM_E_ARG, "fused all-reduce: output vector too long for the receive area");
    out->peer_tab = (void *const *)ctx->tp_peer_tab;
    out->recv = ctx->tp_recv;
    out->flags = ctx->tp_flags;
    out->state = ctx->tp_state;
    out->world = (uint32_t)ctx->tp_world;
    out->rank = (uint32_t)ctx->tp_rank;
    out->cap = (uint32_t)ctx->tp_cap;
    out->spin_limit = wait_limit(ctx, TP_AR_SPIN_LIMIT);
    out->n_units = t.n_hb;
    out->deliver_only = (ctx->tp_fused_ar == 1 || ctx->tp_fused_ar == 3) ? 1u : 0u;
    out->ll_off = ctx->tp_fused_ar >= 3 ? (uint32_t)tp_ll_offset(ctx->tp_world) : 0u;
    if (out->ll_off && t.m_pad > TP_LL_CAP) return fail(ctx, PRISM_E_ARG, "fused all-reduce: output vector too long for the flagged-word area");
    return PRISM_OK;
}

bool gemv_tp_ok(prism_cuda_ctx *ctx, const LutTensor &t) {
    if (ctx->tp_fused_ar >= 3 && t.m_pad > TP_LL_CAP) return false;
    return ctx->tp_world > 1 && ctx->tp_peer_ar && ctx->tp_fused_ar && ctx->tp_cap != 0 && ctx->gemv_variant == 1 && t.bits == 4 &&
           t.k % 32 == 0 && t.k >= 32 && t.n_hb <= (uint32_t)TP_AR_MAX_CTAS && t.m_pad <= ctx->tp_cap;
}

// The second half of the all-reduce when the GEMV kernel has already delivered this rank's partial sums into
// every rank's receive area (GEMV_TP with deliver_only): that kernel has completed, so its stores to peer
// memory are performed; CTA c publishes flag [rank][c], waits for the same flag of every rank (bounded), adds
// the slices in rank order, rounds, adds the residual.  No data crosses NVLink here, only the flags.
__global__ void __launch_bounds__(TP_AR_THREADS) tp_ar_flags_resid_kernel(uint16_t *h, uint32_t n, void *const *peer_tab,
                                                                          const float *recv, unsigned int *flags,
                                                                          unsigned int *state, uint32_t world, uint32_t rank,
                                                                          uint32_t cap, unsigned int *err, uint32_t spin_limit) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t cta = blockIdx.x, tid = threadIdx.x;
    const unsigned int e = state[0] + 1;
    const uint32_t slot = e & 1;
    const uint32_t i = (cta * TP_AR_THREADS + tid) * 4;
    if (tid < world) {
        unsigned int *f = static_cast<unsigned int *>(peer_tab[world + tid]) + rank * TP_AR_MAX_CTAS + cta;
        asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(f), "r"(e) : "memory");
        const unsigned int *fw = flags + tid * TP_AR_MAX_CTAS + cta;
        unsigned int seen = 0, polls = 0;
        for (;;) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(seen) : "l"(fw) : "memory");
            if ((int)(seen - e) >= 0) break;
            if (++polls > spin_limit) {
                atomicExch(err, 3u);
                break;
            }
            if (polls > 64) __nanosleep(polls > 4096 ? 500 : 50);
        }
    }
    __syncthreads();
    if (i < n) {
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t r = 0; r < world; r++) {
            const float4 v = __ldcg(reinterpret_cast<const float4 *>(recv + ((size_t)slot * world + r) * cap + i));
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        uint2 hv = *reinterpret_cast<const uint2 *>(h + i);
        const __half2 h01 = *reinterpret_cast<const __half2 *>(&hv.x), h23 = *reinterpret_cast<const __half2 *>(&hv.y);
        const float o0 = __half2float(__float2half_rn(s.x)) + __low2float(h01);
        const float o1 = __half2float(__float2half_rn(s.y)) + __high2float(h01);
        const float o2 = __half2float(__float2half_rn(s.z)) + __low2float(h23);
        const float o3 = __half2float(__float2half_rn(s.w)) + __high2float(h23);
        const __half2 r01 = __floats2half2_rn(o0, o1), r23 = __floats2half2_rn(o2, o3);
        hv.x = *reinterpret_cast<const unsigned int *>(&r01);
        hv.y = *reinterpret_cast<const unsigned int *>(&r23);
        *reinterpret_cast<uint2 *>(h + i) = hv;
    }
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(&state[1], 1u) == gridDim.x - 1) {
            state[1] = 0;
            state[0] = e;
        }
    }
}

int tp_all_reduce_flags_resid(prism_cuda_ctx *ctx, uint16_t *h, size_t n) {
    if (!tp_peer_ar_ok(ctx, n)) return fail(ctx, PRISM_E_STATE, "peer-memory all-reduce not available for this size");
    const unsigned ctas = (unsigned)((n + TP_AR_THREADS * 4 - 1) / (TP_AR_THREADS * 4));
    launch_pdl(ctx, "tp_ar_flags_resid_kernel", tp_ar_flags_resid_kernel, dim3(ctas), dim3(TP_AR_THREADS), 0, h, (uint32_t)n,
               (void *const *)ctx->tp_peer_tab, (const float *)ctx->tp_recv, ctx->tp_flags, ctx->tp_state, (uint32_t)ctx->tp_world,
               (uint32_t)ctx->tp_rank, (uint32_t)ctx->tp_cap, ctx->dev_err, wait_limit(ctx, TP_AR_SPIN_LIMIT));
    return after_launch(ctx, "tp_ar_flags_resid_kernel");
}

// The reduction when the GEMV kernel has delivered flagged words (GEMV_TP, ll_off != 0): every word carries the
// epoch it belongs to, so nothing but the data crosses NVLink -- no fence at system scope, no flag stores, no
// second trip.  One thread per output row loads the `world` words of its row, re-polls (bounded) the ones that
// have not arrived, adds them in rank order, rounds and adds the residual.  64-thread CTAs with few registers:
// they fit beside a GEMV CTA that owns the rest of an SM, so the grid is resident before the GEMV ends.
constexpr int TP_LL_THREADS = 64;
__device__ __forceinline__ unsigned long long tp_ll_load(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];\n" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__global__ void __launch_bounds__(TP_LL_THREADS) tp_ar_ll_resid_kernel(uint16_t *h, uint32_t n, const unsigned long long *ll,
                                                                       unsigned int *state, uint32_t world, unsigned int *err,
                                                                       uint32_t spin_limit) {
    pdl_launch_dependents();
    pdl_wait();  // the delivering GEMV and everything before it (the previous reduction, which advanced the epoch) are complete
    const uint32_t row = blockIdx.x * TP_LL_THREADS + threadIdx.x;
    const unsigned int e = *reinterpret_cast<volatile unsigned int *>(state) + 1;
    if (row < n) {
        const unsigned long long *p = ll + (size_t)(e & 1) * world * TP_LL_CAP + row;
        unsigned long long v[16];
#pragma unroll
        for (uint32_t r = 0; r < 16; r++) v[r] = r < world ? tp_ll_load(p + (size_t)r * TP_LL_CAP) : 0ull;
        unsigned int polls = 0;
        for (;;) {
            bool all = true;
#pragma unroll
            for (uint32_t r = 0; r < 16; r++) {
                if (r < world && (unsigned int)(v[r] >> 32) != e) {
                    all = false;
                    v[r] = tp_ll_load(p + (size_t)r * TP_LL_CAP);
                }
            }
            if (all) break;
            if (++polls > spin_limit) {
                atomicExch(err, 3u);  // a peer did not deliver: reported by the next synchronising host call
                break;
            }
            if (polls > 64) __nanosleep(polls > 4096 ? 500 : 50);
        }
        float s = 0.0f;
#pragma unroll
        for (uint32_t r = 0; r < 16; r++)
            if (r < world) s += __uint_as_float((unsigned int)v[r]);
        const float o = __half2float(__float2half_rn(s)) + __half2float(__ushort_as_half(h[row]));
        h[row] = __half_as_ushort(__float2half_rn(o));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&state[1], 1u) == gridDim.x - 1) {
            state[1] = 0;
            state[0] = e;
        }
    }
}

int tp_all_reduce_ll_resid(prism_cuda_ctx *ctx, uint16_t *h, size_t n) {
    if (ctx->tp_world <= 1 || ctx->tp_cap == 0 || n > TP_LL_CAP || ctx->tp_world > 16)
        return fail(ctx, PRISM_E_STATE, "flagged-word all-reduce not available for this size");
    const unsigned ctas = (unsigned)((n + TP_LL_THREADS - 1) / TP_LL_THREADS);
    const unsigned long long *ll =
        reinterpret_cast<const unsigned long long *>(reinterpret_cast<const char *>(ctx->tp_recv) + tp_ll_offset(ctx->tp_world));
    launch_pdl(ctx, "tp_ar_ll_resid_kernel", tp_ar_ll_resid_kernel, dim3(ctas), dim3(TP_LL_THREADS), 0, h, (uint32_t)n, ll,
               ctx->tp_state, (uint32_t)ctx->tp_world, ctx->dev_err, wait_limit(ctx, TP_AR_SPIN_LIMIT));
    return after_launch(ctx, "tp_ar_ll_resid_kernel");
}

bool tp_peer_ar_ok(prism_cuda_ctx *ctx, size_t n) {
    return ctx->tp_world > 1 && ctx->tp_peer_ar && ctx->tp_cap != 0 && n <= ctx->tp_cap && n % 4 == 0 &&
           (n + TP_AR_THREADS * 4 - 1) / (TP_AR_THREADS * 4) <= (size_t)TP_AR_MAX_CTAS;
}

int tp_all_reduce_resid_peer(prism_cuda_ctx *ctx, const float *part, uint16_t *h, size_t n) {
    if (!tp_peer_ar_ok(ctx, n))
        return fail(ctx, PRISM_E_STATE, "peer-memory all-reduce not available" +
                                            (ctx->tp_peer_reason.empty() ? std::string(" for this size") : ": " + ctx->tp_peer_reason));
    const unsigned ctas = (unsigned)((n + TP_AR_THREADS * 4 - 1) / (TP_AR_THREADS * 4));
    launch_pdl(ctx, "tp_ar_resid_kernel", tp_ar_resid_kernel, dim3(ctas), dim3(TP_AR_THREADS), 0, part, h, (uint32_t)n,
               (void *const *)ctx->tp_peer_tab, ctx->tp_recv, ctx->tp_flags, ctx->tp_state, (uint32_t)ctx->tp_world,
               (uint32_t)ctx->tp_rank, (uint32_t)ctx->tp_cap, ctx->dev_err, wait_limit(ctx, TP_AR_SPIN_LIMIT));
    return after_launch(ctx, "tp_ar_resid_kernel");
}

static void tp_peer_release(prism_cuda_ctx *ctx) {
    for (int q = 0; q < 32; q++) {
        if (ctx->tp_peer_map[q]) {
            cudaIpcCloseMemHandle(ctx->tp_peer_map[q]);
            ctx->tp_peer_map[q] = nullptr;
        }
    }
    cudaFree(ctx->tp_recv);
    cudaFree(ctx->tp_flags);
    cudaFree(ctx->tp_state);
    cudaFree(ctx->tp_peer_tab);
    ctx->tp_recv = nullptr; ctx->tp_flags = nullptr; ctx->tp_state = nullptr; ctx->tp_peer_tab = nullptr;
    ctx->tp_cap = 0;
}

// This rank's receive area, flags, epoch state and the (still empty) pointer table.
static bool tp_peer_alloc(prism_cuda_ctx *ctx, int T, std::string &why) {
    const size_t ll_bytes = 2ull * T * TP_LL_CAP * sizeof(unsigned long long);  // epoch 0 in every word: nothing delivered
    const size_t recv_bytes = tp_ll_offset(T) + ll_bytes;
    const size_t flag_bytes = (size_t)T * TP_AR_MAX_CTAS * sizeof(unsigned int);
    cudaError_t e;
    if ((e = cudaMalloc((void **)&ctx->tp_recv, recv_bytes)) != cudaSuccess ||
        (e = cudaMalloc((void **)&ctx->tp_flags, flag_bytes)) != cudaSuccess ||
        (e = cudaMalloc((void **)&ctx->tp_state, 2 * sizeof(unsigned int))) != cudaSuccess ||
        (e = cudaMalloc((void **)&ctx->tp_peer_tab, 2 * T * sizeof(void *))) != cudaSuccess ||
        (e = cudaMemsetAsync(ctx->tp_flags, 0, flag_bytes, ctx->stream)) != cudaSuccess ||
        (e = cudaMemsetAsync(reinterpret_cast<char *>(ctx->tp_recv) + tp_ll_offset(T), 0, ll_bytes, ctx->stream)) != cudaSuccess ||
        (e = cudaMemsetAsync(ctx->tp_state, 0, 2 * sizeof(unsigned int), ctx->stream)) != cudaSuccess) {
        why = std::string("receive area allocation: ") + cudaGetErrorString(e);
        (void)cudaGetLastError();
        return false;
    }
    return true;
}

// Allocates this rank's receive area and flags, exchanges the IPC handles through NCCL and maps the
// peers'.  A rank on which a local step fails still takes part in both collectives (with a zeroed
// handle and a "not ok" vote), so no peer is left waiting inside NCCL; the outcome is agreed with a
// min-reduce and every rank takes the same path.  On failure tp_cap stays 0 (the engine then reduces
// with ncclAllReduce), everything allocated here is freed and tp_peer_reason says why.
static int tp_peer_setup(prism_cuda_ctx *ctx) {
    const int T = ctx->tp_world;
    ctx->tp_peer_reason.clear();
    if (T > 16) {
        ctx->tp_peer_reason = "more than 16 ranks";
        return PRISM_OK;
    }
    struct Handles { cudaIpcMemHandle_t recv, flags; };
    Handles mine{};
    std::vector<Handles> all(T);
    std::string why;
    bool ok = tp_peer_alloc(ctx, T, why);
    if (ok) {
        cudaError_t e;
        if ((e = cudaIpcGetMemHandle(&mine.recv, ctx->tp_recv)) != cudaSuccess ||
            (e = cudaIpcGetMemHandle(&mine.flags, ctx->tp_flags)) != cudaSuccess) {
            why = std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(e);
            (void)cudaGetLastError();
            mine = Handles{};
            ok = false;
        }
    }
    // ---- collective 1: everybody's handles (a rank that failed above sends zeros) ----
    Handles *all_dev = nullptr;
    float *flag_dev = nullptr;
    const bool have_tmp = cudaMalloc((void **)&all_dev, sizeof(Handles) * (T + 1)) == cudaSuccess &&
                          cudaMalloc((void **)&flag_dev, sizeof(float)) == cudaSuccess;
    if (!have_tmp) {
        // Without these few bytes this rank cannot even vote; the peers' collectives would wait for it.
        // Report it as an error of tp_init instead of silently degrading.
        (void)cudaGetLastError();
        cudaFree(all_dev);
        cudaFree(flag_dev);
        tp_peer_release(ctx);
        return fail(ctx, PRISM_E_CUDA, "tensor parallel set-up: out of device memory for the handle exchange");
    }
    cudaMemcpyAsync(all_dev + T, &mine, sizeof(Handles), cudaMemcpyHostToDevice, ctx->stream);
    int rc = tp_all_gather_bytes(ctx, all_dev + T, all_dev, sizeof(Handles));
    if (rc == PRISM_OK) {
        cudaMemcpyAsync(all.data(), all_dev, sizeof(Handles) * T, cudaMemcpyDeviceToHost, ctx->stream);
        if (cudaStreamSynchronize(ctx->stream) != cudaSuccess) rc = PRISM_E_CUDA;
    }
    if (rc != PRISM_OK && ok) {
        why = "all-gather of the IPC handles failed";
        ok = false;
    }
    std::vector<void *> tab(2 * T, nullptr);
    for (int q = 0; q < T && ok; q++) {
        if (q == ctx->tp_rank) {
            tab[q] = ctx->tp_recv;
            tab[T + q] = ctx->tp_flags;
            continue;
        }
        void *pr = nullptr, *pf = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&pr, all[q].recv, cudaIpcMemLazyEnablePeerAccess);
        if (e == cudaSuccess) {
            ctx->tp_peer_map[q] = pr;
            e = cudaIpcOpenMemHandle(&pf, all[q].flags, cudaIpcMemLazyEnablePeerAccess);
            if (e == cudaSuccess) ctx->tp_peer_map[16 + q] = pf;
        }
        if (e != cudaSuccess) {
            why = "cudaIpcOpenMemHandle(rank " + std::to_string(q) + "): " + cudaGetErrorString(e);
            (void)cudaGetLastError();
            ok = false;
            break;
        }
        tab[q] = pr;
        tab[T + q] = pf;
    }
    if (ok && cudaMemcpy(ctx->tp_peer_tab, tab.data(), 2 * T * sizeof(void *), cudaMemcpyHostToDevice) != cudaSuccess) {
        why = "copy of the peer pointer table failed";
        (void)cudaGetLastError();
        ok = false;
    }
    // ---- collective 2: every rank must take the same path: agree on the outcome (min over ranks) ----
    float flag_host = ok ? 1.0f : 0.0f;
    cudaMemcpyAsync(flag_dev, &flag_host, sizeof(float), cudaMemcpyHostToDevice, ctx->stream);
    ncclResult_t r = ctx->nccl->AllReduce(flag_dev, flag_dev, 1, ncclFloat32, ncclMin, (ncclComm_t)ctx->nccl_comm, ctx->stream);
    cudaMemcpyAsync(&flag_host, flag_dev, sizeof(float), cudaMemcpyDeviceToHost, ctx->stream);
    cudaStreamSynchronize(ctx->stream);
    cudaFree(all_dev);
    cudaFree(flag_dev);
    if (r != ncclSuccess || flag_host < 0.5f) {
        if (ok) why = r != ncclSuccess ? "the agreement all-reduce failed" : "another rank could not map its peers";
        tp_peer_release(ctx);
        ctx->tp_peer_reason = why;
        return PRISM_OK;
    }
    ctx->tp_cap = TP_AR_CAP_FLOATS;
    return PRISM_OK;
}

}  // namespace prism

using namespace prism;

extern "C" void prism_tp_shutdown(prism_cuda_ctx *ctx) {
    tp_peer_release(ctx);
    if (ctx->nccl_comm && ctx->nccl) {
        ctx->nccl->CommDestroy((ncclComm_t)ctx->nccl_comm);
        ctx->nccl_comm = nullptr;
    }
}

extern "C" {

int prism_cuda_tp_unique_id(uint8_t id[PRISM_NCCL_ID_BYTES]) {
    if (!id) return PRISM_E_NULL;
    std::string err;
    prism_nccl_api *api = load_nccl(err);
    if (!api) return fail(nullptr, PRISM_E_COMM, err);
    static_assert(sizeof(ncclUniqueId) == PRISM_NCCL_ID_BYTES, "ncclUniqueId size");
    ncclUniqueId uid;
    ncclResult_t r = api->GetUniqueId(&uid);
    if (r != ncclSuccess) return fail(nullptr, PRISM_E_COMM, std::string("ncclGetUniqueId: ") + api->GetErrorString(r));
    memcpy(id, &uid, PRISM_NCCL_ID_BYTES);
    return PRISM_OK;
}

int prism_cuda_tp_init(prism_cuda_ctx *ctx, int world, int rank, const uint8_t id[PRISM_NCCL_ID_BYTES]) {
    if (!ctx || !id) return fail(ctx, PRISM_E_NULL, "null argument");
    if (world < 1 || rank < 0 || rank >= world) return fail(ctx, PRISM_E_ARG, "bad world/rank");
    if (ctx->nccl_comm) return fail(ctx, PRISM_E_STATE, "tensor parallel group already initialised");
    ctx->tp_world = world;
    ctx->tp_rank = rank;
    if (world == 1) return PRISM_OK;
    std::string err;
    prism_nccl_api *api = load_nccl(err);
    if (!api) return fail(ctx, PRISM_E_COMM, err);
    PRISM_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    ncclUniqueId uid;
    memcpy(&uid, id, PRISM_NCCL_ID_BYTES);
    ncclComm_t comm;
    ncclResult_t r = api->CommInitRank(&comm, world, uid, rank);
    if (r != ncclSuccess) {
        ctx->tp_world = 1;
        ctx->tp_rank = 0;
        return fail(ctx, PRISM_E_COMM, std::string("ncclCommInitRank: ") + api->GetErrorString(r));
    }
    ctx->nccl = api;
    ctx->nccl_comm = comm;
    return tp_peer_setup(ctx);
}

int prism_cuda_tp_world(prism_cuda_ctx *ctx, int *world, int *rank) {
    if (!ctx) return PRISM_E_NULL;
    if (world) *world = ctx->tp_world;
    if (rank) *rank = ctx->tp_rank;
    return PRISM_OK;
}

int prism_cuda_tp_peer_ready(prism_cuda_ctx *ctx) { return (ctx && ctx->tp_world > 1 && ctx->tp_cap != 0) ? 1 : 0; }

const char *prism_cuda_tp_peer_reason(prism_cuda_ctx *ctx) { return ctx ? ctx->tp_peer_reason.c_str() : ""; }

int prism_cuda_tp_init_loopback(prism_cuda_ctx *ctx, int world, int rank) {
    if (!ctx) return PRISM_E_NULL;
    if (world < 2 || world > 16 || rank < 0 || rank >= world) return fail(ctx, PRISM_E_ARG, "bad world/rank");
    if (ctx->nccl_comm || ctx->tp_cap) return fail(ctx, PRISM_E_STATE, "tensor parallel group already initialised");
    PRISM_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    std::string why;
    if (!tp_peer_alloc(ctx, world, why)) {
        tp_peer_release(ctx);
        return fail(ctx, PRISM_E_CUDA, why);
    }
    // every "peer" is this GPU's own receive area and flag array: rank `rank` delivers to itself, the
    // other ranks' slices and flags are never written
    std::vector<void *> tab(2 * world, nullptr);
    for (int q = 0; q < world; q++) {
        tab[q] = ctx->tp_recv;
        tab[world + q] = ctx->tp_flags;
    }
    cudaError_t e = cudaMemcpy(ctx->tp_peer_tab, tab.data(), 2 * world * sizeof(void *), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        tp_peer_release(ctx);
        return cuda_fail(ctx, e, "cudaMemcpy(peer table)");
    }
    ctx->tp_world = world;
    ctx->tp_rank = rank;
    ctx->tp_loopback = true;
    ctx->tp_cap = TP_AR_CAP_FLOATS;
    return PRISM_OK;
}

int prism_cuda_tp_all_reduce_resid_dev(prism_cuda_ctx *ctx, const void *partial_f32_dev, void *h_f16_dev, size_t n) {
    if (!ctx || !partial_f32_dev || !h_f16_dev) return fail(ctx, PRISM_E_NULL, "null argument");
    if (n == 0) return PRISM_OK;
    if ((reinterpret_cast<uintptr_t>(partial_f32_dev) & 15) || (reinterpret_cast<uintptr_t>(h_f16_dev) & 7))
        return fail(ctx, PRISM_E_ARG, "all_reduce_resid: partial sums must be 16-byte aligned, h 8-byte aligned");
    return tp_all_reduce_resid_peer(ctx, static_cast<const float *>(partial_f32_dev), static_cast<uint16_t *>(h_f16_dev), n);
}

int prism_cuda_tp_all_reduce_dev(prism_cuda_ctx *ctx, void *buf_dev, size_t n_halfs) {
    if (!ctx || !buf_dev) return fail(ctx, PRISM_E_NULL, "null argument");
    if (ctx->tp_world <= 1) return PRISM_OK;
    if (!ctx->nccl || !ctx->nccl_comm) return fail(ctx, PRISM_E_STATE, "no NCCL communicator on this context");
    ncclResult_t r = ctx->nccl->AllReduce(buf_dev, buf_dev, n_halfs, ncclFloat16, ncclSum,
                                          (ncclComm_t)ctx->nccl_comm, ctx->stream);
    if (r != ncclSuccess) return fail(ctx, PRISM_E_COMM, std::string("ncclAllReduce: ") + ctx->nccl->GetErrorString(r));
    ctx->launches++;
    return PRISM_OK;
}

}  // extern "C"
