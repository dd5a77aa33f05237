// extern "C" surface of the backend (include/prism_cuda.h): context, weight
// upload / re-lay, and the host-pointer wrappers around the kernels.
#include <cstdio>
#include <cstring>

#include "../../include/prism_cuda_bench.h"
#include "common.cuh"
#include "pair_table.cuh"
#include "scratch.hpp"

namespace prism {

static thread_local std::string g_create_err;

int fail(prism_cuda_ctx *ctx, int code, const std::string &msg) {
    if (ctx) ctx->err = msg;
    else g_create_err = msg;
    return code;
}

int cuda_fail(prism_cuda_ctx *ctx, cudaError_t e, const char *what) {
    std::string m = std::string(what) + ": " + cudaGetErrorString(e);
    return fail(ctx, PRISM_E_CUDA, m);
}

int after_launch(prism_cuda_ctx *ctx, const char *kernel) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(ctx, e, kernel);
    ctx->launches++;
    return PRISM_OK;
}

// cudaMalloc / cudaFree behind the allocator interface of grow_buf (scratch.hpp).
struct CudaScratchAlloc {
    prism_cuda_ctx *ctx;
    cudaError_t last = cudaSuccess;
    const char *what = "";
    int sync() { what = "cudaStreamSynchronize"; last = cudaStreamSynchronize(ctx->stream); return last == cudaSuccess ? 0 : 1; }
    int release(void *p) { what = "cudaFree"; last = cudaFree(p); return last == cudaSuccess ? 0 : 1; }
    int acquire(void **p, size_t bytes) { what = "cudaMalloc"; last = cudaMalloc(p, bytes); return last == cudaSuccess ? 0 : 1; }
};

// Grows one of the context's scratch buffers to `want` elements.  Pointer and element count are
// written back whatever happens: after a failed allocation both are zero, never a stale size
// beside a null pointer.
template <typename T>
static int grow(prism_cuda_ctx *ctx, T **p, size_t *have, size_t want, bool *grew = nullptr) {
    GrowBuf b{*p, *have};
    CudaScratchAlloc al{ctx};
    const int rc = grow_buf(al, b, want, sizeof(T), grew);
    *p = static_cast<T *>(b.ptr);
    *have = b.count;
    if (rc) {
        (void)cudaGetLastError();
        return cuda_fail(ctx, al.last, al.what);
    }
    return PRISM_OK;
}

int ensure_stage(prism_cuda_ctx *ctx, size_t in_bytes, size_t out_bytes) {
    PRISM_TRY(grow(ctx, &ctx->stage_in, &ctx->stage_in_bytes, in_bytes));
    return grow(ctx, &ctx->stage_out, &ctx->stage_out_bytes, out_bytes);
}

int ensure_splitk(prism_cuda_ctx *ctx, size_t floats, size_t counters) {
    PRISM_TRY(grow(ctx, &ctx->splitk_partials, &ctx->splitk_floats, floats));
    bool grew = false;
    PRISM_TRY(grow(ctx, &ctx->splitk_counters, &ctx->splitk_counter_n, counters, &grew));
    // arrival counters start at zero; each kernel leaves them at zero again
    if (grew)
        PRISM_CUDA_TRY(ctx, cudaMemsetAsync(ctx->splitk_counters, 0, ctx->splitk_counter_n * sizeof(unsigned int), ctx->stream));
    return PRISM_OK;
}

int ensure_act(prism_cuda_ctx *ctx, size_t halfs) { return grow(ctx, &ctx->act_scratch, &ctx->act_halfs, halfs); }

int ensure_tmp(prism_cuda_ctx *ctx, size_t halfs) { return grow(ctx, &ctx->tmp_scratch, &ctx->tmp_halfs, halfs); }

int check_device_error(prism_cuda_ctx *ctx) {
    unsigned int v = 0;
    PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(&v, ctx->dev_err, 4, cudaMemcpyDeviceToHost, ctx->stream));
    PRISM_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return device_error_result(ctx, v);
}

int device_error_result(prism_cuda_ctx *ctx, unsigned int v) {
    if (v == 0) return PRISM_OK;
    cudaMemsetAsync(ctx->dev_err, 0, 4, ctx->stream);  // reported once; the context stays usable
    const std::string code = " (device code " + std::to_string(v) + ")";
    switch (v) {
    case 1:
        return fail(ctx, PRISM_E_STATE, "a kernel refused to run: dynamic shared memory does not start where the table lookups assume" + code);
    case 2:
        return fail(ctx, PRISM_E_TIMEOUT, "a warp-specialised GEMV gave up waiting for its own stage hand-over; its output is incomplete" + code);
    case 3:
        return fail(ctx, PRISM_E_TIMEOUT, "peer-memory all-reduce: a tensor-parallel peer did not deliver its partial sums within the wait "
                                          "limit; the step went on with what had arrived and its result is not valid" + code);
    case 4:
        return fail(ctx, PRISM_E_TIMEOUT, "a grid-wide arrival inside a persistent kernel gave up; its output is incomplete" + code);
    case 6:
        return fail(ctx, PRISM_E_STATE, "the cluster GEMV was not launched with the cluster shape it was given" + code);
    case 5:
        return fail(ctx, PRISM_E_TIMEOUT, "a tcgen05 kernel gave up waiting on an mbarrier; its output is incomplete" + code);
    default:
        return fail(ctx, PRISM_E_STATE, "a kernel reported an unknown error" + code);
    }
}

LutTensor *get_tensor(prism_cuda_ctx *ctx, int32_t handle) {
    if (!ctx || handle < 0 || (size_t)handle >= ctx->tensors.size() || !ctx->tensors[handle].live) {
        if (ctx) ctx->err = "miss handle " + std::to_string(handle);
        return nullptr;
    }
    return &ctx->tensors[handle];
}

int alloc_tensor(prism_cuda_ctx *ctx, const char *name, uint32_t m, uint32_t k, uint32_t bits,
                 int32_t *handle) {
    if (bits != 2 && bits != 4) return fail(ctx, PRISM_E_ARG, "bits must be 2 or 4");
    if (m == 0 || k == 0) return fail(ctx, PRISM_E_ARG, "empty tensor");
    if (((uint64_t)k * bits) % 32 != 0)
        return fail(ctx, PRISM_E_ARG, "dim_n*bits must be a multiple of 32 (whole index words per row)");
    LutTensor t;
    t.name = name ? name : "";
    t.m = m; t.k = k; t.bits = bits;
    t.m_pad = round_up_u32(m, 64);
    t.n_hb = t.m_pad / 32;
    t.row_bytes = (uint32_t)((uint64_t)k * bits / 8);
    t.n_chunks = (t.row_bytes + 15) / 16;
    t.idx_bytes = (size_t)t.n_hb * t.n_chunks * 512;
    t.pal_bytes = (size_t)t.m_pad * t.n_ent() * 2;
    PRISM_CUDA_TRY(ctx, cudaMalloc((void **)&t.idx, t.idx_bytes));
    cudaError_t e = cudaMalloc((void **)&t.pal, t.pal_bytes);
    if (e != cudaSuccess) {
        cudaFree(t.idx);
        return cuda_fail(ctx, e, "cudaMalloc(palettes)");
    }
    t.live = true;
    int32_t h = (int32_t)ctx->tensors.size();
    ctx->tensors.push_back(t);
    if (!t.name.empty()) ctx->by_name[t.name] = h;
    *handle = h;
    return PRISM_OK;
}

int synth_shard(prism_cuda_ctx *ctx, const char *name, uint32_t rows, uint32_t cols, uint32_t bits,
                uint64_t seed, float sigma, uint32_t row0, uint32_t col0, int32_t *handle) {
    if (!ctx || !handle) return fail(ctx, PRISM_E_NULL, "null argument");
    *handle = -1;
    if (bits != 2 && bits != 4) return fail(ctx, PRISM_E_ARG, "bits must be 2 or 4");
    if (col0 % (128 / bits)) return fail(ctx, PRISM_E_ARG, "shard column offset must be a multiple of 128/bits");
    PRISM_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    int32_t h;
    PRISM_TRY(alloc_tensor(ctx, name, rows, cols, bits, &h));
    PRISM_TRY(launch_synth(ctx, ctx->tensors[h], seed, sigma, row0, col0));
    *handle = h;
    return PRISM_OK;
}

}  // namespace prism

using namespace prism;

extern "C" {

int prism_cuda_create(int device, prism_cuda_ctx **out) {
    if (!out) return fail(nullptr, PRISM_E_NULL, "null out pointer");
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0)
        return fail(nullptr, PRISM_E_CUDA, std::string("No CUDA device: ") + cudaGetErrorString(e));
    if (device < 0 || device >= n || device >= PRISM_MAX_DEVICES) return fail(nullptr, PRISM_E_ARG, "device index out of range");
    cudaDeviceProp p;
    if ((e = cudaGetDeviceProperties(&p, device)) != cudaSuccess) return cuda_fail(nullptr, e, "cudaGetDeviceProperties");
    if (p.major != 10)
        return fail(nullptr, PRISM_E_ARG,
                    "this library is built for sm_100a (compute capability 10.x); device is " +
                        std::to_string(p.major) + "." + std::to_string(p.minor));
    if ((e = cudaSetDevice(device)) != cudaSuccess) return cuda_fail(nullptr, e, "cudaSetDevice");
    prism_cuda_ctx *ctx = new prism_cuda_ctx();
    ctx->device = device;
    ctx->sm_count = p.multiProcessorCount;
    if ((e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking)) != cudaSuccess) {
        delete ctx;
        return cuda_fail(nullptr, e, "cudaStreamCreate");
    }
    if ((e = cudaMalloc((void **)&ctx->dev_err, 64)) != cudaSuccess) {
        cudaStreamDestroy(ctx->stream);
        delete ctx;
        return cuda_fail(nullptr, e, "cudaMalloc");
    }
    int rc = probe_smem_base(ctx);
    if (rc != PRISM_OK) {
        g_create_err = ctx->err;
        prism_cuda_destroy(ctx);
        return rc;
    }
    *out = ctx;
    return PRISM_OK;
}

void prism_cuda_destroy(prism_cuda_ctx *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (auto &t : ctx->tensors) {
        if (t.live) {
            cudaFree(t.idx);
            cudaFree(t.pal);
        }
    }
    cudaFree(ctx->stage_in);
    cudaFree(ctx->stage_out);
    cudaFree(ctx->splitk_partials);
    cudaFree(ctx->splitk_counters);
    cudaFree(ctx->act_scratch);
    cudaFree(ctx->tmp_scratch);
    cudaFree(ctx->dev_err);
    cudaFree(ctx->kv_k);
    cudaFree(ctx->kv_v);
    for (auto *t : ctx->rope_tabs) {
        cudaFree(t->dev);
        delete t;
    }
    extern void prism_tp_shutdown(prism_cuda_ctx *);
    prism_tp_shutdown(ctx);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
}

const char *prism_cuda_last_error(prism_cuda_ctx *ctx) { return ctx ? ctx->err.c_str() : g_create_err.c_str(); }

void *prism_cuda_stream(prism_cuda_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }

int prism_cuda_synchronize(prism_cuda_ctx *ctx) {
    if (!ctx) return PRISM_E_NULL;
    return check_device_error(ctx);
}

int prism_cuda_set_option(prism_cuda_ctx *ctx, const char *key, int64_t value) {
    if (!ctx || !key) return PRISM_E_NULL;
    if (!strcmp(key, "gemv_variant")) {
        if (value < 0 || value > 5) return fail(ctx, PRISM_E_ARG, "gemv_variant must be 0..5");
        ctx->gemv_variant = (int)value;
    } else if (!strcmp(key, "gemm_variant")) {
        if (value != 0 && value != 1) return fail(ctx, PRISM_E_ARG, "gemm_variant must be 0 or 1");
        ctx->gemm_variant = (int)value;
    } else if (!strcmp(key, "fuse")) {
        ctx->fuse = value ? 1 : 0;
    } else if (!strcmp(key, "sk_min_chunks")) {
        if (value < 1 || value > 4096) return fail(ctx, PRISM_E_ARG, "sk_min_chunks must be in 1..4096");
        ctx->sk_min_chunks = (int)value;
    } else if (!strcmp(key, "sk_stream_chunks")) {
        if (value < 8 || value > (1 << 20)) return fail(ctx, PRISM_E_ARG, "sk_stream_chunks must be in 8..2^20");
        ctx->sk_stream_chunks = (int)value;
    } else if (!strcmp(key, "cl_max_units")) {
        if (value < 0 || value > (1 << 24)) return fail(ctx, PRISM_E_ARG, "cl_max_units must be in 0..2^24");
        ctx->cl_max_units = (int)value;
    } else if (!strcmp(key, "batch_gemv_max")) {
        if (value < 1 || value > 4096) return fail(ctx, PRISM_E_ARG, "batch_gemv_max must be in 1..4096");
        ctx->batch_gemv_max = (int)value;
    } else if (!strcmp(key, "attn_cluster")) {
        if (value != 0 && value != 1 && value != 2 && value != 4 && value != 8)
            return fail(ctx, PRISM_E_ARG, "attn_cluster must be 0, 1, 2, 4 or 8");
        ctx->attn_cluster = (int)value;
    } else if (!strcmp(key, "ws_whole_blocks")) {
        if (value < 0 || value > 65536) return fail(ctx, PRISM_E_ARG, "ws_whole_blocks must be in 0..65536");
        ctx->ws_whole_blocks = (int)value;
    } else if (!strcmp(key, "ws_whole_fill")) {
        if (value < 1 || value > 100) return fail(ctx, PRISM_E_ARG, "ws_whole_fill must be in 1..100");
        ctx->ws_whole_fill = (int)value;
    } else if (!strcmp(key, "attn_group")) {
        if (value != 0 && value != 1 && value != 2 && value != 4 && value != 8)
            return fail(ctx, PRISM_E_ARG, "attn_group must be 0, 1, 2, 4 or 8");
        ctx->attn_group = (int)value;
    } else if (!strcmp(key, "tp_peer_ar")) {
        ctx->tp_peer_ar = value ? 1 : 0;
    } else if (!strcmp(key, "tp_fused_ar")) {
        if (value < 0 || value > 4) return fail(ctx, PRISM_E_ARG, "tp_fused_ar must be 0, 1, 2, 3 or 4");
        ctx->tp_fused_ar = (int)value;
    } else if (!strcmp(key, "pdl")) {
        ctx->pdl = value ? 1 : 0;
    } else if (!strcmp(key, "prefill_chunk")) {
        if (value < 0 || value > 65536) return fail(ctx, PRISM_E_ARG, "prefill_chunk must be in 0..65536");
        ctx->prefill_chunk = (int)value;
    } else if (!strcmp(key, "cimage_cache")) {
        ctx->cimage_cache = value ? 1 : 0;
    } else if (!strcmp(key, "wait_limit_polls")) {
        if (value < 0 || value > 0x7FFFFFFF) return fail(ctx, PRISM_E_ARG, "wait_limit_polls must be in 0..2^31-1");
        ctx->wait_limit_polls = (uint32_t)value;
    } else {
        return fail(ctx, PRISM_E_ARG, std::string("unknown option ") + key);
    }
    ctx->option_epoch++;
    return PRISM_OK;
}

uint64_t prism_cuda_launch_count(prism_cuda_ctx *ctx) { return ctx ? ctx->launches : 0; }

int prism_cuda_gemv_partition(uint32_t n_blocks, uint32_t n_chunks, uint32_t slots, uint32_t stream_chunks,
                              uint32_t min_chunks, uint32_t *n_ctas, uint32_t *bounds, uint32_t cap) {
    if (!n_ctas) return PRISM_E_NULL;
    if (n_blocks == 0 || n_chunks == 0 || slots == 0 || (uint64_t)n_blocks * n_chunks >= (1ull << 32)) return PRISM_E_ARG;
    const SkPart p = sk_choose_partition(n_blocks, n_chunks, slots, stream_chunks, min_chunks, 128);
    *n_ctas = p.G;
    if (bounds) {
        if (cap < p.G + 1) return PRISM_E_ARG;
        for (uint32_t i = 0; i <= p.G; i++) bounds[i] = sk_boundary(p, i);
    }
    return PRISM_OK;
}

uint32_t prism_cuda_gemv_partition_ctas(uint32_t n_blocks, uint32_t n_chunks, uint32_t slots, uint32_t whole_max_chunks,
                                        uint32_t fill_pct) {
    return ws_choose_slots(n_blocks, n_chunks, slots, whole_max_chunks, fill_pct);
}

int prism_cuda_upload_palettized_shard(prism_cuda_ctx *ctx, const char *name, const uint8_t *payload,
                                       size_t len, uint32_t dim_m, uint32_t dim_n, uint32_t bits,
                                       uint32_t row0, uint32_t rows, uint32_t col0, uint32_t cols,
                                       int32_t *handle) {
    if (!ctx || !payload || !handle) return fail(ctx, PRISM_E_NULL, "null argument");
    *handle = -1;
    if (bits != 2 && bits != 4) return fail(ctx, PRISM_E_ARG, "bits must be 2 or 4");
    if (((uint64_t)dim_n * bits) % 32 != 0) return fail(ctx, PRISM_E_ARG, "dim_n*bits must be a multiple of 32");
    const size_t need = (size_t)dim_m * ((size_t)2 << bits) + (size_t)dim_m * ((size_t)dim_n * bits / 8);
    if (len < need)
        return fail(ctx, PRISM_E_ARG, "truncated payload: " + std::to_string(len) + " < " + std::to_string(need));
    if (rows == 0 || cols == 0 || (uint64_t)row0 + rows > dim_m || (uint64_t)col0 + cols > dim_n)
        return fail(ctx, PRISM_E_ARG, "shard outside the tensor");
    const uint32_t per_chunk = 128 / bits;
    if ((col0 % per_chunk) || (cols != dim_n && cols % per_chunk))
        return fail(ctx, PRISM_E_ARG, "shard columns must be multiples of 128/bits");
    PRISM_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    PRISM_TRY(ensure_stage(ctx, need, 0));
    PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(ctx->stage_in, payload, need, cudaMemcpyHostToDevice, ctx->stream));
    int32_t h;
    PRISM_TRY(alloc_tensor(ctx, name, rows, cols, bits, &h));
    int rc = launch_relay(ctx, ctx->stage_in, dim_m, dim_n, row0, col0, ctx->tensors[h]);
    if (rc) return rc;
    PRISM_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));  // payload is caller-owned: done with it
    *handle = h;
    return PRISM_OK;
}

int prism_cuda_upload_palettized(prism_cuda_ctx *ctx, const char *name, const uint8_t *payload, size_t len,
                                 uint32_t dim_m, uint32_t dim_n, uint32_t bits, int32_t *handle) {
    return prism_cuda_upload_palettized_shard(ctx, name, payload, len, dim_m, dim_n, bits, 0, dim_m, 0,
                                              dim_n, handle);
}

int prism_cuda_synth_palettized(prism_cuda_ctx *ctx, const char *name, uint32_t dim_m, uint32_t dim_n,
                                uint32_t bits, uint64_t seed, float sigma, int32_t *handle) {
    return synth_shard(ctx, name, dim_m, dim_n, bits, seed, sigma, 0, 0, handle);
}

int prism_cuda_find_tensor(prism_cuda_ctx *ctx, const char *name, int32_t *handle) {
    if (!ctx || !name || !handle) return fail(ctx, PRISM_E_NULL, "null argument");
    auto it = ctx->by_name.find(name);
    if (it == ctx->by_name.end() || !ctx->tensors[it->second].live) {
        *handle = -1;
        return fail(ctx, PRISM_E_NOTFOUND, std::string("miss ") + name);
    }
    *handle = it->second;
    return PRISM_OK;
}

int prism_cuda_tensor_dims(prism_cuda_ctx *ctx, int32_t handle, uint32_t *dim_m, uint32_t *dim_n,
                           uint32_t *bits) {
    LutTensor *t = get_tensor(ctx, handle);
    if (!t) return ctx ? PRISM_E_NOTFOUND : PRISM_E_NULL;
    if (dim_m) *dim_m = t->m;
    if (dim_n) *dim_n = t->k;
    if (bits) *bits = t->bits;
    return PRISM_OK;
}

int prism_cuda_free_tensor(prism_cuda_ctx *ctx, int32_t handle) {
    LutTensor *t = get_tensor(ctx, handle);
    if (!t) return ctx ? PRISM_E_NOTFOUND : PRISM_E_NULL;
    PRISM_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    cudaFree(t->idx);
    cudaFree(t->pal);
    t->idx = nullptr; t->pal = nullptr; t->live = false;
    if (!t->name.empty()) ctx->by_name.erase(t->name);
    return PRISM_OK;
}

int prism_cuda_download_payload(prism_cuda_ctx *ctx, int32_t handle, uint8_t *payload, size_t len) {
    LutTensor *t = get_tensor(ctx, handle);
    if (!t) return ctx ? PRISM_E_NOTFOUND : PRISM_E_NULL;
    if (!payload) return fail(ctx, PRISM_E_NULL, "null payload");
    const size_t need = (size_t)t->m * t->n_ent() * 2 + (size_t)t->m * t->row_bytes;
    if (len != need) return fail(ctx, PRISM_E_ARG, "payload length must be " + std::to_string(need));
    PRISM_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    PRISM_TRY(ensure_stage(ctx, 0, need));
    PRISM_TRY(launch_unrelay(ctx, *t, ctx->stage_out));
    PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(payload, ctx->stage_out, need, cudaMemcpyDeviceToHost, ctx->stream));
    PRISM_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return PRISM_OK;
}

int prism_cuda_dequant_dev(prism_cuda_ctx *ctx, int32_t handle, void *out_dev) {
    LutTensor *t = get_tensor(ctx, handle);
    if (!t) return ctx ? PRISM_E_NOTFOUND : PRISM_E_NULL;
    if (!out_dev) return fail(ctx, PRISM_E_NULL, "null output");
    return launch_dequant(ctx, *t, (uint16_t *)out_dev);
}

int prism_cuda_dequant(prism_cuda_ctx *ctx, int32_t handle, uint16_t *out_host) {
    LutTensor *t = get_tensor(ctx, handle);
    if (!t) return ctx ? PRISM_E_NOTFOUND : PRISM_E_NULL;
    if (!out_host) return fail(ctx, PRISM_E_NULL, "null output");
    const size_t bytes = (size_t)t->m * t->k * 2;
    PRISM_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    PRISM_TRY(ensure_stage(ctx, 0, bytes));
    PRISM_TRY(launch_dequant(ctx, *t, (uint16_t *)ctx->stage_out));
    PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(out_host, ctx->stage_out, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    PRISM_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return PRISM_OK;
}

// ---- GEMV -------------------------------------------------------------------------------------

int prism_cuda_gemv_dev(prism_cuda_ctx *ctx, int32_t handle, const void *x_dev, void *y_dev) {
    LutTensor *t = get_tensor(ctx, handle);
    if (!t) return ctx ? PRISM_E_NOTFOUND : PRISM_E_NULL;
    if (!x_dev || !y_dev) return fail(ctx, PRISM_E_NULL, "null vector");
    return launch_gemv(ctx, GEMV_PLAIN, *t, nullptr, (const uint16_t *)x_dev, round_up_u32(t->k, 8),
                       (uint16_t *)y_dev, t->m, nullptr, 1);
}

int prism_cuda_gemv_residual_dev(prism_cuda_ctx *ctx, int32_t handle, const void *x_dev,
                                 const void *resid_dev, void *y_dev) {
    LutTensor *t = get_tensor(ctx, handle);
    if (!t) return ctx ? PRISM_E_NOTFOUND : PRISM_E_NULL;
    if (!x_dev || !y_dev || !resid_dev) return fail(ctx, PRISM_E_NULL, "null vector");
    return launch_gemv(ctx, GEMV_RESID, *t, nullptr, (const uint16_t *)x_dev, round_up_u32(t->k, 8),
                       (uint16_t *)y_dev, t->m, (const uint16_t *)resid_dev, 1);
}

// host in -> stage_in, kernel, stage_out -> host out
static int host_call_begin(prism_cuda_ctx *ctx, const void *in, size_t in_bytes, size_t out_bytes) {
    PRISM_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    PRISM_TRY(ensure_stage(ctx, in_bytes, out_bytes));
    if (in_bytes)
        PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(ctx->stage_in, in, in_bytes, cudaMemcpyHostToDevice, ctx->stream));
    return PRISM_OK;
}
static int host_call_end(prism_cuda_ctx *ctx, void *out, size_t out_bytes) {
    if (out_bytes)
        PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(out, ctx->stage_out, out_bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return check_device_error(ctx);
}

int prism_cuda_gemv(prism_cuda_ctx *ctx, int32_t handle, const uint16_t *x, uint16_t *y) {
    LutTensor *t = get_tensor(ctx, handle);
    if (!t) return ctx ? PRISM_E_NOTFOUND : PRISM_E_NULL;
    if (!x || !y) return fail(ctx, PRISM_E_NULL, "null vector");
    PRISM_TRY(host_call_begin(ctx, x, (size_t)t->k * 2, (size_t)t->m * 2));
    PRISM_TRY(prism_cuda_gemv_dev(ctx, handle, ctx->stage_in, ctx->stage_out));
    return host_call_end(ctx, y, (size_t)t->m * 2);
}

int prism_cuda_gemv_key(prism_cuda_ctx *ctx, const char *key, const uint16_t *x, size_t x_len, uint16_t *y,
                        size_t y_len) {
    int32_t h;
    PRISM_TRY(prism_cuda_find_tensor(ctx, key, &h));
    const LutTensor &t = ctx->tensors[h];
    if (x_len != t.k || y_len != t.m)
        return fail(ctx, PRISM_E_ARG, std::string("gemv ") + key + ": slice lengths do not match the tensor");
    return prism_cuda_gemv(ctx, h, x, y);
}

// ---- fused gate/up and MLP -----------------------------------------------------------------------

int prism_cuda_fused_gate_up_dev(prism_cuda_ctx *ctx, int32_t gate, int32_t up, const void *x_dev,
                                 void *out_dev) {
    LutTensor *g = get_tensor(ctx, gate);
    LutTensor *u = get_tensor(ctx, up);
    if (!g || !u) return ctx ? PRISM_E_NOTFOUND : PRISM_E_NULL;
    if (!x_dev || !out_dev) return fail(ctx, PRISM_E_NULL, "null vector");
    return launch_gemv(ctx, GEMV_SWIGLU, *g, u, (const uint16_t *)x_dev, round_up_u32(g->k, 8),
                       (uint16_t *)out_dev, g->m, nullptr, 1);
}

int prism_cuda_fused_gate_up(prism_cuda_ctx *ctx, int32_t gate, int32_t up, const uint16_t *x, uint16_t *out) {
    LutTensor *g = get_tensor(ctx, gate);
    if (!g) return ctx ? PRISM_E_NOTFOUND : PRISM_E_NULL;
    if (!x || !out) return fail(ctx, PRISM_E_NULL, "null vector");
    PRISM_TRY(host_call_begin(ctx, x, (size_t)g->k * 2, (size_t)g->m * 2));
    PRISM_TRY(prism_cuda_fused_gate_up_dev(ctx, gate, up, ctx->stage_in, ctx->stage_out));
    return host_call_end(ctx, out, (size_t)g->m * 2);
}

int prism_cuda_fused_gate_up_key(prism_cuda_ctx *ctx, const char *gate_key, const char *up_key,
                                 const uint16_t *x, size_t x_len, uint16_t *out, size_t out_len) {
    int32_t hg, hu;
    PRISM_TRY(prism_cuda_find_tensor(ctx, gate_key, &hg));
    PRISM_TRY(prism_cuda_find_tensor(ctx, up_key, &hu));
    const LutTensor &t = ctx->tensors[hg];
    if (x_len != t.k || out_len != t.m) return fail(ctx, PRISM_E_ARG, "fused_gate_up: slice lengths do not match");
    return prism_cuda_fused_gate_up(ctx, hg, hu, x, out);
}

int prism_cuda_mlp_dev(prism_cuda_ctx *ctx, int32_t gate, int32_t up, int32_t down, const void *x_dev,
                       void *out_dev) {
    LutTensor *g = get_tensor(ctx, gate);
    LutTensor *u = get_tensor(ctx, up);
    LutTensor *d = get_tensor(ctx, down);
    if (!g || !u || !d) return ctx ? PRISM_E_NOTFOUND : PRISM_E_NULL;
    if (!x_dev || !out_dev) return fail(ctx, PRISM_E_NULL, "null vector");
    if (d->k != g->m) return fail(ctx, PRISM_E_ARG, "mlp: down.dim_n must equal gate.dim_m");
    PRISM_TRY(ensure_act(ctx, round_up_u32(g->m_pad, 8)));
    PRISM_TRY(launch_gemv(ctx, GEMV_SWIGLU, *g, u, (const uint16_t *)x_dev, round_up_u32(g->k, 8),
                          ctx->act_scratch, g->m_pad, nullptr, 1));
    return launch_gemv(ctx, GEMV_PLAIN, *d, nullptr, ctx->act_scratch, g->m_pad, (uint16_t *)out_dev, d->m,
                       nullptr, 1);
}

int prism_cuda_mlp(prism_cuda_ctx *ctx, int32_t gate, int32_t up, int32_t down, const uint16_t *x,
                   uint16_t *out) {
    LutTensor *g = get_tensor(ctx, gate);
    LutTensor *d = get_tensor(ctx, down);
    if (!g || !d) return ctx ? PRISM_E_NOTFOUND : PRISM_E_NULL;
    if (!x || !out) return fail(ctx, PRISM_E_NULL, "null vector");
    PRISM_TRY(host_call_begin(ctx, x, (size_t)g->k * 2, (size_t)d->m * 2));
    PRISM_TRY(prism_cuda_mlp_dev(ctx, gate, up, down, ctx->stage_in, ctx->stage_out));
    return host_call_end(ctx, out, (size_t)d->m * 2);
}

// ---- prefill GEMM -----------------------------------------------------------------------------------

int prism_cuda_gemm_dev(prism_cuda_ctx *ctx, int32_t handle, const void *X_dev, uint32_t m_tok, void *Y_dev) {
    LutTensor *t = get_tensor(ctx, handle);
    if (!t) return ctx ? PRISM_E_NOTFOUND : PRISM_E_NULL;
    if (!X_dev || !Y_dev) return fail(ctx, PRISM_E_NULL, "null matrix");
    if (m_tok == 0) return PRISM_OK;
    return launch_gemm(ctx, *t, (const uint16_t *)X_dev, m_tok, (uint16_t *)Y_dev);
}

int prism_cuda_gemm(prism_cuda_ctx *ctx, int32_t handle, const uint16_t *X, uint32_t m_tok, uint16_t *Y) {
    LutTensor *t = get_tensor(ctx, handle);
    if (!t) return ctx ? PRISM_E_NOTFOUND : PRISM_E_NULL;
    if (!X || !Y) return fail(ctx, PRISM_E_NULL, "null matrix");
    if (m_tok == 0) return PRISM_OK;
    PRISM_TRY(host_call_begin(ctx, X, (size_t)m_tok * t->k * 2, (size_t)m_tok * t->m * 2));
    PRISM_TRY(prism_cuda_gemm_dev(ctx, handle, ctx->stage_in, m_tok, ctx->stage_out));
    return host_call_end(ctx, Y, (size_t)m_tok * t->m * 2);
}

// ---- measurement helper ---------------------------------------------------------------------------------
// Cycles through `n_sets` distinct weight sets so the working set exceeds L2, inside one CUDA
// graph replayed `reps` times between two events.  kind 0: gemv (1 handle per set); 1: fused
// gate/up (2 handles: gate, up); 2: whole MLP (3 handles: gate, up, down).
int prism_cuda_bench_cycle(prism_cuda_ctx *ctx, int kind, const int32_t *handles, uint32_t n_sets, uint32_t reps,
                           const void *x_dev, double *ms_out) {
    if (!ctx || !handles || !ms_out || !x_dev) return fail(ctx, PRISM_E_NULL, "null argument");
    if (reinterpret_cast<uintptr_t>(x_dev) & 15) return fail(ctx, PRISM_E_ARG, "activations must be 16-byte aligned");
    if (kind < 0 || kind > 2 || n_sets == 0 || reps == 0) return fail(ctx, PRISM_E_ARG, "bad bench arguments");
    const int per = kind + 1;
    for (uint32_t i = 0; i < n_sets * per; i++)
        if (!get_tensor(ctx, handles[i])) return PRISM_E_NOTFOUND;
    PRISM_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    const LutTensor &t0 = ctx->tensors[handles[0]];
    const size_t mid_b = (size_t)t0.m_pad * 2;
    PRISM_TRY(ensure_stage(ctx, 0, mid_b + 4096));
    auto pass = [&]() -> int {
        for (uint32_t s = 0; s < n_sets; s++) {
            const int32_t *h = handles + (size_t)s * per;
            if (kind == 0) PRISM_TRY(prism_cuda_gemv_dev(ctx, h[0], x_dev, ctx->stage_out));
            else if (kind == 1) PRISM_TRY(prism_cuda_fused_gate_up_dev(ctx, h[0], h[1], x_dev, ctx->stage_out));
            else PRISM_TRY(prism_cuda_mlp_dev(ctx, h[0], h[1], h[2], x_dev, ctx->stage_out));
        }
        return PRISM_OK;
    };
    PRISM_TRY(pass());  // eager warm-up: scratch sizes, kernel attributes
    PRISM_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    cudaGraph_t g = nullptr;
    cudaGraphExec_t ge = nullptr;
    PRISM_CUDA_TRY(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    const uint64_t l0 = ctx->launches;
    int rc = pass();
    const uint64_t per_pass = ctx->launches - l0;
    cudaError_t ce = cudaStreamEndCapture(ctx->stream, &g);
    if (rc != PRISM_OK) { if (g) cudaGraphDestroy(g); return rc; }
    if (ce != cudaSuccess) return cuda_fail(ctx, ce, "cudaStreamEndCapture");
    ce = cudaGraphInstantiate(&ge, g, 0);
    cudaGraphDestroy(g);
    if (ce != cudaSuccess) return cuda_fail(ctx, ce, "cudaGraphInstantiate");
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    for (int w = 0; w < 3; w++) cudaGraphLaunch(ge, ctx->stream);
    cudaEventRecord(e0, ctx->stream);
    for (uint32_t r = 0; r < reps; r++) cudaGraphLaunch(ge, ctx->stream);
    cudaEventRecord(e1, ctx->stream);
    ce = cudaStreamSynchronize(ctx->stream);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaGraphExecDestroy(ge);
    ctx->launches = l0 + per_pass * (reps + 3);
    if (ce != cudaSuccess) return cuda_fail(ctx, ce, "bench cycle");
    *ms_out = ms;
    return PRISM_OK;
}

// Measurement: `reps` prefill GEMMs of the caller's m_tok activation rows against one tensor, between
// two events on the context stream.
int prism_cuda_bench_gemm(prism_cuda_ctx *ctx, int32_t handle, const void *X_dev, uint32_t m_tok, uint32_t reps,
                          double *ms_out) {
    LutTensor *t = get_tensor(ctx, handle);
    if (!t) return ctx ? PRISM_E_NOTFOUND : PRISM_E_NULL;
    if (!ms_out || !X_dev || m_tok == 0 || reps == 0) return fail(ctx, PRISM_E_ARG, "bad bench arguments");
    if (reinterpret_cast<uintptr_t>(X_dev) & 15) return fail(ctx, PRISM_E_ARG, "activations must be 16-byte aligned");
    PRISM_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    const size_t out_b = (size_t)m_tok * t->m * 2;
    PRISM_TRY(ensure_stage(ctx, 0, out_b));
    PRISM_TRY(launch_gemm(ctx, *t, (const uint16_t *)X_dev, m_tok, (uint16_t *)ctx->stage_out));  // warm-up
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    cudaEventRecord(e0, ctx->stream);
    int rc = PRISM_OK;
    for (uint32_t r = 0; r < reps && rc == PRISM_OK; r++)
        rc = launch_gemm(ctx, *t, (const uint16_t *)X_dev, m_tok, (uint16_t *)ctx->stage_out);
    cudaEventRecord(e1, ctx->stream);
    cudaError_t ce = cudaStreamSynchronize(ctx->stream);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (rc != PRISM_OK) return rc;
    if (ce != cudaSuccess) return cuda_fail(ctx, ce, "bench gemm");
    *ms_out = ms;
    return check_device_error(ctx);
}

// ---- glue ops on host slices (MetalBackend::{norm_metal,...}) ---------------------------------------

int prism_cuda_rms_norm(prism_cuda_ctx *ctx, const uint16_t *in, uint16_t *out, uint32_t n, float eps) {
    if (!ctx || !in || !out) return fail(ctx, PRISM_E_NULL, "null argument");
    if (n == 0) return PRISM_OK;
    PRISM_TRY(host_call_begin(ctx, in, (size_t)n * 2, (size_t)n * 2));
    PRISM_TRY(launch_rms_norm(ctx, (const uint16_t *)ctx->stage_in, (uint16_t *)ctx->stage_out, n, eps, 1));
    return host_call_end(ctx, out, (size_t)n * 2);
}

int prism_cuda_rope(prism_cuda_ctx *ctx, uint16_t *x, uint32_t n, int64_t pos, uint32_t head_dim, float base) {
    if (!ctx || !x) return fail(ctx, PRISM_E_NULL, "null argument");
    if (head_dim == 0 || (head_dim & 1)) return fail(ctx, PRISM_E_ARG, "rope: head_dim must be even");
    if (n == 0) return PRISM_OK;
    PRISM_TRY(host_call_begin(ctx, x, (size_t)n * 2, 0));
    PRISM_TRY(launch_rope(ctx, (uint16_t *)ctx->stage_in, n, nullptr, pos, head_dim, base, 1, n));
    PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(x, ctx->stage_in, (size_t)n * 2, cudaMemcpyDeviceToHost, ctx->stream));
    PRISM_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return PRISM_OK;
}

int prism_cuda_softmax(prism_cuda_ctx *ctx, const uint16_t *in, uint16_t *out, uint32_t n) {
    if (!ctx || !in || !out) return fail(ctx, PRISM_E_NULL, "null argument");
    if (n == 0) return PRISM_OK;
    PRISM_TRY(host_call_begin(ctx, in, (size_t)n * 2, (size_t)n * 2));
    PRISM_TRY(launch_softmax(ctx, (const uint16_t *)ctx->stage_in, (uint16_t *)ctx->stage_out, n));
    return host_call_end(ctx, out, (size_t)n * 2);
}

int prism_cuda_silu(prism_cuda_ctx *ctx, uint16_t *x, uint32_t n) {
    if (!ctx || !x) return fail(ctx, PRISM_E_NULL, "null argument");
    if (n == 0) return PRISM_OK;
    PRISM_TRY(host_call_begin(ctx, x, (size_t)n * 2, 0));
    PRISM_TRY(launch_silu(ctx, (uint16_t *)ctx->stage_in, n));
    PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(x, ctx->stage_in, (size_t)n * 2, cudaMemcpyDeviceToHost, ctx->stream));
    PRISM_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return PRISM_OK;
}

int prism_cuda_vec_add(prism_cuda_ctx *ctx, uint16_t *a, const uint16_t *b, uint32_t n) {
    if (!ctx || !a || !b) return fail(ctx, PRISM_E_NULL, "null argument");
    if (n == 0) return PRISM_OK;
    const size_t bytes = (size_t)n * 2, off = (bytes + 255) / 256 * 256;
    PRISM_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    PRISM_TRY(ensure_stage(ctx, off + bytes, 0));
    PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(ctx->stage_in, a, bytes, cudaMemcpyHostToDevice, ctx->stream));
    PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(ctx->stage_in + off, b, bytes, cudaMemcpyHostToDevice, ctx->stream));
    PRISM_TRY(launch_vec_add(ctx, (uint16_t *)ctx->stage_in, (const uint16_t *)(ctx->stage_in + off), n));
    PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(a, ctx->stage_in, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    PRISM_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return PRISM_OK;
}

int prism_cuda_attention(prism_cuda_ctx *ctx, const uint16_t *q, const uint16_t *k, const uint16_t *v,
                         uint32_t seq_len, uint32_t num_heads, uint32_t kv_heads, uint32_t head_dim,
                         uint16_t *out) {
    if (!ctx || !q || !k || !v || !out) return fail(ctx, PRISM_E_NULL, "null argument");
    if (!num_heads || !kv_heads || !head_dim || num_heads % kv_heads)
        return fail(ctx, PRISM_E_ARG, "attention: bad head configuration");
    const size_t qb = (size_t)num_heads * head_dim * 2, kvb = (size_t)seq_len * kv_heads * head_dim * 2;
    auto al = [](size_t x) { return (x + 255) / 256 * 256; };
    PRISM_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    PRISM_TRY(ensure_stage(ctx, al(qb) + 2 * al(kvb) + 256, qb));
    uint8_t *dq = ctx->stage_in, *dk = dq + al(qb), *dv = dk + al(kvb);
    PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(dq, q, qb, cudaMemcpyHostToDevice, ctx->stream));
    if (kvb) {
        PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(dk, k, kvb, cudaMemcpyHostToDevice, ctx->stream));
        PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(dv, v, kvb, cudaMemcpyHostToDevice, ctx->stream));
    }
    AttnArgs a{};
    a.q = (const uint16_t *)dq; a.q_stride = num_heads * head_dim; a.k = dk; a.v = dv; a.out = (uint16_t *)ctx->stage_out;
    if (seq_len == 0) return fail(ctx, PRISM_E_ARG, "attention: seq_len must be > 0");
    a.pos_dev = nullptr; a.pos_host = (int32_t)seq_len - 1; a.slot_mul = 1; a.slot_add = 0;
    a.nh = num_heads; a.nkv = kv_heads; a.hd = head_dim; a.batch = 1;
    a.seq_stride = 0; a.int8 = 0; a.max_seq = seq_len ? seq_len : 1;
    PRISM_TRY(launch_attention(ctx, a));
    return host_call_end(ctx, out, qb);
}

// ---- backend-held KV cache: the kv_bufs of MetalBackend (engine_impl.rs:47-49, 109-119, 256-286) --------

int prism_cuda_kv_init(prism_cuda_ctx *ctx, uint32_t num_layers, uint32_t kv_dim, uint32_t max_seq) {
    if (!ctx) return PRISM_E_NULL;
    if (!num_layers || !kv_dim || !max_seq || kv_dim % 8) return fail(ctx, PRISM_E_ARG, "kv_init: zero dimension, or kv_dim not a multiple of 8");
    PRISM_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    PRISM_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    cudaFree(ctx->kv_k);
    cudaFree(ctx->kv_v);
    ctx->kv_k = ctx->kv_v = nullptr;
    ctx->kv_layers = ctx->kv_dim = ctx->kv_max_seq = 0;
    const size_t bytes = (size_t)num_layers * max_seq * kv_dim * 2;
    PRISM_CUDA_TRY(ctx, cudaMalloc((void **)&ctx->kv_k, bytes));
    cudaError_t e = cudaMalloc((void **)&ctx->kv_v, bytes);
    if (e != cudaSuccess) {
        cudaFree(ctx->kv_k);
        ctx->kv_k = nullptr;
        return cuda_fail(ctx, e, "cudaMalloc(kv cache)");
    }
    ctx->kv_layers = num_layers; ctx->kv_dim = kv_dim; ctx->kv_max_seq = max_seq;
    return PRISM_OK;
}

int prism_cuda_kv_append(prism_cuda_ctx *ctx, uint32_t layer, const uint16_t *k, const uint16_t *v, uint64_t token_idx) {
    if (!ctx || !k || !v) return fail(ctx, PRISM_E_NULL, "null argument");
    if (!ctx->kv_k) return fail(ctx, PRISM_E_STATE, "kv_append: no cache (prism_cuda_kv_init first)");
    if (layer >= ctx->kv_layers || token_idx >= ctx->kv_max_seq)
        return fail(ctx, PRISM_E_ARG, "kv_append: layer or token index outside the cache");
    PRISM_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    const size_t off = ((size_t)layer * ctx->kv_max_seq + token_idx) * ctx->kv_dim, bytes = (size_t)ctx->kv_dim * 2;
    PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(ctx->kv_k + off, k, bytes, cudaMemcpyHostToDevice, ctx->stream));
    PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(ctx->kv_v + off, v, bytes, cudaMemcpyHostToDevice, ctx->stream));
    PRISM_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return PRISM_OK;
}

int prism_cuda_attention_kv(prism_cuda_ctx *ctx, uint32_t layer, const uint16_t *q, uint32_t seq_len, uint32_t num_heads,
                            uint32_t kv_heads, uint32_t head_dim, uint16_t *out) {
    if (!ctx || !q || !out) return fail(ctx, PRISM_E_NULL, "null argument");
    if (!ctx->kv_k) return fail(ctx, PRISM_E_STATE, "attention_kv: no cache (prism_cuda_kv_init first)");
    if (!num_heads || !kv_heads || !head_dim || num_heads % kv_heads) return fail(ctx, PRISM_E_ARG, "attention: bad head configuration");
    if (layer >= ctx->kv_layers || kv_heads * head_dim != ctx->kv_dim || seq_len == 0 || seq_len > ctx->kv_max_seq)
        return fail(ctx, PRISM_E_ARG, "attention_kv: layer, kv width or seq_len does not match the cache");
    const size_t qb = (size_t)num_heads * head_dim * 2;
    PRISM_TRY(host_call_begin(ctx, q, qb, qb));
    AttnArgs a{};
    const size_t off = (size_t)layer * ctx->kv_max_seq * ctx->kv_dim;
    a.q = (const uint16_t *)ctx->stage_in; a.q_stride = num_heads * head_dim;
    a.k = ctx->kv_k + off; a.v = ctx->kv_v + off; a.out = (uint16_t *)ctx->stage_out;
    a.pos_dev = nullptr; a.pos_host = (int32_t)seq_len - 1; a.slot_mul = 1; a.slot_add = 0;
    a.nh = num_heads; a.nkv = kv_heads; a.hd = head_dim; a.batch = 1;
    a.seq_stride = 0; a.int8 = 0; a.max_seq = seq_len;
    PRISM_TRY(launch_attention(ctx, a));
    return host_call_end(ctx, out, qb);
}

int prism_cuda_attention_step_kv(prism_cuda_ctx *ctx, uint32_t layer, const uint16_t *q, const uint16_t *k, const uint16_t *v,
                                 uint64_t token_idx, uint32_t num_heads, uint32_t kv_heads, uint32_t head_dim, uint32_t rope_k,
                                 float rope_base, uint16_t *out) {
    if (!ctx || !q || !k || !v || !out) return fail(ctx, PRISM_E_NULL, "null argument");
    if (!ctx->kv_k) return fail(ctx, PRISM_E_STATE, "attention_step_kv: no cache (prism_cuda_kv_init first)");
    if (!num_heads || !kv_heads || !head_dim || num_heads % kv_heads) return fail(ctx, PRISM_E_ARG, "attention: bad head configuration");
    if (layer >= ctx->kv_layers || kv_heads * head_dim != ctx->kv_dim || token_idx >= ctx->kv_max_seq)
        return fail(ctx, PRISM_E_ARG, "attention_step_kv: layer, kv width or token index does not match the cache");
    const uint32_t qd = num_heads * head_dim, kvd = ctx->kv_dim, stride = round_up_u32(qd + 2 * kvd, 8);
    PRISM_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    PRISM_TRY(ensure_stage(ctx, (size_t)stride * 2, (size_t)qd * 2));
    uint16_t *row = reinterpret_cast<uint16_t *>(ctx->stage_in);
    int32_t *pos_dev = reinterpret_cast<int32_t *>(ctx->dev_err + 4);
    const int32_t pos = (int32_t)token_idx;
    PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(row, q, (size_t)qd * 2, cudaMemcpyHostToDevice, ctx->stream));
    PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(row + qd, k, (size_t)kvd * 2, cudaMemcpyHostToDevice, ctx->stream));
    PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(row + qd + kvd, v, (size_t)kvd * 2, cudaMemcpyHostToDevice, ctx->stream));
    PRISM_CUDA_TRY(ctx, cudaMemcpyAsync(pos_dev, &pos, 4, cudaMemcpyHostToDevice, ctx->stream));
    AttnArgs a{};
    const size_t off = (size_t)layer * ctx->kv_max_seq * kvd;
    a.q = row; a.q_stride = stride; a.k = ctx->kv_k + off; a.v = ctx->kv_v + off; a.out = (uint16_t *)ctx->stage_out;
    a.pos_dev = pos_dev; a.pos_host = pos; a.slot_mul = 1; a.slot_add = 0;
    a.nh = num_heads; a.nkv = kv_heads; a.hd = head_dim; a.batch = 1;
    a.seq_stride = 0; a.int8 = 0; a.max_seq = ctx->kv_max_seq;
    if (!attn_fused_eligible(a)) return fail(ctx, PRISM_E_ARG, "attention_step_kv: head_dim must be 32, 64, 128 or 256");
    PRISM_TRY(launch_attn_fused(ctx, a, row + qd, row + qd + kvd, rope_k, rope_base));
    return host_call_end(ctx, out, (size_t)qd * 2);
}

int prism_cuda_argmax(prism_cuda_ctx *ctx, const uint16_t *logits, uint32_t n, uint32_t *index) {
    if (!ctx || !logits || !index) return fail(ctx, PRISM_E_NULL, "null argument");
    if (n == 0) { *index = 0; return PRISM_OK; }
    PRISM_TRY(host_call_begin(ctx, logits, (size_t)n * 2, 4));
    PRISM_TRY(launch_argmax(ctx, (const uint16_t *)ctx->stage_in, n, n, 1, (uint32_t *)ctx->stage_out));
    return host_call_end(ctx, index, 4);
}

}  // extern "C"
