// Offline quantiser on the GPU: one thread fits and encodes one output row, with exactly the
// operations, in exactly the order, of the reference's CPU quantiser, so the payload is
// bit-identical to it.
//
//   fit_palette      src/quantization/palette.rs:75-174   deterministic k-means++ seeding (first
//                    centroid = channel[n/2], golden-ratio threshold :177-182), <= max_iter Lloyd
//                    steps, early exit when the largest shift < 0.001, codebook sorted by |value|
//                    descending (stable)
//   encode_channel   src/quantization/palette.rs:189-217  nearest of the 16 entries, first wins on
//                    ties, element 2i in the low nibble
//   payload          src/lut/compiler.rs:50-61            all palettes as fp16, then all index rows
//
// Every sum that the CPU code carries from element to element (the seeding's total and running sum,
// the per-cluster sums of a Lloyd step) is carried the same way here, by the one thread that owns
// the row; rows are independent, so the parallelism is over rows.  Arithmetic uses the explicit
// round-to-nearest intrinsics: no multiply-add contraction (Rust never contracts a*b+c).  The two
// scratch arrays of the CPU code are not needed: the seeding's running minimum distance is the
// minimum over the centroids chosen so far and is recomputed, and a Lloyd step assigns and
// accumulates in one pass.
#include "common.cuh"

namespace prism {

constexpr int PQ_THREADS = 128;

__device__ __forceinline__ float pq_dist(float x, float c) {
    const float diff = __fsub_rn(x, c);
    return __fmul_rn(diff, diff);
}

// weighted_threshold (palette.rs:177-182)
__device__ __forceinline__ float pq_threshold(float total, uint32_t seed) {
    const double v = __dmul_rn((double)seed, 0.6180339887498949);
    const double frac = __dsub_rn(v, floor(v));
    return __fmul_rn(total, (float)frac);
}

__global__ void __launch_bounds__(PQ_THREADS) palettize_rows_kernel(const float *__restrict__ w, uint32_t dm,
                                                                    uint32_t dn, uint32_t k_req, uint32_t max_iter,
                                                                    uint8_t *__restrict__ payload) {
    const uint32_t r = blockIdx.x * PQ_THREADS + threadIdx.x;
    if (r >= dm) return;
    const float *ch = w + (size_t)r * dn;
    const uint32_t n = dn;
    float cb[16];
#pragma unroll
    for (int i = 0; i < 16; i++) cb[i] = 0.0f;
    uint32_t k = k_req > 16 ? 16 : k_req;
    if (k > n) k = n;

    // ---- seeding ----------------------------------------------------------------------------------
    uint32_t nc = 0;
    if (k > 0) cb[nc++] = ch[n / 2];
    for (uint32_t it = 1; it < k; it++) {
        // min_d[i] after this round = the smallest squared distance to centroids 0..nc-1
        float total = 0.0f;
        for (uint32_t i = 0; i < n; i++) {
            const float x = ch[i];
            float md = 3.40282347e+38f;
            for (uint32_t c = 0; c < nc; c++) {
                const float d = pq_dist(x, cb[c]);
                if (d < md) md = d;
            }
            total = __fadd_rn(total, md);
        }
        if (total <= 0.0f) {
            cb[nc] = ch[((size_t)nc * n / k) % n];
            nc++;
            continue;
        }
        const float target = pq_threshold(total, nc);
        float cum = 0.0f;
        uint32_t picked = 0;
        for (uint32_t i = 0; i < n; i++) {
            const float x = ch[i];
            float md = 3.40282347e+38f;
            for (uint32_t c = 0; c < nc; c++) {
                const float d = pq_dist(x, cb[c]);
                if (d < md) md = d;
            }
            cum = __fadd_rn(cum, md);
            if (cum >= target) {
                picked = i;
                break;
            }
        }
        cb[nc++] = ch[picked];
    }

    // ---- Lloyd steps --------------------------------------------------------------------------------
    for (uint32_t iter = 0; iter < max_iter && k > 0; iter++) {
        float sum[16];
        uint32_t cnt[16];
#pragma unroll
        for (int c = 0; c < 16; c++) {
            sum[c] = 0.0f;
            cnt[c] = 0;
        }
        for (uint32_t i = 0; i < n; i++) {
            const float x = ch[i];
            float best_d = 3.40282347e+38f;
            uint32_t best = 0;
            for (uint32_t c = 0; c < k; c++) {
                const float d = pq_dist(x, cb[c]);
                if (d < best_d) {
                    best_d = d;
                    best = c;
                }
            }
            sum[best] = __fadd_rn(sum[best], x);
            cnt[best]++;
        }
        float max_shift = 0.0f;
        for (uint32_t c = 0; c < k; c++) {
            if (cnt[c] > 0) {
                const float nv = __fdiv_rn(sum[c], (float)cnt[c]);
                const float shift = fabsf(__fsub_rn(cb[c], nv));
                if (shift > max_shift) max_shift = shift;
                cb[c] = nv;
            }
        }
        if (max_shift < 0.001f) break;
    }

    // ---- stable sort of the k centroids, |v| descending --------------------------------------------
    for (uint32_t i = 1; i < k; i++) {
        const float v = cb[i];
        uint32_t j = i;
        while (j > 0 && fabsf(cb[j - 1]) < fabsf(v)) {
            cb[j] = cb[j - 1];
            j--;
        }
        cb[j] = v;
    }

    // ---- encode against all 16 entries (unused ones are 0) and emit ---------------------------------
    uint8_t *pal = payload + (size_t)r * 32;
    uint8_t *idx = payload + (size_t)dm * 32 + (size_t)r * (dn / 2);
    uint8_t cur = 0;
    for (uint32_t i = 0; i < n; i++) {
        const float x = ch[i];
        uint32_t best = 0;
        float best_d = 3.40282347e+38f;
#pragma unroll
        for (uint32_t c = 0; c < 16; c++) {
            const float d = pq_dist(x, cb[c]);
            if (d < best_d) {
                best_d = d;
                best = c;
            }
        }
        if ((i & 1) == 0) {
            cur = (uint8_t)best;
            if (i + 1 == n) idx[i / 2] = cur;
        } else {
            idx[i / 2] = (uint8_t)(cur | (best << 4));
        }
    }
    // little-endian fp16 bit patterns; the palette of a row starts on a 32-byte boundary
    uint16_t *pal16 = reinterpret_cast<uint16_t *>(pal);
    for (int i = 0; i < 16; i++) pal16[i] = __half_as_ushort(__float2half_rn(cb[i]));
}

int launch_palettize(prism_cuda_ctx *ctx, const float *w_dev, uint32_t dm, uint32_t dn, uint32_t k, uint32_t max_iter,
                     uint8_t *payload_dev) {
    palettize_rows_kernel<<<(dm + PQ_THREADS - 1) / PQ_THREADS, PQ_THREADS, 0, ctx->stream>>>(w_dev, dm, dn, k, max_iter,
                                                                                               payload_dev);
    return after_launch(ctx, "palettize_rows_kernel");
}

}  // namespace prism

using namespace prism;

extern "C" int prism_cuda_palettize_dev(prism_cuda_ctx *ctx, const float *weights_dev, uint32_t dim_m, uint32_t dim_n,
                                        uint32_t k, uint32_t max_iter, uint8_t *payload_dev) {
    if (!ctx || !weights_dev || !payload_dev) return fail(ctx, PRISM_E_NULL, "null argument");
    if (dim_m == 0 || dim_n == 0 || dim_n % 2 != 0 || k == 0)
        return fail(ctx, PRISM_E_ARG, "palettize: dim_m, dim_n > 0, dim_n even, k >= 1");
    return launch_palettize(ctx, weights_dev, dim_m, dim_n, k, max_iter, payload_dev);
}

extern "C" int prism_cuda_palettize(prism_cuda_ctx *ctx, const float *weights, uint32_t dim_m, uint32_t dim_n, uint32_t k,
                                    uint32_t max_iter, uint8_t *payload, size_t len) {
    if (!ctx || !weights || !payload) return fail(ctx, PRISM_E_NULL, "null argument");
    if (dim_m == 0 || dim_n == 0 || dim_n % 2 != 0 || k == 0)
        return fail(ctx, PRISM_E_ARG, "palettize: dim_m, dim_n > 0, dim_n even, k >= 1");
    const size_t need = (size_t)dim_m * 32 + (size_t)dim_m * (dim_n / 2);
    if (len != need) return fail(ctx, PRISM_E_ARG, "palettize: payload must hold dim_m*32 + dim_m*dim_n/2 bytes");
    PRISM_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    float *w_dev = nullptr;
    uint8_t *p_dev = nullptr;
    const size_t w_bytes = (size_t)dim_m * dim_n * sizeof(float);
    PRISM_CUDA_TRY(ctx, cudaMalloc((void **)&w_dev, w_bytes));
    cudaError_t e = cudaMalloc((void **)&p_dev, need);
    if (e != cudaSuccess) {
        cudaFree(w_dev);
        return cuda_fail(ctx, e, "cudaMalloc(payload)");
    }
    int rc = PRISM_OK;
    e = cudaMemcpyAsync(w_dev, weights, w_bytes, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) rc = launch_palettize(ctx, w_dev, dim_m, dim_n, k, max_iter, p_dev);
    if (e == cudaSuccess && rc == PRISM_OK) e = cudaMemcpyAsync(payload, p_dev, need, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess && rc == PRISM_OK) e = cudaStreamSynchronize(ctx->stream);
    cudaFree(w_dev);
    cudaFree(p_dev);
    if (rc != PRISM_OK) return rc;
    if (e != cudaSuccess) return cuda_fail(ctx, e, "palettize");
    return PRISM_OK;
}
