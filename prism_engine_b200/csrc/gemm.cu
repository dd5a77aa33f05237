// Prefill palettized GEMM: Y[t][:] = lut_gemv(X[t][:]) for every activation row
// (prefill_cpu, src/lut/engine_impl.rs:1046-1053; kernel counterpart
// templates/palettized_gemm.metal:16-117).
#include "common.cuh"

namespace prism {

int launch_gemm(prism_cuda_ctx *ctx, const LutTensor &t, const uint16_t *X, uint32_t m_tok, uint16_t *Y) {
    if (t.k % 8) return fail(ctx, PRISM_E_ARG, "gemm: dim_n must be a multiple of 8");
    if (ctx->gemm_variant == 1 && gemm_tc5_eligible(ctx, t, m_tok)) return launch_gemm_tc5(ctx, t, X, m_tok, Y);
    // activation rows as the batch dimension of the GEMV kernel, 32768 rows per launch
    for (uint32_t t0 = 0; t0 < m_tok; t0 += 32768) {
        const uint32_t nb = m_tok - t0 < 32768 ? m_tok - t0 : 32768;
        PRISM_TRY(launch_gemv(ctx, GEMV_PLAIN, t, nullptr, X + (size_t)t0 * t.k, t.k, Y + (size_t)t0 * t.m, t.m,
                              nullptr, nb));
    }
    return PRISM_OK;
}

}  // namespace prism
