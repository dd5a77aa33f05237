/*
 * prism_cuda_bench.h -- measurement entry points of libprism_cuda.
 *
 * Not part of the backend interface a Rust CudaBackend binds (include/prism_cuda.h): these exist so a
 * benchmark can time exactly one kind of launch on the context stream with CUDA events, with working
 * sets larger than L2.  None has a counterpart in the reference.
 */
#ifndef PRISM_CUDA_BENCH_H
#define PRISM_CUDA_BENCH_H

#include "prism_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Times only the palettized GEMV launches of a decode step, `reps` passes over every weight of the
 * model between two events on the context stream; returns elapsed ms, algorithmic bytes moved and
 * launches issued. */
int prism_cuda_engine_profile_gemv(prism_cuda_engine *eng, uint32_t reps, double *ms_out,
                                   uint64_t *bytes_out, uint32_t *launches_out);
/* Times one other kind of launch of the decode step in isolation, `reps` passes of all of a step's
 * launches of that kind back to back between two events: part 1 = the fused attention kernel of every
 * layer at the current position, part 2 = the tensor-parallel reduction after every row-parallel matmul
 * (two per layer; 0 launches on one GPU).  Every rank of a tensor-parallel group must make the same call. */
int prism_cuda_engine_profile_part(prism_cuda_engine *eng, uint32_t part, uint32_t reps, double *ms_out,
                                   uint32_t *launches_out);
/* Cycles through n_sets distinct weight sets (working set > L2) inside one CUDA graph replayed `reps`
 * times.  kind 0 = GEMV (1 handle per set), 1 = fused gate/up (gate, up), 2 = MLP (gate, up, down).
 * x_dev: dim_n fp16 activations on the device. */
int prism_cuda_bench_cycle(prism_cuda_ctx *ctx, int kind, const int32_t *handles, uint32_t n_sets,
                           uint32_t reps, const void *x_dev, double *ms_out);
/* `reps` prefill GEMMs of the m_tok activation rows X_dev [m_tok][dim_n] (device, fp16) against one
 * tensor between two events on the context stream. */
int prism_cuda_bench_gemm(prism_cuda_ctx *ctx, int32_t handle, const void *X_dev, uint32_t m_tok, uint32_t reps,
                          double *ms_out);

#ifdef __cplusplus
}
#endif
#endif /* PRISM_CUDA_BENCH_H */
