/*
 * CPU restatement of the decoder-block operators around Vesper's attention path --
 * TEST INFRASTRUCTURE ONLY.  Only tests/, the smoke check and the benchmark's
 * cpu_baseline leg may call it; the CUDA library never links or loads it.
 * Every function cites the reference file:line it follows.  Pinned against the
 * compiled reference (oracle/_ref) and the committed fixtures in tests/golden.
 */
#ifndef VESPER_BLOCK_ORACLE_H
#define VESPER_BLOCK_ORACLE_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* y[M,N] = x[M,K] w[N,K]^T with the summation order of gemm_cpu_tiled_worker
 * (src/ops/cpu/gemm_cpu.cpp:12-48): K in chunks of 32, each chunk summed on its own
 * and then added to the output element. */
void vo_linear(const float* x, const float* w, float* y, int64_t M, int64_t N, int64_t K);
/* rms_norm_cpu_dispatch, src/ops/normalization.cpp:451-481. */
void vo_rms_norm(const float* x, const float* w, float* y, int64_t M, int64_t dim, float eps);
/* silu(gate) * up with silu(x) = x * (1 / (1 + exp(-x))): silu_cpu_dispatch
 * src/ops/elementwise.cpp:1172-1177 followed by mul (silu_mul CPU branch, :1309-1313). */
void vo_silu_mul(const float* gate, const float* up, float* y, int64_t n);
/* embedding_cpu_dispatch, src/ops/embedding.cpp:78-110 (no padding index, no max_norm).
 * Returns -1 on an id outside [0, vocab). */
int vo_embedding(const int32_t* ids, const float* table, float* y, int64_t M, int64_t vocab, int64_t dim);
/* argmax_cpu_dispatch, src/ops/sampling_ops.cpp:18-38: first maximum wins. */
void vo_argmax(const float* logits, int32_t* out, int64_t B, int64_t vocab);
/* check_stop_tokens_cpu_dispatch, src/ops/sampling_ops.cpp:263-288. */
void vo_check_stop_tokens(const int32_t* tokens, int32_t* out, int64_t B, const int64_t* stop_ids,
                          int64_t n_stop, int64_t min_generated, int64_t generated_count);

#ifdef __cplusplus
}
#endif
#endif
