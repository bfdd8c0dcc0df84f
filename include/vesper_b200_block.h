/*
 * vesper_b200 -- C ABI of the decoder-block operators that surround the
 * attention hot path (projections, normalisation, gated MLP, embedding, greedy
 * sampling).  Same conventions as vesper_b200.h: every pointer is borrowed
 * device memory, nothing is allocated or freed, launches are asynchronous on
 * the caller's stream, the return value is VB200_OK or a negative vb200_status.
 * "file:line" citations name the reference interface each entry point stands
 * behind, relative to the reference project root.
 *
 * Number formats: weights and activations bf16, the residual stream and the
 * logits fp32, all accumulation fp32.
 */
#ifndef VESPER_B200_BLOCK_H
#define VESPER_B200_BLOCK_H

#include "vesper_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* What vb200_linear does with each accumulated output element acc[m, n]. */
typedef enum vb200_epilogue {
    VB200_EPI_BF16 = 0,     /* out_bf16[m, n]  = acc                                            */
    VB200_EPI_F32 = 1,      /* out_f32[m, n]   = acc            (logits)                        */
    VB200_EPI_ADD_F32 = 2,  /* out_f32[m, n]  += acc            (residual: h = h + proj(x))     */
    VB200_EPI_SWIGLU = 3    /* out_bf16[m, n/2] = silu(acc[m, n]) * acc[m, n+1], n even:
                               W holds gate and up rows interleaved (row 2j = gate_j,
                               row 2j+1 = up_j), see vb200_interleave_rows                      */
} vb200_epilogue;

/* y = x W^T.  x [M, K] bf16 with row stride ldx, W [N, K] bf16 with row stride
 * ldw (the layout of nn::Linear::weight), out [M, N] (or [M, N/2]) with row
 * stride ldo; strides in elements.  K % 8 == 0, bases and strides 16-byte
 * aligned.  M <= 64 runs the weight-streaming kernel (K split over a cluster,
 * `splits` = 0 lets the library choose), larger M the tiled tensor-core kernel.
 * Replaces gemm_cuda_dispatch(a, b, c, false, true) as nn::Linear::forward and
 * FusedQKVLinear::forward_split use it (src/ops/gemm.cpp:13,183;
 * src/nn/linear.cpp:41-48, 86-104), the residual ops::add of
 * ModelTransformerBlock::forward (src/models/transformer_block.cpp:183-205)
 * and silu_mul_cuda_dispatch (include/vesper/ops/elementwise.h:105) when the
 * epilogue asks for them. */
int vb200_linear(int device, void* stream, const void* x, int64_t ldx, const void* w, int64_t ldw,
                 void* out, int64_t ldo, int32_t M, int32_t N, int32_t K, int32_t epilogue, int32_t splits);

/* y = x W^T + bias: vb200_linear with nn::Linear's optional bias (fp32 [N], src/nn/linear.cpp:26-35,44-46)
 * added to every output row before the epilogue's own step (for VB200_EPI_SWIGLU the bias has the
 * interleaved gate / up layout of the weight rows).  bias == NULL is vb200_linear. */
int vb200_linear_bias(int device, void* stream, const void* x, int64_t ldx, const void* w, int64_t ldw,
                      const float* bias, void* out, int64_t ldo, int32_t M, int32_t N, int32_t K,
                      int32_t epilogue, int32_t splits);

/* The same product in fp32 (x, W, out fp32; bias fp32 [N] or NULL; any M, N, K and strides >= the row), on CUDA
 * cores: the number format of the reference's own modules (nn::Linear::forward, src/nn/linear.cpp:41-48, on fp32
 * tensors through gemm_cuda_dispatch, src/ops/cuda/gemm.cu:257-388), kept so that fp32 modules are not silently
 * down-converted.  Not tuned: the serving path is bf16. */
int vb200_linear_f32(int device, void* stream, const float* x, int64_t ldx, const float* w, int64_t ldw, const float* bias,
                     float* out, int64_t ldo, int32_t M, int32_t N, int32_t K);

/* The general form, with every option of the GEMM kernels.  Beyond bias and epilogue it carries the two
 * halves of a DEFERRED RMSNorm, which removes the norm kernels from a decode step:
 *     rmsnorm(h) * g @ W^T  =  inv_rms(h) * ((h * g) @ W^T)        (inv_rms is one scalar per row)
 *   producer (epilogue VB200_EPI_ADD_F32, out = the fp32 residual stream h): scaled_copy [M, N] bf16 also
 *     receives bf16(h_new * copy_scale), copy_scale [N] = the weight g of the NEXT norm;
 *   consumer (x = that scaled copy): every output row is multiplied by inv_rms of the matching fp32 row of
 *     rms_rows [M, rms_dim] (M <= 64: computed inside the kernel while the weights stream), or by
 *     row_scale [M] precomputed with vb200_row_inv_rms (any M).  The scale applies before bias and epilogue. */
typedef struct vb200_linear_args {
    size_t struct_size;
    int32_t device;
    void* stream;
    const void* x;  int64_t ldx;        /* [M, K] bf16 */
    const void* w;  int64_t ldw;        /* [N, K] bf16 */
    void* out;      int64_t ldo;
    int32_t M, N, K;
    int32_t epilogue;                   /* vb200_epilogue */
    int32_t splits;
    const float* bias;                  /* [N] or NULL */
    void* scaled_copy;                  /* [M, N] bf16, row stride N, or NULL (VB200_EPI_ADD_F32 only) */
    const float* copy_scale;            /* [N] */
    const float* rms_rows;              /* [M, rms_dim] fp32, row stride rms_ld elements (0 = rms_dim), or NULL */
    int64_t rms_ld;
    int32_t rms_dim;
    float rms_eps;
    const float* row_scale;             /* [M] or NULL */
} vb200_linear_args;
int vb200_linear_ex(const vb200_linear_args* a);
/* inv_rms[m] = 1 / sqrt(mean(h[m, :]^2) + eps), h fp32 [M, dim] with row stride ld elements. */
int vb200_row_inv_rms(int device, void* stream, const float* h, int64_t ld, float* inv_rms, int32_t M, int32_t dim, float eps);
/* vb200_embedding plus scaled_out[m, :] = bf16(out[m, :] * scale) (no 1/rms): the producer half of a deferred norm. */
int vb200_embedding_scaled(int device, void* stream, const void* ids, int32_t ids64, const void* table,
                           float* out, int32_t M, int32_t dim, int32_t vocab, const float* scale, void* scaled_out);

/* h += x W^T followed by the RMSNorm of the finished rows, xn = rmsnorm(h) * norm_weight (bf16) -- the
 * output projection / down projection of a block, its residual add, and the NEXT norm in the block
 * sequence (src/models/transformer_block.cpp:183-205) as one call (two launches chained by
 * programmatic dependent launch).  h [M, N] fp32 and xn [M, N] bf16 are contiguous (row stride N). */
int vb200_linear_add_rmsnorm(int device, void* stream, const void* x, int64_t ldx, const void* w, int64_t ldw,
                             float* h, int32_t M, int32_t N, int32_t K, const float* norm_weight, float eps,
                             void* xn_out, int32_t splits);

/* out[2j] = a[j], out[2j+1] = b[j] for j < rows, rows of `cols` bf16 elements:
 * builds the interleaved (gate, up) weight VB200_EPI_SWIGLU expects from
 * SwiGLUMLP's gate_proj / up_proj weights (src/nn/swiglu.cpp:20-34). */
int vb200_interleave_rows(int device, void* stream, const void* a, const void* b, void* out,
                          int64_t rows, int64_t cols);

/* RMSNorm over the last dimension: out_bf16[m, :] = x[m, :] * rsqrt(mean(x^2) + eps) * weight,
 * x fp32 [M, dim] (the residual stream), weight fp32 [dim].  Replaces
 * rms_norm_cuda_dispatch (src/ops/normalization.cpp:446-450; CPU form :451-481). */
int vb200_rms_norm(int device, void* stream, const float* x, const float* weight, void* out_bf16,
                   int32_t M, int32_t dim, float eps);

/* out_bf16 = silu(gate) * up elementwise over n bf16 elements.  Replaces
 * silu_mul_cuda_dispatch (src/ops/elementwise.cpp:1297-1328) for callers that
 * keep separate gate / up projections. */
int vb200_silu_mul(int device, void* stream, const void* gate, const void* up, void* out, int64_t n);

/* out_f32[m, :] = table_bf16[ids[m], :], ids int32 (ids64 == 0) or int64.
 * Replaces embedding_cuda_dispatch (include/vesper/ops/embedding.h:19).  An id
 * outside [0, vocab) writes zeros and sets the kernel status word. */
int vb200_embedding(int device, void* stream, const void* ids, int32_t ids64, const void* table,
                    float* out, int32_t M, int32_t dim, int32_t vocab);
/* The same gather, plus xn_out[m, :] = rmsnorm(out[m, :]) * norm_weight (bf16): embedding and the first
 * block's attention norm in one launch. */
int vb200_embedding_rmsnorm(int device, void* stream, const void* ids, int32_t ids64, const void* table,
                            float* out, int32_t M, int32_t dim, int32_t vocab, const float* norm_weight,
                            float eps, void* xn_out);

/* Greedy step: out_ids[b] = argmax_v logits[b, v] (first maximum wins, as
 * argmax_cpu_dispatch, src/ops/sampling_ops.cpp:18-38; replaces
 * argmax_cuda_dispatch, include/vesper/ops/sampling_ops.h:62).  Optional, all
 * on the device so a generation loop needs no host round trip
 * (src/generation/generator.cpp:75-131):
 *   history + history_ld + step : also stores the id at history[b*history_ld + step]
 *   pos_dev[B] + pos_base       : when pos_dev is given the column is pos_dev[b] instead
 *                                 of `step` (e.g. the per-sequence cache lengths the decode
 *                                 kernel advances, so a replayed CUDA graph needs no new
 *                                 arguments) and the number generated so far is
 *                                 pos_dev[b] - pos_base + 1, else step + 1
 *   stop_ids[n_stop], done[B]   : done[b] |= id in stop_ids (check_stop_tokens,
 *                                 src/ops/sampling_ops.cpp:263-288), applied
 *                                 when the number generated >= min_new_tokens */
typedef struct vb200_greedy_args {
    size_t struct_size;
    int32_t device;
    void* stream;
    const float* logits;   /* [B, vocab], row stride ld_logits */
    int64_t ld_logits;
    int32_t B, vocab;
    int32_t* out_ids;      /* [B] */
    int32_t* history;      /* nullable */
    int64_t history_ld;
    int32_t step;
    const int32_t* stop_ids;  /* nullable, device */
    int32_t n_stop;
    int32_t min_new_tokens;
    int32_t* done;         /* nullable, [B] */
    const int32_t* pos_dev;   /* nullable, device [B] */
    int32_t pos_base;
} vb200_greedy_args;
int vb200_greedy_step(const vb200_greedy_args* a);

#ifdef __cplusplus
}
#endif
#endif /* VESPER_B200_BLOCK_H */
