/*
 * CPU oracle for Vesper's attention hot path -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the reference's fp32 CPU algorithms, kept in the
 * reference's own operation order so that results agree with the reference
 * bit for bit on the same toolchain.  Nothing in the shipped CUDA path may
 * call into this file; only the parity tests, the smoke check and the CPU
 * baseline leg of the benchmark use it, and only as the checker.
 *
 * Parity is pinned: tests/golden holds input/output vectors produced by the
 * unmodified reference (built by oracle/Makefile from the reference sources)
 * and tests/test_oracle_golden.py checks this restatement against them.
 *
 * Every function cites the reference file:line it follows (paths relative to
 * the reference project root).
 */
#ifndef VESPER_ATTN_ORACLE_H
#define VESPER_ATTN_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ops::flash_attention_cpu_dispatch, src/ops/flash_attention.cpp:218-364.
 * q,k,v,o: [B,H,N,D] contiguous fp32; lse: [B,H,N] (natural log). */
void vo_flash_attention_fwd(const float* q, const float* k, const float* v,
                            float* o, float* lse,
                            int64_t B, int64_t H, int64_t N, int64_t D,
                            float scale, int is_causal);

/* Standard path of functional::scaled_dot_product_attention,
 * src/nn/functional.cpp:399-421 (matmul -> div sqrt(D) -> +mask -> softmax -> matmul).
 * q: [B,H,Tq,D]; k,v: [B,H,Tk,D]; out: [B,H,Tq,D].  is_causal requires Tq==Tk
 * (the reference adds a [Tq,Tq] mask to [Tq,Tk] scores).
 * scores_out (nullable): [B,H,Tq,Tk] scaled (and masked) scores before softmax. */
void vo_sdpa_standard(const float* q, const float* k, const float* v, float* out,
                      float* scores_out,
                      int64_t B, int64_t H, int64_t Tq, int64_t Tk, int64_t D,
                      int is_causal);

/* Router functional::scaled_dot_product_attention, src/nn/functional.cpp:370-422:
 * query length >= 512 goes to the flash op with scale 1/sqrt(D), else the
 * standard path.  Returns 0, or -1 when the flash route is taken with Tq != Tk
 * (the reference throws there, src/ops/flash_attention.cpp:49-51). */
int vo_sdpa(const float* q, const float* k, const float* v, float* out,
            int64_t B, int64_t H, int64_t Tq, int64_t Tk, int64_t D, int is_causal);

/* functional::compute_rope_frequencies, src/nn/functional.cpp:424-441.
 * freqs: [T, D/2] angles (start_pos+m) * theta^(-2i/D), all in fp32. */
void vo_rope_frequencies(int T, int D, int start_pos, float theta, float* freqs);

/* functional::apply_rotary_emb, src/nn/functional.cpp:443-494: rotation of the
 * adjacent pairs (x[2i], x[2i+1]) by freqs[s,i].  x,out: [B,H,S,D]. */
void vo_apply_rotary_emb(const float* x, const float* freqs, float* out,
                         int64_t B, int64_t H, int64_t S, int64_t D);

/* ops::repeat_kv_cpu_dispatch, src/ops/attention_ops.cpp:30-57 on a
 * CONTIGUOUS input.  in: [B,KVH,S,D]; out: [B,KVH*n_rep,S,D]. */
void vo_repeat_kv(const float* in, float* out,
                  int64_t B, int64_t KVH, int64_t S, int64_t D, int64_t n_rep);

/* nn::KVCache::update, src/nn/transformer.cpp:56-93.  Caches [B,H,cap,D];
 * new_k,new_v [B,H,T,D] are written at rows start_pos..start_pos+T;
 * *current_len = max(*current_len, start_pos+T). */
void vo_kv_cache_update(float* k_cache, float* v_cache,
                        const float* new_k, const float* new_v,
                        int64_t B, int64_t H, int64_t cap, int64_t D,
                        int64_t T, int64_t start_pos, int64_t* current_len);

/* Contiguous copy of the active view [:,:,0:len,:] of a [B,H,cap,D] cache
 * (what Tensor::contiguous() gives for the view returned by KVCache::update). */
void vo_cache_active(const float* cache, float* out,
                     int64_t B, int64_t H, int64_t cap, int64_t D, int64_t len);

/* The attention core of GroupedQueryAttention::forward(x, cache, start_pos),
 * src/nn/gqa_attention.cpp:111-159, between the QKV projection and the output
 * projection, composed from the functions above with the cache views made
 * contiguous before repeat_kv (the reference indexes the strided view as if it
 * were contiguous, src/ops/attention_ops.cpp:34-52, which is wrong whenever
 * n_rep > 1 and cap != current_len):
 *   RoPE(q,k at start_pos) -> cache update -> contiguous -> repeat_kv ->
 *   SDPA(causal = T>1).
 * q: [B,Hq,T,D]; k_new,v_new: [B,Hkv,T,D]; caches [B,Hkv,cap,D]; out [B,Hq,T,D].
 * For T>1 with start_pos>0 (not expressible in the reference) the mask is
 * bottom-right aligned: key j visible to query i iff j <= start_pos+i.
 * lse_out (nullable): [B,Hq,T] natural-log LSE of the scaled scores, in double
 * arithmetic from fp32 scores.  Returns 0. */
int vo_gqa_attention_cached(const float* q, const float* k_new, const float* v_new,
                            float* k_cache, float* v_cache,
                            float* out, float* lse_out,
                            int64_t B, int64_t Hq, int64_t Hkv, int64_t T, int64_t D,
                            int64_t cap, int64_t start_pos, float theta, int use_rope,
                            int64_t* current_len);

/* Decode against per-sequence lengths (an extension the reference cannot
 * express, defined as the reference's standard path applied per sequence on
 * contiguous slices).  q: [B,Hq,D] (already rotated), caches [B,Hkv,cap,D],
 * lens[B]; out [B,Hq,D]; lse_out (nullable) [B,Hq]. */
void vo_decode_ragged(const float* q, const float* k_cache, const float* v_cache,
                      const int32_t* lens, float* out, float* lse_out,
                      int64_t B, int64_t Hq, int64_t Hkv, int64_t cap, int64_t D);

/* Log-sum-exp merge of R partial results, the algebra of
 * src/ops/flash_attention.cpp:309-345 applied across partials:
 * m* = max m_r, l* = sum l_r e^{m_r-m*}, O* = sum O_r l_r e^{m_r-m*} / l*.
 * m,l: [R,rows]; o: [R,rows,D] (each O_r already normalised by l_r);
 * out [rows,D]; lse_out (nullable) [rows] = m* + ln l*. */
void vo_lse_combine(const float* m, const float* l, const float* o,
                    float* out, float* lse_out,
                    int64_t R, int64_t rows, int64_t D);

/* Round-to-nearest-even fp32 -> bf16 -> fp32, include/vesper/core/half.h:162-173. */
/* flash_attention_backward_cpu_dispatch, src/ops/flash_attention.cpp:366-482 (no dropout):
 * Di = rowsum(dO * O); for every visible (query i, key j): p = exp(scale q_i.k_j - lse_i),
 * dV_j += p dO_i, dS = p (dO_i.v_j - Di_i), dQ_i += scale dS k_j, dK_j += scale dS q_i,
 * accumulated in the reference's loop order.  All tensors [B,H,N,D] fp32, lse [B,H,N];
 * dq, dk, dv are overwritten. */
void vo_flash_attention_bwd(const float* d_out, const float* q, const float* k, const float* v,
                            const float* out, const float* lse, float* dq, float* dk, float* dv,
                            int64_t B, int64_t H, int64_t N, int64_t D, float scale, int causal);

float vo_bf16_round(float x);
void vo_bf16_round_array(const float* in, float* out, int64_t n);

#ifdef __cplusplus
}
#endif
#endif
