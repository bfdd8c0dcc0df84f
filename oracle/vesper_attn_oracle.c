/*
 * CPU oracle for Vesper's attention hot path -- TEST INFRASTRUCTURE ONLY.
 * See vesper_attn_oracle.h.  Parity is pinned against vectors produced by the
 * unmodified reference (tests/golden).  Build with -O2 -ffp-contract=off so
 * that no fused multiply-add changes the reference's rounding sequence.
 */
#include "vesper_attn_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#define VO_MIN(a, b) ((a) < (b) ? (a) : (b))
#define VO_MAX(a, b) ((a) > (b) ? (a) : (b))

/* src/ops/flash_attention.cpp:218-364: 32x32 tiles; per query row the scores of
 * one key block are computed, the running max/sum updated and the accumulator
 * rescaled -- in exactly this order so the fp32 roundings match. */
void vo_flash_attention_fwd(const float* Q, const float* K, const float* V,
                            float* O, float* L,
                            int64_t B, int64_t H, int64_t N, int64_t D,
                            float scale, int is_causal)
{
    enum { BLOCK_M = 32, BLOCK_N = 32 };
    float* acc = (float*)malloc(sizeof(float) * BLOCK_M * (size_t)D);
    float m_prev[BLOCK_M], l_prev[BLOCK_M], scores[BLOCK_N];

    for (int64_t bh = 0; bh < B * H; ++bh) {
        const float* q_ptr = Q + bh * N * D;
        const float* k_ptr = K + bh * N * D;
        const float* v_ptr = V + bh * N * D;
        float* o_ptr = O + bh * N * D;
        float* l_ptr = L + bh * N;

        for (int64_t q_start = 0; q_start < N; q_start += BLOCK_M) {
            int64_t q_end = VO_MIN(q_start + BLOCK_M, N);
            for (int64_t i = 0; i < BLOCK_M * D; ++i) acc[i] = 0.0f;
            for (int i = 0; i < BLOCK_M; ++i) { m_prev[i] = -INFINITY; l_prev[i] = 0.0f; }

            /* :276 causal key range ends with the query block */
            int64_t k_end_limit = is_causal ? VO_MIN(q_end, N) : N;

            for (int64_t k_start = 0; k_start < k_end_limit; k_start += BLOCK_N) {
                int64_t k_end = VO_MIN(k_start + BLOCK_N, k_end_limit);
                int64_t nk = k_end - k_start;
                for (int64_t qi = q_start; qi < q_end; ++qi) {
                    int ql = (int)(qi - q_start);
                    float m_block = -INFINITY;
                    for (int64_t ki = k_start; ki < k_end; ++ki) {
                        if (is_causal && ki > qi) {           /* :293-296 */
                            scores[ki - k_start] = -INFINITY;
                            continue;
                        }
                        float score = 0.0f;                   /* :299-303 */
                        for (int64_t d = 0; d < D; ++d)
                            score += q_ptr[qi * D + d] * k_ptr[ki * D + d];
                        score *= scale;
                        scores[ki - k_start] = score;
                        m_block = VO_MAX(m_block, score);
                    }
                    float m_new = VO_MAX(m_prev[ql], m_block);  /* :309 */
                    float l_block = 0.0f;
                    for (int64_t i = 0; i < nk; ++i) {          /* :313-331 */
                        scores[i] = expf(scores[i] - m_new);
                        l_block += scores[i];
                    }
                    float scale_prev = expf(m_prev[ql] - m_new);  /* :334 */
                    l_prev[ql] = l_prev[ql] * scale_prev + l_block;
                    for (int64_t d = 0; d < D; ++d) {            /* :338-343 */
                        acc[ql * D + d] *= scale_prev;
                        for (int64_t ki = k_start; ki < k_end; ++ki)
                            acc[ql * D + d] += scores[ki - k_start] * v_ptr[ki * D + d];
                    }
                    m_prev[ql] = m_new;
                }
            }
            for (int64_t qi = q_start; qi < q_end; ++qi) {       /* :350-360 */
                int ql = (int)(qi - q_start);
                float inv_l = 1.0f / l_prev[ql];
                for (int64_t d = 0; d < D; ++d)
                    o_ptr[qi * D + d] = acc[ql * D + d] * inv_l;
                l_ptr[qi] = m_prev[ql] + logf(l_prev[ql]);
            }
        }
    }
    free(acc);
}

/* src/nn/functional.cpp:399-421 with the pieces it calls:
 * batched matmul CPU loop src/ops/gemm.cpp:252-279 (sequential fp32 sum over k),
 * scalar div src/ops/cpu/elementwise_cpu.cpp:93-95, mask add
 * src/nn/functional.cpp:26-57, softmax src/ops/normalization.cpp:83-119
 * (max, sum of exp(x-max), exp(x-max)/sum). */
void vo_sdpa_standard(const float* q, const float* k, const float* v, float* out,
                      float* scores_out,
                      int64_t B, int64_t H, int64_t Tq, int64_t Tk, int64_t D,
                      int is_causal)
{
    float sqrt_d = sqrtf((float)D);
    float* s = (float*)malloc(sizeof(float) * (size_t)Tk);
    for (int64_t bh = 0; bh < B * H; ++bh) {
        const float* qp = q + bh * Tq * D;
        const float* kp = k + bh * Tk * D;
        const float* vp = v + bh * Tk * D;
        float* op = out + bh * Tq * D;
        for (int64_t m = 0; m < Tq; ++m) {
            for (int64_t n = 0; n < Tk; ++n) {
                float sum = 0.0f;
                for (int64_t kk = 0; kk < D; ++kk) sum += qp[m * D + kk] * kp[n * D + kk];
                float sc = sum / sqrt_d;
                if (is_causal) sc = sc + ((n > m) ? -INFINITY : 0.0f);
                s[n] = sc;
            }
            if (scores_out) memcpy(scores_out + (bh * Tq + m) * Tk, s, sizeof(float) * (size_t)Tk);
            float max_val = -INFINITY;
            for (int64_t n = 0; n < Tk; ++n) if (s[n] > max_val) max_val = s[n];
            float sum_exp = 0.0f;
            for (int64_t n = 0; n < Tk; ++n) sum_exp += expf(s[n] - max_val);
            for (int64_t n = 0; n < Tk; ++n) s[n] = expf(s[n] - max_val) / sum_exp;
            for (int64_t d = 0; d < D; ++d) {
                float sum = 0.0f;
                for (int64_t n = 0; n < Tk; ++n) sum += s[n] * vp[n * D + d];
                op[m * D + d] = sum;
            }
        }
    }
    free(s);
}

/* src/nn/functional.cpp:385-395 */
int vo_sdpa(const float* q, const float* k, const float* v, float* out,
            int64_t B, int64_t H, int64_t Tq, int64_t Tk, int64_t D, int is_causal)
{
    if (Tq >= 512) {
        if (Tq != Tk) return -1;
        float scale = 1.0f / sqrtf((float)D);
        float* lse = (float*)malloc(sizeof(float) * (size_t)(B * H * Tq));
        vo_flash_attention_fwd(q, k, v, out, lse, B, H, Tq, D, scale, is_causal);
        free(lse);
        return 0;
    }
    vo_sdpa_standard(q, k, v, out, NULL, B, H, Tq, Tk, D, is_causal);
    return 0;
}

/* src/nn/functional.cpp:424-441: float pow, then int * float. */
void vo_rope_frequencies(int T, int D, int start_pos, float theta, float* freqs)
{
    int half = D / 2;
    for (int m = 0; m < T; ++m) {
        int pos = start_pos + m;
        for (int i = 0; i < half; ++i) {
            float freq = powf(theta, -2.0f * i / D);
            freqs[m * half + i] = pos * freq;
        }
    }
}

/* src/nn/functional.cpp:443-494; cos/sin are fp32 std::cos/std::sin
 * (src/ops/elementwise.cpp:1038-1044); out_r = x_r*cos - x_i*sin and
 * out_i = x_r*sin + x_i*cos, each product rounded to fp32 first (separate
 * mul/sub/add ops, :472-478). */
void vo_apply_rotary_emb(const float* x, const float* freqs, float* out,
                         int64_t B, int64_t H, int64_t S, int64_t D)
{
    int64_t half = D / 2;
    for (int64_t bh = 0; bh < B * H; ++bh)
        for (int64_t s = 0; s < S; ++s)
            for (int64_t i = 0; i < half; ++i) {
                float c = cosf(freqs[s * half + i]);
                float sn = sinf(freqs[s * half + i]);
                float xr = x[(bh * S + s) * D + 2 * i];
                float xi = x[(bh * S + s) * D + 2 * i + 1];
                float t1 = xr * c, t2 = xi * sn, t3 = xr * sn, t4 = xi * c;
                out[(bh * S + s) * D + 2 * i] = t1 - t2;
                out[(bh * S + s) * D + 2 * i + 1] = t3 + t4;
            }
}

/* src/ops/attention_ops.cpp:30-57 */
void vo_repeat_kv(const float* in, float* out,
                  int64_t B, int64_t KVH, int64_t S, int64_t D, int64_t n_rep)
{
    int64_t QH = KVH * n_rep;
    for (int64_t b = 0; b < B; ++b)
        for (int64_t qh = 0; qh < QH; ++qh) {
            int64_t kvh = qh / n_rep;
            memcpy(out + ((b * QH + qh) * S) * D, in + ((b * KVH + kvh) * S) * D,
                   sizeof(float) * (size_t)(S * D));
        }
}

/* src/nn/transformer.cpp:56-93 */
void vo_kv_cache_update(float* k_cache, float* v_cache,
                        const float* new_k, const float* new_v,
                        int64_t B, int64_t H, int64_t cap, int64_t D,
                        int64_t T, int64_t start_pos, int64_t* current_len)
{
    for (int64_t bh = 0; bh < B * H; ++bh) {
        memcpy(k_cache + (bh * cap + start_pos) * D, new_k + bh * T * D, sizeof(float) * (size_t)(T * D));
        memcpy(v_cache + (bh * cap + start_pos) * D, new_v + bh * T * D, sizeof(float) * (size_t)(T * D));
    }
    if (start_pos + T > *current_len) *current_len = start_pos + T;
}

void vo_cache_active(const float* cache, float* out,
                     int64_t B, int64_t H, int64_t cap, int64_t D, int64_t len)
{
    for (int64_t bh = 0; bh < B * H; ++bh)
        memcpy(out + bh * len * D, cache + bh * cap * D, sizeof(float) * (size_t)(len * D));
}

/* LSE of one query row from fp32 scaled scores, in double:
 * m + ln sum exp(s - m), the quantity src/ops/flash_attention.cpp:359 stores. */
static float vo_row_lse(const float* s, int64_t n)
{
    double m = -INFINITY;
    for (int64_t i = 0; i < n; ++i) if (s[i] > m) m = s[i];
    double sum = 0.0;
    for (int64_t i = 0; i < n; ++i) sum += exp((double)s[i] - m);
    return (float)(m + log(sum));
}

/* Standard path with a bottom-right aligned causal mask (key j visible to
 * query i iff j <= offset+i); offset = Tk-Tq.  Same arithmetic as
 * vo_sdpa_standard; with offset 0 the two are identical. */
static void vo_sdpa_offset(const float* q, const float* k, const float* v, float* out,
                           float* lse_out, int64_t BH, int64_t Tq, int64_t Tk, int64_t D,
                           int is_causal, int64_t offset)
{
    float sqrt_d = sqrtf((float)D);
    float* s = (float*)malloc(sizeof(float) * (size_t)Tk);
    float* p = (float*)malloc(sizeof(float) * (size_t)Tk);
    for (int64_t bh = 0; bh < BH; ++bh) {
        const float* qp = q + bh * Tq * D;
        const float* kp = k + bh * Tk * D;
        const float* vp = v + bh * Tk * D;
        float* op = out + bh * Tq * D;
        for (int64_t m = 0; m < Tq; ++m) {
            for (int64_t n = 0; n < Tk; ++n) {
                float sum = 0.0f;
                for (int64_t kk = 0; kk < D; ++kk) sum += qp[m * D + kk] * kp[n * D + kk];
                float sc = sum / sqrt_d;
                if (is_causal) sc = sc + ((n > m + offset) ? -INFINITY : 0.0f);
                s[n] = sc;
            }
            if (lse_out) lse_out[bh * Tq + m] = vo_row_lse(s, Tk);
            float max_val = -INFINITY;
            for (int64_t n = 0; n < Tk; ++n) if (s[n] > max_val) max_val = s[n];
            float sum_exp = 0.0f;
            for (int64_t n = 0; n < Tk; ++n) sum_exp += expf(s[n] - max_val);
            for (int64_t n = 0; n < Tk; ++n) p[n] = expf(s[n] - max_val) / sum_exp;
            for (int64_t d = 0; d < D; ++d) {
                float sum = 0.0f;
                for (int64_t n = 0; n < Tk; ++n) sum += p[n] * vp[n * D + d];
                op[m * D + d] = sum;
            }
        }
    }
    free(s); free(p);
}

/* src/nn/gqa_attention.cpp:111-159 (steps 2-6), see the header for how the
 * cache views are made contiguous before repeat_kv. */
int vo_gqa_attention_cached(const float* q, const float* k_new, const float* v_new,
                            float* k_cache, float* v_cache,
                            float* out, float* lse_out,
                            int64_t B, int64_t Hq, int64_t Hkv, int64_t T, int64_t D,
                            int64_t cap, int64_t start_pos, float theta, int use_rope,
                            int64_t* current_len)
{
    int64_t n_rep = Hq / Hkv;
    size_t nq = (size_t)(B * Hq * T * D), nk = (size_t)(B * Hkv * T * D);
    float* q_rot = (float*)malloc(sizeof(float) * nq);
    float* k_rot = (float*)malloc(sizeof(float) * nk);
    if (use_rope) {
        float* freqs = (float*)malloc(sizeof(float) * (size_t)(T * (D / 2)));
        vo_rope_frequencies((int)T, (int)D, (int)start_pos, theta, freqs);
        vo_apply_rotary_emb(q, freqs, q_rot, B, Hq, T, D);
        vo_apply_rotary_emb(k_new, freqs, k_rot, B, Hkv, T, D);
        free(freqs);
    } else {
        memcpy(q_rot, q, sizeof(float) * nq);
        memcpy(k_rot, k_new, sizeof(float) * nk);
    }
    vo_kv_cache_update(k_cache, v_cache, k_rot, v_new, B, Hkv, cap, D, T, start_pos, current_len);
    int64_t len = *current_len;

    size_t nact = (size_t)(B * Hkv * len * D);
    float* k_act = (float*)malloc(sizeof(float) * nact);
    float* v_act = (float*)malloc(sizeof(float) * nact);
    vo_cache_active(k_cache, k_act, B, Hkv, cap, D, len);
    vo_cache_active(v_cache, v_act, B, Hkv, cap, D, len);
    float* k_rep = k_act; float* v_rep = v_act;
    if (n_rep > 1) {                       /* src/ops/attention_ops.cpp:93-95 */
        k_rep = (float*)malloc(sizeof(float) * nact * (size_t)n_rep);
        v_rep = (float*)malloc(sizeof(float) * nact * (size_t)n_rep);
        vo_repeat_kv(k_act, k_rep, B, Hkv, len, D, n_rep);
        vo_repeat_kv(v_act, v_rep, B, Hkv, len, D, n_rep);
    }
    int use_causal = (T > 1);              /* src/nn/gqa_attention.cpp:146 */
    if (T >= 512 && T == len) {            /* flash route, src/nn/functional.cpp:387 */
        float scale = 1.0f / sqrtf((float)D);
        float* lse = lse_out ? lse_out : (float*)malloc(sizeof(float) * (size_t)(B * Hq * T));
        vo_flash_attention_fwd(q_rot, k_rep, v_rep, out, lse, B, Hq, T, D, scale, use_causal);
        if (!lse_out) free(lse);
    } else {
        vo_sdpa_offset(q_rot, k_rep, v_rep, out, lse_out, B * Hq, T, len, D, use_causal, len - T);
    }
    if (n_rep > 1) { free(k_rep); free(v_rep); }
    free(k_act); free(v_act); free(q_rot); free(k_rot);
    return 0;
}

void vo_decode_ragged(const float* q, const float* k_cache, const float* v_cache,
                      const int32_t* lens, float* out, float* lse_out,
                      int64_t B, int64_t Hq, int64_t Hkv, int64_t cap, int64_t D)
{
    int64_t n_rep = Hq / Hkv;
    for (int64_t b = 0; b < B; ++b)
        for (int64_t h = 0; h < Hq; ++h) {
            int64_t kvh = h / n_rep;       /* src/ops/attention_ops.cpp:47 */
            const float* kp = k_cache + (b * Hkv + kvh) * cap * D;
            const float* vp = v_cache + (b * Hkv + kvh) * cap * D;
            vo_sdpa_offset(q + (b * Hq + h) * D, kp, vp, out + (b * Hq + h) * D,
                           lse_out ? lse_out + (b * Hq + h) : NULL,
                           1, 1, lens[b], D, 0, 0);
        }
}

void vo_lse_combine(const float* m, const float* l, const float* o,
                    float* out, float* lse_out,
                    int64_t R, int64_t rows, int64_t D)
{
    for (int64_t r = 0; r < rows; ++r) {
        float m_star = -INFINITY;
        for (int64_t p = 0; p < R; ++p) m_star = VO_MAX(m_star, m[p * rows + r]);
        float l_star = 0.0f;
        for (int64_t p = 0; p < R; ++p) l_star += l[p * rows + r] * expf(m[p * rows + r] - m_star);
        for (int64_t d = 0; d < D; ++d) {
            float acc = 0.0f;
            for (int64_t p = 0; p < R; ++p)
                acc += o[(p * rows + r) * D + d] * l[p * rows + r] * expf(m[p * rows + r] - m_star);
            out[r * D + d] = acc / l_star;
        }
        if (lse_out) lse_out[r] = m_star + logf(l_star);
    }
}

/* include/vesper/core/half.h:162-173 (bias 0x7FFF + lsb, then truncate). */
float vo_bf16_round(float x)
{
    uint32_t bits;
    memcpy(&bits, &x, sizeof(bits));
    uint32_t bias = 0x7FFFu + ((bits >> 16) & 1u);
    bits += bias;
    bits &= 0xFFFF0000u;
    float r;
    memcpy(&r, &bits, sizeof(r));
    return r;
}

void vo_bf16_round_array(const float* in, float* out, int64_t n)
{
    for (int64_t i = 0; i < n; ++i) out[i] = vo_bf16_round(in[i]);
}

void vo_flash_attention_bwd(const float* d_out, const float* q, const float* k, const float* v,
                            const float* out, const float* lse, float* dq, float* dk, float* dv,
                            int64_t B, int64_t H, int64_t N, int64_t D, float scale, int causal) {
    memset(dq, 0, sizeof(float) * (size_t)(B * H * N * D));
    memset(dk, 0, sizeof(float) * (size_t)(B * H * N * D));
    memset(dv, 0, sizeof(float) * (size_t)(B * H * N * D));
    float* Di = (float*)malloc(sizeof(float) * (size_t)N);
    for (int64_t bh = 0; bh < B * H; ++bh) {
        const float* qp = q + bh * N * D; const float* kp = k + bh * N * D; const float* vp = v + bh * N * D;
        const float* op = out + bh * N * D; const float* dop = d_out + bh * N * D; const float* lp = lse + bh * N;
        float* dqp = dq + bh * N * D; float* dkp = dk + bh * N * D; float* dvp = dv + bh * N * D;
        for (int64_t i = 0; i < N; ++i) {
            float sum = 0.0f;
            for (int64_t d = 0; d < D; ++d) sum += dop[i * D + d] * op[i * D + d];
            Di[i] = sum;
        }
        for (int64_t qi = 0; qi < N; ++qi) {
            const float li = lp[qi];
            const int64_t k_end = causal ? qi + 1 : N;
            for (int64_t ki = 0; ki < k_end; ++ki) {
                float score = 0.0f;
                for (int64_t d = 0; d < D; ++d) score += qp[qi * D + d] * kp[ki * D + d];
                score *= scale;
                const float p = expf(score - li);
                for (int64_t d = 0; d < D; ++d) dvp[ki * D + d] += p * dop[qi * D + d];
                float dp = 0.0f;
                for (int64_t d = 0; d < D; ++d) dp += dop[qi * D + d] * vp[ki * D + d];
                const float ds = p * (dp - Di[qi]);
                for (int64_t d = 0; d < D; ++d) {
                    dqp[qi * D + d] += scale * ds * kp[ki * D + d];
                    dkp[ki * D + d] += scale * ds * qp[qi * D + d];
                }
            }
        }
    }
    free(Di);
}
