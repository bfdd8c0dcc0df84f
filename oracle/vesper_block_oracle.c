/* See vesper_block_oracle.h -- TEST INFRASTRUCTURE ONLY. */
#include "vesper_block_oracle.h"

#include <math.h>
#include <string.h>

void vo_linear(const float* x, const float* w, float* y, int64_t M, int64_t N, int64_t K) {
    for (int64_t i = 0; i < M; ++i) {
        for (int64_t j = 0; j < N; ++j) {
            float c = 0.0f;
            for (int64_t k0 = 0; k0 < K; k0 += 32) {
                const int64_t k1 = k0 + 32 < K ? k0 + 32 : K;
                float sum = 0.0f;
                for (int64_t k = k0; k < k1; ++k) sum += x[i * K + k] * w[j * K + k];
                c += sum;
            }
            y[i * N + j] = c;
        }
    }
}

void vo_rms_norm(const float* x, const float* w, float* y, int64_t M, int64_t dim, float eps) {
    for (int64_t i = 0; i < M; ++i) {
        const float* in = x + i * dim;
        float sum_sq = 0.0f;
        for (int64_t j = 0; j < dim; ++j) sum_sq += in[j] * in[j];
        const float rms = sqrtf(sum_sq / dim + eps);
        const float inv_rms = 1.0f / rms;
        for (int64_t j = 0; j < dim; ++j) y[i * dim + j] = in[j] * inv_rms * w[j];
    }
}

void vo_silu_mul(const float* gate, const float* up, float* y, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        const float s = 1.0f / (1.0f + expf(-gate[i]));
        y[i] = (gate[i] * s) * up[i];
    }
}

int vo_embedding(const int32_t* ids, const float* table, float* y, int64_t M, int64_t vocab, int64_t dim) {
    for (int64_t i = 0; i < M; ++i) {
        if (ids[i] < 0 || ids[i] >= vocab) return -1;
        memcpy(y + i * dim, table + (int64_t)ids[i] * dim, sizeof(float) * dim);
    }
    return 0;
}

void vo_argmax(const float* logits, int32_t* out, int64_t B, int64_t vocab) {
    for (int64_t b = 0; b < B; ++b) {
        const float* row = logits + b * vocab;
        float max_val = row[0];
        int32_t max_idx = 0;
        for (int64_t i = 1; i < vocab; ++i)
            if (row[i] > max_val) { max_val = row[i]; max_idx = (int32_t)i; }
        out[b] = max_idx;
    }
}

void vo_check_stop_tokens(const int32_t* tokens, int32_t* out, int64_t B, const int64_t* stop_ids,
                          int64_t n_stop, int64_t min_generated, int64_t generated_count) {
    for (int64_t b = 0; b < B; ++b) {
        int32_t stop = 0;
        if (generated_count >= min_generated)
            for (int64_t i = 0; i < n_stop; ++i)
                if (tokens[b] == (int32_t)stop_ids[i]) { stop = 1; break; }
        out[b] = stop;
    }
}
