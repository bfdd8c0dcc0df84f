// Internal launch interfaces between api.cu and the kernel translation units.
#pragma once

#include "common.cuh"
#include "../../include/vesper_b200_block.h"

namespace vb200 {

constexpr int kMaxHalfDim = 64;   // head_dim <= 128

struct InvFreq {
    float v[kMaxHalfDim];
};

// A strided [B,H,S,D] view in elements.
struct View4 {
    void* ptr;
    long long sb, sh, ss;
};
inline View4 to_view(const vb200_tensor4& t) { return View4{t.ptr, t.stride_b, t.stride_h, t.stride_s}; }

// ---- rope_append.cu ----
// table[t][i] = (cos, sin)(float(start_pos + t) * inv_freq[i]),  t < T, i < D/2
int launch_rope_table(cudaStream_t s, float2* table, int T, int D, int start_pos, const InvFreq& f);
// dst rows [dst_row0, dst_row0+T) of k_dst/v_dst <- rotate(k) / v.  table == nullptr: no rotation.
// v / v_dst may be null (K only).
// inv_freq != nullptr (with table == nullptr): angles computed in the kernel for positions dst_row0 + t.
int launch_kv_append(cudaStream_t s, int dtype, int B, int H, int T, int D,
                     View4 k, View4 v, View4 k_dst, View4 v_dst, int dst_row0, const float2* table,
                     const InvFreq* inv_freq = nullptr);
// table + rotated K + V rows in one launch: table[t][i] as launch_rope_table writes it, k_dst / v_dst rows
// [dst_row0, dst_row0 + T) as launch_kv_append does with that table.  v / v_dst may be null (K only).
int launch_rope_append_fused(cudaStream_t s, int dtype, int B, int H, int T, int D, View4 k, View4 v, View4 k_dst, View4 v_dst,
                             int dst_row0, float2* table, const InvFreq& f);
int launch_apply_rope_f32(cudaStream_t s, float* x, const float* cos_t, const float* sin_t,
                          int batch, int heads, int seq_len, int head_dim);
int launch_repeat_kv(cudaStream_t s, int dtype, View4 in, void* out, int B, int Hkv, int S, int D, int n_rep);

// ---- prefill_f32.cu / prefill_sm100.cu ----
struct PrefillParams {
    int dtype;
    int B, Hq, Hkv, T, D;
    int Skv;            // number of keys = start_pos + T
    int start_pos;      // causal offset: key j visible to query i iff j <= start_pos + i
    int causal;
    float scale;
    View4 q, k, v, o;   // k, v: the tensors attention reads (cache or inputs), [B,Hkv,>=Skv,D]
    float* lse;         // [B,Hq,T] or null
    const float2* q_rope_table;   // [T, D/2] (cos,sin) for the query rows, or null
    InvFreq inv_freq;             // rotation frequencies (valid when q_rope_table is set)
    int* status;                  // device status word (bounded waits)
};
int launch_prefill_f32(cudaStream_t s, const PrefillParams& p);
int launch_prefill_sm100(cudaStream_t s, const PrefillParams& p);
int launch_prefill_pair_sm100(cudaStream_t s, const PrefillParams& p);   // head_dim 128: two SMs per work item (cta_group::2)

// ---- decode_exchange.cu (declared first: the decode kernel can run the exchange as its tail) ----
struct ExchangeParams {
    int world, rank;
    void* peers[VB200_EXCHANGE_MAX_WORLD];   // exchange buffer of every rank as this GPU addresses it; [rank] = own
    const float* partial;                    // local [rows, D+2]
    long long rows;
    long long rows_per_cta;                  // filled in by the launcher
    int stage_floats;                        // dynamic shared memory of the stand-alone kernel, in floats (0: none)
    int D, dtype;
    void* out;                               // [rows, D]
    float* lse;                              // [rows] or null
    unsigned step;                           // 0 = take the next step number from the buffer's own counter
    long long timeout_cycles;
    int* status;
};

// ---- decode_splitkv.cu ----
struct DecodeParams {
    int dtype;
    int B, Hq, Hkv, D;
    float scale;
    View4 q, k_new, v_new, o;
    float* lse;
    View4 k_cache, v_cache;
    int cache_cap;
    int* seq_lens;
    int uniform_len;
    int advance_lens;
    int append;          // 1: k_new/v_new are appended at row len and attended to
    int rope;
    InvFreq inv_freq;
    long long pos_offset;
    int num_splits;      // resolved (>= 1)
    int chunk;           // keys per split (multiple of the kernel's tile)
    float* partial_out;  // null or [B,Hq,D+2]
    const int* q_positions;  // device int32[B]: absolute position of the query, or null (= pos_offset + len)
    float* workspace;    // ws_header ints (length used per sequence), then [B,Hkv,num_splits,n_rep,D+2]
    int ws_header;       // floats reserved at the front of the workspace (multiple of 64)
    int* status;         // device status word (bounded waits)
    int cluster_merge;   // 1: the splits of a (batch, kv_head) form one thread-block cluster that merges its partials itself
    // Sequence-sharded decode in ONE launch (warp-MMA split kernel only): the CTA that delivers the last split of a
    // (batch, kv_head) merges the splits and runs the exchange protocol for that group's rows (exchange_rows in
    // decode_exchange.cuh) -- no combine kernel, no exchange kernel, no partial records in HBM.
    int fused_exchange;
    ExchangeParams xchg;
};
// Length bookkeeping of one decode step for sequence b, shared by the split kernels and the combine
// kernel.  len = cached keys attended to; append = whether the new token is written and attended to.
// The token does not fit when len + 1 exceeds the cache capacity or the num_splits * chunk keys the
// grid was planned for: then it is skipped (no write, no length advance), `overflow` is set and the
// split kernel records it in the status word.  A length beyond what the grid covers is clamped too.
struct StepLen {
    int len, total;
    bool append, overflow;
    // packed into the workspace header slot of the sequence: bit 30 = appended, low bits = total
    __host__ __device__ int header() const { return total | (append ? (1 << 30) : 0); }
    __host__ __device__ static int header_total(int h) { return h & ((1 << 30) - 1); }
    __host__ __device__ static bool header_appended(int h) { return (h >> 30) & 1; }
};
#ifdef __CUDACC__
__device__ __forceinline__ StepLen step_length(const DecodeParams& p, int b) {
    StepLen s;
    const int raw = p.seq_lens ? p.seq_lens[b] : p.uniform_len;
    const long long planned = static_cast<long long>(p.num_splits) * p.chunk;
    const int limit = static_cast<int>(planned < p.cache_cap ? planned : p.cache_cap);
    s.overflow = raw < 0 || raw + (p.append ? 1 : 0) > limit;
    s.len = raw < 0 ? 0 : (raw > limit ? limit : raw);
    s.append = p.append && !s.overflow;
    s.total = s.len + (s.append ? 1 : 0);
    return s;
}
#endif
int decode_tile_keys();
int launch_decode_generic_split(cudaStream_t s, const DecodeParams& p);   // decode_generic.cu
int launch_decode(cudaStream_t s, const DecodeParams& p);
// decode_gqa_mma.cu: split kernel with warp-MMA products (instantiated for Hq / Hkv of 4 and 8); same workspace layout
template <typename T, int NREP> int launch_decode_gqa_mma_split(cudaStream_t s, const DecodeParams& p);
int launch_lse_combine(cudaStream_t s, const float* partials, int R, long long rows, int D,
                       int dtype, void* out, float* lse);

// ---- flash_bwd_f32.cu ----
struct AttnBwdParams {
    int B, H, N, D, causal;
    float scale;
    const float *d_out, *q, *k, *v, *out, *lse;   // contiguous [B,H,N,D]; lse [B,H,N]
    float *dq, *dk, *dv;
    float* delta;                                 // workspace [B,H,N]
};
int launch_attention_bwd_f32(cudaStream_t s, const AttnBwdParams& p);

// ---- decode_exchange.cu ----
size_t exchange_buffer_bytes(int world, long long rows, int D);
int launch_exchange_combine(cudaStream_t s, ExchangeParams p);

// ---- linear_sm100.cu ----
struct LinearParams {
    const void* x;  long long ldx;   // [M, K] bf16
    const void* w;  long long ldw;   // [N, K] bf16
    void* out;      long long ldo;   // [M, N] bf16 / fp32, or [M, N/2] bf16 for the SwiGLU epilogue
    int M, N, K;
    int epilogue;                    // vb200_epilogue
    int splits;                      // K slices per cluster of the skinny kernel, 0 = choose
    int* status;                     // device status word (bounded waits)
    const float* bias;               // [N] fp32 added to every output row before the epilogue's own step, or null
    // optional, with the += epilogue: RMSNorm of the finished rows, out_norm[m,:] = out[m,:] * inv_rms * norm_w
    const float* norm_w;             // [N]
    void* norm_out;                  // [M, N] bf16, row stride norm_ld; null = no fused norm
    long long norm_ld;
    float norm_eps;
    // Deferred RMSNorm (decode path: no norm kernel at all).  rmsnorm(h) * g @ W^T = inv_rms(h) * ((h * g) @ W^T):
    //   producer side, with the += epilogue: also scaled_copy[m,n] = bf16(out[m,n] * copy_scale[n])  (h * g of the NEXT norm)
    //   consumer side: the rows of the output are multiplied by inv_rms of the fp32 rows `rms_rows` (the residual
    //   stream h, [M, rms_dim], contiguous), computed inside the skinny kernel while the weights stream, or taken
    //   from the precomputed array `row_scale` [M] (tiled kernel)
    void* scaled_copy;               // [M, N] bf16, row stride N, or null
    const float* copy_scale;         // [N]
    const float* rms_rows;           // [M, rms_dim] fp32 (row stride rms_ld) or null
    long long rms_ld;
    int rms_dim;
    float rms_eps;
    const float* row_scale;          // [M] or null
};
int launch_linear(cudaStream_t s, const LinearParams& p);
// inv_rms[m] = 1 / sqrt(mean(h[m,:]^2) + eps)
int launch_row_inv_rms(cudaStream_t s, const float* h, long long ld, float* inv_rms, int M, int dim, float eps);

// ---- block_ops.cu ----
int launch_interleave_rows(cudaStream_t s, const void* a, const void* b, void* out, long long rows, long long cols);
int launch_rms_norm(cudaStream_t s, const float* x, const float* weight, void* out_bf16, int M, int dim, float eps);
int launch_silu_mul(cudaStream_t s, const void* gate, const void* up, void* out, long long n);
int launch_linear_f32(cudaStream_t s, const float* x, long long ldx, const float* w, long long ldw, const float* bias, float* out,
                      long long ldo, int M, int N, int K);
// norm_w / norm_out (nullable): also out_norm[m,:] = rmsnorm(out[m,:]) * norm_w as bf16
int launch_embedding(cudaStream_t s, const void* ids, int ids64, const void* table, float* out, int M, int dim,
                     int vocab, int* status, const float* norm_w = nullptr, void* norm_out = nullptr, float norm_eps = 0.f,
                     int scaled_copy_only = 0);   // 1: norm_out = bf16(out * norm_w) without the 1/rms factor (deferred norm)
int launch_greedy_step(cudaStream_t s, const vb200_greedy_args& a);

}  // namespace vb200
