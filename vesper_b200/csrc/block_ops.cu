// The memory-bound operators of a decoder block around attention: RMSNorm on the fp32 residual
// stream, SiLU-gated multiply, embedding gather, greedy argmax with the stop-token bookkeeping of
// the generation loop, and the one-off interleave of the gate / up projection weights.
// Each is one pass over its operands with 16-byte accesses; reference semantics are cited per kernel.
#include "kernels.h"

namespace vb200 {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

// out[m,:] = x[m,:] * (1 / sqrt(mean(x^2) + eps)) * w   -- rms_norm_cpu_dispatch,
// src/ops/normalization.cpp:451-481 (sum of squares, 1/sqrt(ss/n + eps), x * inv_rms * w).
// One CTA of 256 threads per row; the row stays in registers between the two passes.
constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 8;        // float4 per thread: dim <= 256 * 4 * 8 = 8192

__global__ void __launch_bounds__(kNormThreads)
rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ w, __nv_bfloat16* __restrict__ out, int dim, float eps) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const long long row = blockIdx.x;
    const float4* xr = reinterpret_cast<const float4*>(x + row * dim);
    const int nvec = dim >> 2;
    float4 v[kNormMaxVec];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
        const int idx = threadIdx.x + i * kNormThreads;
        if (idx < nvec) {
            v[i] = xr[idx];
            ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        }
    }
    __shared__ float part[kNormThreads / 32];
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < kNormThreads / 32; ++i) tot += part[i];
    const float inv_rms = 1.0f / sqrtf(tot / static_cast<float>(dim) + eps);
    const float4* wr = reinterpret_cast<const float4*>(w);
    uint2* orow = reinterpret_cast<uint2*>(out + row * dim);
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
        const int idx = threadIdx.x + i * kNormThreads;
        if (idx < nvec) {
            const float4 g = __ldg(wr + idx);
            uint2 o;
            o.x = Elem<__nv_bfloat16>::pack2(v[i].x * inv_rms * g.x, v[i].y * inv_rms * g.y);
            o.y = Elem<__nv_bfloat16>::pack2(v[i].z * inv_rms * g.z, v[i].w * inv_rms * g.w);
            orow[idx] = o;
        }
    }
}

// inv_rms[m] = 1 / sqrt(mean(x[m,:]^2) + eps): the per-row factor of a deferred RMSNorm.  One warp per row.
__global__ void row_inv_rms_kernel(const float* __restrict__ x, long long ld, float* __restrict__ inv_rms, int M, int dim, float eps) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= M) return;
    const float4* xr = reinterpret_cast<const float4*>(x + static_cast<long long>(row) * ld);
    float ss = 0.f;
    for (int c = lane; c < dim / 4; c += 32) {
        const float4 v = xr[c];
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = warp_sum(ss);
    if (lane == 0) inv_rms[row] = 1.0f / sqrtf(ss / static_cast<float>(dim) + eps);
}

// silu(g) * u with silu(g) = g * sigmoid(g) -- ops::silu_mul, src/ops/elementwise.cpp:1297-1328.
__global__ void silu_mul_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up, uint4* __restrict__ out, long long nvec) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const uint4 g = gate[i], u = up[i];
        const uint32_t gs[4] = {g.x, g.y, g.z, g.w}, us[4] = {u.x, u.y, u.z, u.w};
        uint32_t r[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 a = Elem<__nv_bfloat16>::unpack2(gs[e]), b = Elem<__nv_bfloat16>::unpack2(us[e]);
            r[e] = Elem<__nv_bfloat16>::pack2(a.x / (1.0f + __expf(-a.x)) * b.x, a.y / (1.0f + __expf(-a.y)) * b.y);
        }
        out[i] = make_uint4(r[0], r[1], r[2], r[3]);
    }
}

// out[m,:] = float(table[ids[m],:]) -- ops::embedding, src/ops/embedding.cpp:10-17; optionally also the
// RMSNorm of the row (the first block's attention norm) so a decode step starts with one launch less.
__global__ void __launch_bounds__(256)
embedding_kernel(const void* __restrict__ ids, int ids64, const __nv_bfloat16* __restrict__ table,
                 float* __restrict__ out, int dim, int vocab, int* status, const float* __restrict__ norm_w,
                 __nv_bfloat16* __restrict__ norm_out, float norm_eps, int scaled_copy_only) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const long long m = blockIdx.x;
    const long long id = ids64 ? static_cast<const long long*>(ids)[m] : static_cast<const int*>(ids)[m];
    const bool bad = id < 0 || id >= vocab;
    if (bad && threadIdx.x == 0) atomicCAS(status, 0, (2 << 24) | 0x61);
    const uint4* src = reinterpret_cast<const uint4*>(table + (bad ? 0 : id) * dim);
    float4* dst = reinterpret_cast<float4*>(out + m * dim);
    float ss = 0.f;
    for (int i = threadIdx.x; i < dim / 8; i += blockDim.x) {
        const uint4 u = bad ? make_uint4(0, 0, 0, 0) : __ldg(src + i);
        const float2 a = Elem<__nv_bfloat16>::unpack2(u.x), b = Elem<__nv_bfloat16>::unpack2(u.y);
        const float2 c = Elem<__nv_bfloat16>::unpack2(u.z), d = Elem<__nv_bfloat16>::unpack2(u.w);
        dst[2 * i] = make_float4(a.x, a.y, b.x, b.y);
        dst[2 * i + 1] = make_float4(c.x, c.y, d.x, d.y);
        ss += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y + c.x * c.x + c.y * c.y + d.x * d.x + d.y * d.y;
    }
    if (norm_out == nullptr) return;
    __shared__ float part[8];
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += part[i];
    // scaled_copy_only: the consumer GEMM applies 1/rms to its output rows (deferred norm)
    const float inv_rms = scaled_copy_only ? 1.0f : 1.0f / sqrtf(tot / static_cast<float>(dim) + norm_eps);
    uint4* nd = reinterpret_cast<uint4*>(norm_out + m * dim);
    const float4* g = reinterpret_cast<const float4*>(norm_w);
    for (int i = threadIdx.x; i < dim / 8; i += blockDim.x) {
        const uint4 u = bad ? make_uint4(0, 0, 0, 0) : __ldg(src + i);
        const float2 a = Elem<__nv_bfloat16>::unpack2(u.x), b = Elem<__nv_bfloat16>::unpack2(u.y);
        const float2 c = Elem<__nv_bfloat16>::unpack2(u.z), d = Elem<__nv_bfloat16>::unpack2(u.w);
        const float4 g0 = __ldg(g + 2 * i), g1 = __ldg(g + 2 * i + 1);
        uint4 o;
        o.x = Elem<__nv_bfloat16>::pack2(a.x * inv_rms * g0.x, a.y * inv_rms * g0.y);
        o.y = Elem<__nv_bfloat16>::pack2(b.x * inv_rms * g0.z, b.y * inv_rms * g0.w);
        o.z = Elem<__nv_bfloat16>::pack2(c.x * inv_rms * g1.x, c.y * inv_rms * g1.y);
        o.w = Elem<__nv_bfloat16>::pack2(d.x * inv_rms * g1.z, d.y * inv_rms * g1.w);
        nd[i] = o;
    }
}

// Greedy step of the generation loop (src/generation/generator.cpp:75-131): argmax with the first
// maximum winning (argmax_cpu_dispatch, src/ops/sampling_ops.cpp:18-38), the id appended to the
// history, done[b] |= id in stop_ids once min_new_tokens are out (check_stop_tokens, :263-288).
constexpr int kArgmaxThreads = 1024;
__global__ void __launch_bounds__(kArgmaxThreads)
greedy_step_kernel(const float* __restrict__ logits, long long ld, int vocab, int* __restrict__ out_ids,
                   int* __restrict__ history, long long history_ld, int step,
                   const int* __restrict__ stop_ids, int n_stop, int min_new, int* __restrict__ done,
                   const int* __restrict__ pos_dev, int pos_base) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int b = blockIdx.x;
    const float* row = logits + b * ld;
    float best = -INFINITY;
    int best_i = 0x7FFFFFFF;
    for (int i = threadIdx.x; i < vocab; i += kArgmaxThreads) {     // ascending i per thread: strict > keeps the first
        const float v = row[i];
        if (v > best || best_i == 0x7FFFFFFF) { best = v; best_i = i; }
    }
    auto better = [](float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        const int oi = __shfl_xor_sync(0xFFFFFFFFu, best_i, o);
        if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
    }
    __shared__ float sv[kArgmaxThreads / 32];
    __shared__ int si[kArgmaxThreads / 32];
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = best_i; }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = sv[threadIdx.x]; best_i = si[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
            const int oi = __shfl_xor_sync(0xFFFFFFFFu, best_i, o);
            if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
        }
        if (threadIdx.x == 0) {
            if (best_i == 0x7FFFFFFF) best_i = 0;
            out_ids[b] = best_i;
            const int col = pos_dev ? pos_dev[b] : step;
            const int generated = pos_dev ? col - pos_base + 1 : step + 1;
            if (history) history[b * history_ld + col] = best_i;
            if (done && generated >= min_new) {
                int stop = 0;
                for (int i = 0; i < n_stop; ++i) stop |= (stop_ids[i] == best_i);
                if (stop) done[b] = 1;
            }
        }
    }
}

// out row 2j = a row j, out row 2j+1 = b row j.
__global__ void interleave_rows_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b, uint4* __restrict__ out,
                                       long long rows, long long vec_per_row) {
    const long long total = rows * vec_per_row;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long r = i / vec_per_row, c = i - r * vec_per_row;
        out[(2 * r) * vec_per_row + c] = a[i];
        out[(2 * r + 1) * vec_per_row + c] = b[i];
    }
}

template <typename... KArgs, typename... Args>
int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    VB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
    note_launch();
    return VB200_OK;
}

}  // namespace

int launch_rms_norm(cudaStream_t s, const float* x, const float* weight, void* out_bf16, int M, int dim, float eps) {
    if (dim % 4 != 0 || dim > kNormThreads * 4 * kNormMaxVec)
        return set_detail(VB200_ERR_UNSUPPORTED, "rms_norm: dim must be a multiple of 4 and <= 8192");
    return launch_pdl(rms_norm_kernel, dim3(static_cast<unsigned>(M)), dim3(kNormThreads), s, x, weight,
                      static_cast<__nv_bfloat16*>(out_bf16), dim, eps);
}

int launch_row_inv_rms(cudaStream_t s, const float* h, long long ld, float* inv_rms, int M, int dim, float eps) {
    if (dim % 4 != 0 || ld % 4 != 0) return set_detail(VB200_ERR_ALIGNMENT, "row_inv_rms: dim must be a multiple of 4");
    return launch_pdl(row_inv_rms_kernel, dim3(static_cast<unsigned>((M + 7) / 8)), dim3(256), s, h, ld, inv_rms, M, dim, eps);
}

// fp32 y = x W^T + bias on CUDA cores: 64 x 64 output tiles, 16 x 16 threads with a 4 x 4 register block each, K in
// steps of 16 through shared memory.  For the reference's fp32 modules (parity at 1e-4); bf16 goes to linear_sm100.cu.
__global__ void __launch_bounds__(256) linear_f32_kernel(const float* __restrict__ x, long long ldx, const float* __restrict__ w, long long ldw,
                                                         const float* __restrict__ bias, float* __restrict__ out, long long ldo, int M, int N, int K) {
    __shared__ float xs[16][64 + 1], ws[16][64 + 1];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += 16) {
        for (int i = threadIdx.x; i < 64 * 16; i += 256) {
            const int r = i >> 4, k = i & 15;
            xs[k][r] = (m0 + r < M && k0 + k < K) ? x[static_cast<long long>(m0 + r) * ldx + k0 + k] : 0.f;
            ws[k][r] = (n0 + r < N && k0 + k < K) ? w[static_cast<long long>(n0 + r) * ldw + k0 + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = xs[k][ty * 4 + i]; b[i] = ws[k][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < M && n < N) out[static_cast<long long>(m) * ldo + n] = acc[i][j] + (bias ? bias[n] : 0.f);
        }
}

int launch_linear_f32(cudaStream_t s, const float* x, long long ldx, const float* w, long long ldw, const float* bias, float* out,
                      long long ldo, int M, int N, int K) {
    dim3 grid(static_cast<unsigned>((N + 63) / 64), static_cast<unsigned>((M + 63) / 64));
    linear_f32_kernel<<<grid, 256, 0, s>>>(x, ldx, w, ldw, bias, out, ldo, M, N, K);
    note_launch();
    VB200_CUDA_TRY(cudaPeekAtLastError());
    return VB200_OK;
}

int launch_silu_mul(cudaStream_t s, const void* gate, const void* up, void* out, long long n) {
    if (n % 8 != 0) return set_detail(VB200_ERR_ALIGNMENT, "silu_mul: element count must be a multiple of 8");
    const long long nvec = n / 8;
    long long blocks = (nvec + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (blocks < 1) blocks = 1;
    return launch_pdl(silu_mul_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), s, static_cast<const uint4*>(gate),
                      static_cast<const uint4*>(up), static_cast<uint4*>(out), nvec);
}

int launch_embedding(cudaStream_t s, const void* ids, int ids64, const void* table, float* out, int M, int dim,
                     int vocab, int* status, const float* norm_w, void* norm_out, float norm_eps, int scaled_copy_only) {
    if (dim % 8 != 0) return set_detail(VB200_ERR_ALIGNMENT, "embedding: dim must be a multiple of 8");
    return launch_pdl(embedding_kernel, dim3(static_cast<unsigned>(M)), dim3(256), s, ids, ids64,
                      static_cast<const __nv_bfloat16*>(table), out, dim, vocab, status, norm_w,
                      static_cast<__nv_bfloat16*>(norm_out), norm_eps, scaled_copy_only);
}

int launch_greedy_step(cudaStream_t s, const vb200_greedy_args& a) {
    return launch_pdl(greedy_step_kernel, dim3(static_cast<unsigned>(a.B)), dim3(kArgmaxThreads), s, a.logits,
                      static_cast<long long>(a.ld_logits), a.vocab, a.out_ids, a.history, static_cast<long long>(a.history_ld),
                      a.step, a.stop_ids, a.n_stop, a.min_new_tokens, a.done, a.pos_dev, a.pos_base);
}

int launch_interleave_rows(cudaStream_t s, const void* a, const void* b, void* out, long long rows, long long cols) {
    if (cols % 8 != 0) return set_detail(VB200_ERR_ALIGNMENT, "interleave_rows: cols must be a multiple of 8");
    const long long total = rows * (cols / 8);
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (blocks < 1) blocks = 1;
    interleave_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(static_cast<const uint4*>(a), static_cast<const uint4*>(b),
                                                                        static_cast<uint4*>(out), rows, cols / 8);
    note_launch();
    VB200_CUDA_TRY(cudaPeekAtLastError());
    return VB200_OK;
}

}  // namespace vb200
