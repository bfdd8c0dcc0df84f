// Flash-attention backward in fp32 (the dtype of the reference's training path): dQ, dK, dV from the
// saved output and log-sum-exp, recomputing P tile by tile -- flash_attention_backward_cpu_dispatch,
// src/ops/flash_attention.cpp:366-482, without dropout:
//   Di = rowsum(dO * O);  P = exp(scale Q K^T - LSE);  dV = P^T dO;  dS = P * (dO V^T - Di);
//   dQ = scale dS K;  dK = scale dS^T Q.
// Three launches, all deterministic (no atomics): the row sums; one CTA per 32-key tile walking the query
// tiles that see it (dK, dV in registers); one CTA per 32-query tile walking its key tiles (dQ in registers).
// CUDA cores, 32 x 32 tiles, rows padded by one float in shared memory so both access patterns of the
// tile products are bank-conflict free.  Training is outside the inference hot path: this kernel is
// built for correctness and a sane speed, not tuned.
#include "kernels.h"

namespace vb200 {
namespace {

constexpr int kT = 32;             // tile edge
constexpr int kBwdThreads = 256;

__global__ void bwd_delta_kernel(const float* __restrict__ d_out, const float* __restrict__ out, float* __restrict__ delta,
                                 long long rows, int D) {
    const long long row = blockIdx.x * static_cast<long long>(blockDim.x / 32) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    float s = 0.f;
    for (int d = lane; d < D; d += 32) s += d_out[row * D + d] * out[row * D + d];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
    if (lane == 0) delta[row] = s;
}

// rows [r0, r0 + 32) of a [N, D] matrix into a padded tile; rows past N become zeros
__device__ __forceinline__ void load_tile(float* dst, const float* __restrict__ src, int r0, int N, int D, int ld) {
    for (int idx = threadIdx.x; idx < kT * D; idx += kBwdThreads) {
        const int r = idx / D, d = idx - r * D;
        dst[r * ld + d] = (r0 + r < N) ? src[static_cast<long long>(r0 + r) * D + d] : 0.f;
    }
}

// p and ds of the (query tile i0, key tile j0) pair: thread t owns query i0 + t/8 and keys j0 + 4 (t%8) .. + 3
__device__ __forceinline__ void tile_p_ds(const float* Qs, const float* Ks, const float* Vs, const float* dOs, const float* Ls,
                                          const float* Dis, float* Ps, float* dSs, int i0, int j0, int N, int D, int ld,
                                          float scale, int causal) {
    const int i = threadIdx.x >> 3, jb = (threadIdx.x & 7) * 4;
    float s[4] = {0.f, 0.f, 0.f, 0.f}, dp[4] = {0.f, 0.f, 0.f, 0.f};
    for (int d = 0; d < D; ++d) {
        const float qv = Qs[i * ld + d], gv = dOs[i * ld + d];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            s[c] = fmaf(qv, Ks[(jb + c) * ld + d], s[c]);
            dp[c] = fmaf(gv, Vs[(jb + c) * ld + d], dp[c]);
        }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const int gi = i0 + i, gj = j0 + jb + c;
        const bool visible = gi < N && gj < N && (!causal || gj <= gi);
        const float p = visible ? expf(s[c] * scale - Ls[i]) : 0.f;
        Ps[i * (kT + 1) + jb + c] = p;
        dSs[i * (kT + 1) + jb + c] = p * (dp[c] - Dis[i]);
    }
}

template <int DMAX>
__global__ void __launch_bounds__(kBwdThreads)
bwd_dkdv_kernel(AttnBwdParams p) {
    extern __shared__ float sm[];
    const int D = p.D, ld = D + 1, N = p.N;
    float* Ks = sm; float* Vs = Ks + kT * ld; float* Qs = Vs + kT * ld; float* dOs = Qs + kT * ld;
    float* Ps = dOs + kT * ld; float* dSs = Ps + kT * (kT + 1); float* Ls = dSs + kT * (kT + 1); float* Dis = Ls + kT;
    const int j0 = blockIdx.x * kT;
    const long long bh = static_cast<long long>(blockIdx.z) * p.H + blockIdx.y;
    const float* q = p.q + bh * N * D; const float* k = p.k + bh * N * D; const float* v = p.v + bh * N * D;
    const float* d_out = p.d_out + bh * N * D; const float* lse = p.lse + bh * N; const float* delta = p.delta + bh * N;
    load_tile(Ks, k, j0, N, D, ld);
    load_tile(Vs, v, j0, N, D, ld);
    // thread t accumulates key j0 + t/8, dims (t%8) + 8 m
    const int j = threadIdx.x >> 3, dl = threadIdx.x & 7;
    float dk[DMAX / 8], dv[DMAX / 8];
#pragma unroll
    for (int m = 0; m < DMAX / 8; ++m) { dk[m] = 0.f; dv[m] = 0.f; }
    const int i_first = p.causal ? j0 : 0;                      // query tiles before the key tile see none of it
    for (int i0 = i_first; i0 < N; i0 += kT) {
        __syncthreads();
        load_tile(Qs, q, i0, N, D, ld);
        load_tile(dOs, d_out, i0, N, D, ld);
        if (threadIdx.x < kT) {
            const int gi = i0 + threadIdx.x;
            Ls[threadIdx.x] = gi < N ? lse[gi] : 0.f;
            Dis[threadIdx.x] = gi < N ? delta[gi] : 0.f;
        }
        __syncthreads();
        tile_p_ds(Qs, Ks, Vs, dOs, Ls, Dis, Ps, dSs, i0, j0, N, D, ld, p.scale, p.causal);
        __syncthreads();
        for (int i = 0; i < kT; ++i) {
            const float pv = Ps[i * (kT + 1) + j], ds = dSs[i * (kT + 1) + j];
#pragma unroll
            for (int m = 0; m < DMAX / 8; ++m) {
                const int d = dl + 8 * m;
                if (d < D) {
                    dv[m] = fmaf(pv, dOs[i * ld + d], dv[m]);
                    dk[m] = fmaf(ds, Qs[i * ld + d], dk[m]);
                }
            }
        }
    }
    if (j0 + j < N) {
#pragma unroll
        for (int m = 0; m < DMAX / 8; ++m) {
            const int d = dl + 8 * m;
            if (d < D) {
                p.dk[(bh * N + j0 + j) * D + d] = dk[m] * p.scale;
                p.dv[(bh * N + j0 + j) * D + d] = dv[m];
            }
        }
    }
}

template <int DMAX>
__global__ void __launch_bounds__(kBwdThreads)
bwd_dq_kernel(AttnBwdParams p) {
    extern __shared__ float sm[];
    const int D = p.D, ld = D + 1, N = p.N;
    float* Ks = sm; float* Vs = Ks + kT * ld; float* Qs = Vs + kT * ld; float* dOs = Qs + kT * ld;
    float* Ps = dOs + kT * ld; float* dSs = Ps + kT * (kT + 1); float* Ls = dSs + kT * (kT + 1); float* Dis = Ls + kT;
    const int i0 = blockIdx.x * kT;
    const long long bh = static_cast<long long>(blockIdx.z) * p.H + blockIdx.y;
    const float* q = p.q + bh * N * D; const float* k = p.k + bh * N * D; const float* v = p.v + bh * N * D;
    const float* d_out = p.d_out + bh * N * D; const float* lse = p.lse + bh * N; const float* delta = p.delta + bh * N;
    load_tile(Qs, q, i0, N, D, ld);
    load_tile(dOs, d_out, i0, N, D, ld);
    if (threadIdx.x < kT) {
        const int gi = i0 + threadIdx.x;
        Ls[threadIdx.x] = gi < N ? lse[gi] : 0.f;
        Dis[threadIdx.x] = gi < N ? delta[gi] : 0.f;
    }
    const int i = threadIdx.x >> 3, dl = threadIdx.x & 7;
    float dq[DMAX / 8];
#pragma unroll
    for (int m = 0; m < DMAX / 8; ++m) dq[m] = 0.f;
    const int j_end = p.causal ? min(N, i0 + kT) : N;           // key tiles past the query tile are invisible
    for (int j0 = 0; j0 < j_end; j0 += kT) {
        __syncthreads();
        load_tile(Ks, k, j0, N, D, ld);
        load_tile(Vs, v, j0, N, D, ld);
        __syncthreads();
        tile_p_ds(Qs, Ks, Vs, dOs, Ls, Dis, Ps, dSs, i0, j0, N, D, ld, p.scale, p.causal);
        __syncthreads();
        for (int jj = 0; jj < kT; ++jj) {
            const float ds = dSs[i * (kT + 1) + jj];
#pragma unroll
            for (int m = 0; m < DMAX / 8; ++m) {
                const int d = dl + 8 * m;
                if (d < D) dq[m] = fmaf(ds, Ks[jj * ld + d], dq[m]);
            }
        }
    }
    if (i0 + i < N) {
#pragma unroll
        for (int m = 0; m < DMAX / 8; ++m) {
            const int d = dl + 8 * m;
            if (d < D) p.dq[(bh * N + i0 + i) * D + d] = dq[m] * p.scale;
        }
    }
}

size_t bwd_smem_bytes(int D) { return sizeof(float) * (4 * kT * (D + 1) + 2 * kT * (kT + 1) + 2 * kT); }

template <int DMAX>
int launch_bwd_t(cudaStream_t s, const AttnBwdParams& p) {
    const size_t smem = bwd_smem_bytes(p.D);
    static thread_local bool configured[64] = {};      // per device ordinal: the attribute belongs to the device's context
    int dev = 0;
    VB200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return set_detail(VB200_ERR_NO_DEVICE, "device ordinal out of range");
    if (!configured[dev]) {
        VB200_CUDA_TRY(cudaFuncSetAttribute(bwd_dkdv_kernel<DMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bwd_smem_bytes(DMAX))));
        VB200_CUDA_TRY(cudaFuncSetAttribute(bwd_dq_kernel<DMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bwd_smem_bytes(DMAX))));
        configured[dev] = true;
    }
    const long long rows = static_cast<long long>(p.B) * p.H * p.N;
    bwd_delta_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, s>>>(p.d_out, p.out, p.delta, rows, p.D);
    dim3 grid(static_cast<unsigned>((p.N + kT - 1) / kT), static_cast<unsigned>(p.H), static_cast<unsigned>(p.B));
    bwd_dkdv_kernel<DMAX><<<grid, kBwdThreads, smem, s>>>(p);
    bwd_dq_kernel<DMAX><<<grid, kBwdThreads, smem, s>>>(p);
    note_launch(3);
    VB200_CUDA_TRY(cudaPeekAtLastError());
    return VB200_OK;
}

}  // namespace

int launch_attention_bwd_f32(cudaStream_t s, const AttnBwdParams& p) {
    if (p.D <= 64) return launch_bwd_t<64>(s, p);
    if (p.D <= 128) return launch_bwd_t<128>(s, p);
    return set_detail(VB200_ERR_UNSUPPORTED, "attention backward supports head_dim <= 128");
}

}  // namespace vb200
