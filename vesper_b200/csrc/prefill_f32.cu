// fp32 attention forward on CUDA cores (fp32 in, fp32 math, fp32 out).
//
// This is the dtype the reference's flash op runs in
// (flash_attention_cuda_dispatch, src/ops/cuda/flash_attention.cu:518-544), so
// it keeps full fp32 accuracy instead of down-converting to a tensor-core
// type.  Same math as flash_attention_cpu_dispatch
// (src/ops/flash_attention.cpp:218-364): s = scale * q.k, causal j <= i,
// online softmax, O = acc / l, LSE = m + ln l.
//
// Tiling: 64 query rows x 64 keys per step, 256 threads as a 16x16 grid; each
// thread owns a 4x4 block of the score tile and a 4 x (D/16) block of O.
#include "kernels.h"

namespace vb200 {

namespace {

constexpr int kBM = 64, kBN = 64, kThreads = 256;

__device__ __forceinline__ float rowgroup_max(float v) {
#pragma unroll
    for (int o = 8; o >= 1; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}
__device__ __forceinline__ float rowgroup_sum(float v) {
#pragma unroll
    for (int o = 8; o >= 1; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

__global__ void __launch_bounds__(kThreads) prefill_f32_kernel(PrefillParams p) {
    extern __shared__ __align__(16) float smem[];
    const int D = p.D;
    const int pitch = D + 4;
    float* Qs = smem;
    float* Ks = Qs + kBM * pitch;
    float* Vs = Ks + kBN * pitch;
    float* Ps = Vs + kBN * pitch;          // [kBM][kBN + 4]
    constexpr int ppitch = kBN + 4;

    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int qt = gridDim.x - 1 - blockIdx.x;   // longest (last) causal tiles first
    const int hq = blockIdx.y, b = blockIdx.z;
    const int hkv = hq / (p.Hq / p.Hkv);
    const int q0 = qt * kBM;
    const int vecs = D >> 2;

    const float* qg = static_cast<const float*>(p.q.ptr) + b * p.q.sb + hq * p.q.sh;
    const float* kg = static_cast<const float*>(p.k.ptr) + b * p.k.sb + hkv * p.k.sh;
    const float* vg = static_cast<const float*>(p.v.ptr) + b * p.v.sb + hkv * p.v.sh;

    // Q tile (rotated on the way in when a table is given)
    for (int i = tid; i < kBM * vecs; i += kThreads) {
        int r = i / vecs, c = i - r * vecs;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (q0 + r < p.T) {
            x = *reinterpret_cast<const float4*>(qg + static_cast<long long>(q0 + r) * p.q.ss + c * 4);
            if (p.q_rope_table) {
                const float2* tp = p.q_rope_table + static_cast<long long>(q0 + r) * (D / 2) + c * 2;
                float2 cs0 = tp[0], cs1 = tp[1];
                float t1 = __fmul_rn(x.x, cs0.x), t2 = __fmul_rn(x.y, cs0.y), t3 = __fmul_rn(x.x, cs0.y), t4 = __fmul_rn(x.y, cs0.x);
                x.x = __fsub_rn(t1, t2); x.y = __fadd_rn(t3, t4);
                t1 = __fmul_rn(x.z, cs1.x); t2 = __fmul_rn(x.w, cs1.y); t3 = __fmul_rn(x.z, cs1.y); t4 = __fmul_rn(x.w, cs1.x);
                x.z = __fsub_rn(t1, t2); x.w = __fadd_rn(t3, t4);
            }
        }
        *reinterpret_cast<float4*>(Qs + r * pitch + c * 4) = x;
    }

    float m_i[4], l_i[4], acc[4][2][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        m_i[i] = -INFINITY; l_i[i] = 0.f;
#pragma unroll
        for (int g = 0; g < 2; ++g)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][g][e] = 0.f;
    }

    int kv_end = p.Skv;
    if (p.causal) kv_end = min(p.Skv, p.start_pos + min(q0 + kBM, p.T));

    for (int k0 = 0; k0 < kv_end; k0 += kBN) {
        __syncthreads();   // previous tile fully consumed (also orders the Q stores)
        for (int i = tid; i < kBN * vecs; i += kThreads) {
            int r = i / vecs, c = i - r * vecs;
            float4 kx = make_float4(0.f, 0.f, 0.f, 0.f), vx = kx;
            if (k0 + r < kv_end) {
                kx = *reinterpret_cast<const float4*>(kg + static_cast<long long>(k0 + r) * p.k.ss + c * 4);
                vx = *reinterpret_cast<const float4*>(vg + static_cast<long long>(k0 + r) * p.v.ss + c * 4);
            }
            *reinterpret_cast<float4*>(Ks + r * pitch + c * 4) = kx;
            *reinterpret_cast<float4*>(Vs + r * pitch + c * 4) = vx;
        }
        __syncthreads();

        float s[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
        for (int d = 0; d < D; d += 4) {
            float4 qv[4], kv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) qv[i] = *reinterpret_cast<const float4*>(Qs + (ty + 16 * i) * pitch + d);
#pragma unroll
            for (int j = 0; j < 4; ++j) kv[j] = *reinterpret_cast<const float4*>(Ks + (tx + 16 * j) * pitch + d);
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    s[i][j] = fmaf(qv[i].x, kv[j].x, s[i][j]);
                    s[i][j] = fmaf(qv[i].y, kv[j].y, s[i][j]);
                    s[i][j] = fmaf(qv[i].z, kv[j].z, s[i][j]);
                    s[i][j] = fmaf(qv[i].w, kv[j].w, s[i][j]);
                }
        }

        float alpha[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int row = q0 + ty + 16 * i;
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int kc = k0 + tx + 16 * j;
                bool ok = kc < p.Skv && (!p.causal || kc <= p.start_pos + row);
                s[i][j] = ok ? s[i][j] * p.scale : -INFINITY;
                mx = fmaxf(mx, s[i][j]);
            }
            mx = rowgroup_max(mx);
            float m_new = fmaxf(m_i[i], mx);
            float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            alpha[i] = expf(m_i[i] - m_use);       // exp(-inf) = 0 on the first tile
            float ls = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float pv = expf(s[i][j] - m_use);
                ls += pv;
                Ps[(ty + 16 * i) * ppitch + tx + 16 * j] = pv;
            }
            l_i[i] = l_i[i] * alpha[i] + ls;       // per-thread partial; reduced at the end
            m_i[i] = m_new;
        }
        __syncthreads();

#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int g = 0; g < 2; ++g)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[i][g][e] *= alpha[i];

        for (int kk = 0; kk < kBN; kk += 4) {
            float4 pr[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) pr[i] = *reinterpret_cast<const float4*>(Ps + (ty + 16 * i) * ppitch + kk);
#pragma unroll
            for (int g = 0; g < 2; ++g) {
                int dc = g * 64 + tx * 4;
                if (dc < D) {
                    float4 v0 = *reinterpret_cast<const float4*>(Vs + (kk + 0) * pitch + dc);
                    float4 v1 = *reinterpret_cast<const float4*>(Vs + (kk + 1) * pitch + dc);
                    float4 v2 = *reinterpret_cast<const float4*>(Vs + (kk + 2) * pitch + dc);
                    float4 v3 = *reinterpret_cast<const float4*>(Vs + (kk + 3) * pitch + dc);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        acc[i][g][0] = fmaf(pr[i].x, v0.x, acc[i][g][0]); acc[i][g][1] = fmaf(pr[i].x, v0.y, acc[i][g][1]);
                        acc[i][g][2] = fmaf(pr[i].x, v0.z, acc[i][g][2]); acc[i][g][3] = fmaf(pr[i].x, v0.w, acc[i][g][3]);
                        acc[i][g][0] = fmaf(pr[i].y, v1.x, acc[i][g][0]); acc[i][g][1] = fmaf(pr[i].y, v1.y, acc[i][g][1]);
                        acc[i][g][2] = fmaf(pr[i].y, v1.z, acc[i][g][2]); acc[i][g][3] = fmaf(pr[i].y, v1.w, acc[i][g][3]);
                        acc[i][g][0] = fmaf(pr[i].z, v2.x, acc[i][g][0]); acc[i][g][1] = fmaf(pr[i].z, v2.y, acc[i][g][1]);
                        acc[i][g][2] = fmaf(pr[i].z, v2.z, acc[i][g][2]); acc[i][g][3] = fmaf(pr[i].z, v2.w, acc[i][g][3]);
                        acc[i][g][0] = fmaf(pr[i].w, v3.x, acc[i][g][0]); acc[i][g][1] = fmaf(pr[i].w, v3.y, acc[i][g][1]);
                        acc[i][g][2] = fmaf(pr[i].w, v3.z, acc[i][g][2]); acc[i][g][3] = fmaf(pr[i].w, v3.w, acc[i][g][3]);
                    }
                }
            }
        }
    }

    float* og = static_cast<float*>(p.o.ptr) + b * p.o.sb + hq * p.o.sh;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int row = q0 + ty + 16 * i;
        float l = rowgroup_sum(l_i[i]);
        if (row >= p.T) continue;
        float inv = 1.0f / l;
#pragma unroll
        for (int g = 0; g < 2; ++g) {
            int dc = g * 64 + tx * 4;
            if (dc < D)
                *reinterpret_cast<float4*>(og + static_cast<long long>(row) * p.o.ss + dc) =
                    make_float4(acc[i][g][0] * inv, acc[i][g][1] * inv, acc[i][g][2] * inv, acc[i][g][3] * inv);
        }
        if (p.lse && tx == 0)
            p.lse[(static_cast<long long>(b) * p.Hq + hq) * p.T + row] = m_i[i] + logf(l);
    }
}

}  // namespace

int launch_prefill_f32(cudaStream_t s, const PrefillParams& p) {
    if (p.D % 4 != 0 || p.D > 128 || p.D < 4) return set_detail(VB200_ERR_UNSUPPORTED, "fp32 attention needs head_dim % 4 == 0 and <= 128");
    size_t smem = sizeof(float) * (static_cast<size_t>(kBM + 2 * kBN) * (p.D + 4) + kBM * (kBN + 4));
    static thread_local bool configured[64] = {};      // per device ordinal: the attribute belongs to the device's context
    int dev = 0;
    VB200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return set_detail(VB200_ERR_NO_DEVICE, "device ordinal out of range");
    if (!configured[dev]) {
        VB200_CUDA_TRY(cudaFuncSetAttribute(prefill_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 120 * 1024));
        configured[dev] = true;
    }
    dim3 grid((p.T + kBM - 1) / kBM, p.Hq, p.B);
    prefill_f32_kernel<<<grid, kThreads, smem, s>>>(p);
    note_launch();
    note_prefill_kernel("prefill_f32_kernel");
    VB200_CUDA_TRY(cudaPeekAtLastError());
    return VB200_OK;
}

}  // namespace vb200
