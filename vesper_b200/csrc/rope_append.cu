// RoPE table, fused K-rotation + KV-cache append, and the two small surface
// kernels (in-place RoPE with a caller table, repeat_kv).
//
// Reference behaviour reproduced here:
//   angle table  a[m,i] = float(start_pos+m) * inv_freq[i]   src/nn/functional.cpp:430-435
//   rotation     x'[2i]   = x[2i] cos a - x[2i+1] sin a
//                x'[2i+1] = x[2i] sin a + x[2i+1] cos a      src/nn/functional.cpp:468-478
//   cache write  rows [start_pos, start_pos+T) of [B,H,cap,D] src/nn/transformer.cpp:56-75
//   K is cached after rotation, V unrotated                  src/nn/gqa_attention.cpp:124-137
#include "kernels.h"

namespace vb200 {

__global__ void rope_table_kernel(float2* __restrict__ table, int T, int half, int start_pos, InvFreq f) {
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= T * half) return;
    int t = idx / half, i = idx - t * half;
    // int -> float, then one fp32 multiply: the reference's `pos * freq`.
    float ang = __int2float_rn(start_pos + t) * f.v[i];
    float s, c;
    sincosf(ang, &s, &c);   // accurate path: arguments reach 1e5 at long context
    table[idx] = make_float2(c, s);
}

int launch_rope_table(cudaStream_t s, float2* table, int T, int D, int start_pos, const InvFreq& f) {
    int n = T * (D / 2);
    if (n <= 0) return VB200_OK;
    rope_table_kernel<<<(n + 255) / 256, 256, 0, s>>>(table, T, D / 2, start_pos, f);
    note_launch();
    VB200_CUDA_TRY(cudaPeekAtLastError());
    return VB200_OK;
}

// One thread moves 8 consecutive elements of one row (16 bytes for bf16/fp16,
// 32 bytes for fp32) of K (rotated) and of V (copied).
template <typename T>
struct Vec8 {
    static_assert(sizeof(T) == 2, "16-bit types");
    uint4 raw;
    __device__ void load(const T* p) { raw = *reinterpret_cast<const uint4*>(p); }
    __device__ void store(T* p) const { *reinterpret_cast<uint4*>(p) = raw; }
    __device__ void get(float (&f)[8]) const {
        const uint32_t* u = &raw.x;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 t = Elem<T>::unpack2(u[i]);
            f[2 * i] = t.x; f[2 * i + 1] = t.y;
        }
    }
    __device__ void set(const float (&f)[8]) {
        uint32_t* u = &raw.x;
#pragma unroll
        for (int i = 0; i < 4; ++i) u[i] = Elem<T>::pack2(f[2 * i], f[2 * i + 1]);
    }
};
template <>
struct Vec8<float> {
    float4 a, b;
    __device__ void load(const float* p) {
        a = *reinterpret_cast<const float4*>(p); b = *reinterpret_cast<const float4*>(p + 4);
    }
    __device__ void store(float* p) const {
        *reinterpret_cast<float4*>(p) = a; *reinterpret_cast<float4*>(p + 4) = b;
    }
    __device__ void get(float (&f)[8]) const {
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
    __device__ void set(const float (&f)[8]) {
        a = make_float4(f[0], f[1], f[2], f[3]); b = make_float4(f[4], f[5], f[6], f[7]);
    }
};

// Rotation with separately rounded products, as the reference's mul/mul/sub
// and mul/mul/add sequence does (no fused multiply-add).
__device__ __forceinline__ void rotate_pair(float& xr, float& xi, float2 cs) {
    float t1 = __fmul_rn(xr, cs.x), t2 = __fmul_rn(xi, cs.y);
    float t3 = __fmul_rn(xr, cs.y), t4 = __fmul_rn(xi, cs.x);
    xr = __fsub_rn(t1, t2);
    xi = __fadd_rn(t3, t4);
}

template <typename T>
__global__ void kv_append_kernel(int B, int H, int Tn, int D, View4 k, View4 v, View4 kd, View4 vd,
                                 int dst_row0, const float2* __restrict__ table, InvFreq f, int compute_angles) {
    int vecs = D / 8;
    long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    long long total = static_cast<long long>(B) * H * Tn * vecs;
    if (idx >= total) return;
    int c = static_cast<int>(idx % vecs);
    long long r = idx / vecs;
    int t = static_cast<int>(r % Tn); r /= Tn;
    int h = static_cast<int>(r % H);
    int b = static_cast<int>(r / H);

    const T* kp = static_cast<const T*>(k.ptr) + b * k.sb + h * k.sh + t * k.ss + c * 8;
    T* kdp = static_cast<T*>(kd.ptr) + b * kd.sb + h * kd.sh + static_cast<long long>(dst_row0 + t) * kd.ss + c * 8;
    Vec8<T> x;
    x.load(kp);
    if (table != nullptr) {
        float e[8];
        x.get(e);
        const float2* tp = table + static_cast<long long>(t) * (D / 2) + c * 4;
#pragma unroll
        for (int i = 0; i < 4; ++i) rotate_pair(e[2 * i], e[2 * i + 1], __ldg(tp + i));
        x.set(e);
    } else if (compute_angles) {
        float e[8];
        x.get(e);
        float pos = __int2float_rn(dst_row0 + t);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 cs;
            sincosf(pos * f.v[c * 4 + i], &cs.y, &cs.x);
            rotate_pair(e[2 * i], e[2 * i + 1], cs);
        }
        x.set(e);
    }
    x.store(kdp);
    if (v.ptr != nullptr) {
        const T* vp = static_cast<const T*>(v.ptr) + b * v.sb + h * v.sh + t * v.ss + c * 8;
        T* vdp = static_cast<T*>(vd.ptr) + b * vd.sb + h * vd.sh + static_cast<long long>(dst_row0 + t) * vd.ss + c * 8;
        Vec8<T> y;
        y.load(vp);
        y.store(vdp);
    }
}

// The angle table and the K rotation + cache append of a prompt pass in ONE launch.  A CTA owns kRopeRows consecutive
// positions: it computes their (cos, sin) once (accurate sincosf of the reference's fp32 angle), keeps them in shared
// memory, writes them to the table the attention kernel rotates Q with (only the CTAs of the first (batch, head) chunk
// do), and moves those rows of K (rotated) and V (copied) for its chunk of (batch, head) pairs -- one table kernel, one
// launch gap and one trip of the table through L2 less than table-then-append.
constexpr int kRopeRows = 8;

template <typename T>
__global__ void __launch_bounds__(256) rope_append_fused_kernel(int B, int H, int Tn, int D, View4 k, View4 v, View4 kd, View4 vd, int dst_row0,
                                                                float2* __restrict__ table, InvFreq f, int bh_per_cta) {
    __shared__ float2 cs[kRopeRows][kMaxHalfDim];
    const int half = D / 2, vecs = D / 8;
    const int t0 = blockIdx.x * kRopeRows;
    const int rows = min(kRopeRows, Tn - t0);
    for (int i = threadIdx.x; i < rows * half; i += blockDim.x) {
        const int r = i / half, pr = i - r * half;
        float sn, c;
        sincosf(__int2float_rn(dst_row0 + t0 + r) * f.v[pr], &sn, &c);       // int -> float, one fp32 multiply: the reference's pos * freq
        cs[r][pr] = make_float2(c, sn);
        if (blockIdx.y == 0 && table != nullptr) table[static_cast<long long>(t0 + r) * half + pr] = make_float2(c, sn);
    }
    __syncthreads();
    const int bh0 = blockIdx.y * bh_per_cta;
    const int nbh = min(bh_per_cta, B * H - bh0);
    const int per_bh = rows * vecs;
    for (int i = threadIdx.x; i < nbh * per_bh; i += blockDim.x) {
        const int bh = bh0 + i / per_bh, rem = i % per_bh;
        const int r = rem / vecs, c = rem - r * vecs;
        const int b = bh / H, h = bh - b * H, t = t0 + r;
        const T* kp = static_cast<const T*>(k.ptr) + b * k.sb + h * k.sh + static_cast<long long>(t) * k.ss + c * 8;
        T* kdp = static_cast<T*>(kd.ptr) + b * kd.sb + h * kd.sh + static_cast<long long>(dst_row0 + t) * kd.ss + c * 8;
        Vec8<T> x;
        x.load(kp);
        float e[8];
        x.get(e);
#pragma unroll
        for (int j = 0; j < 4; ++j) rotate_pair(e[2 * j], e[2 * j + 1], cs[r][c * 4 + j]);
        x.set(e);
        x.store(kdp);
        if (v.ptr != nullptr) {
            const T* vp = static_cast<const T*>(v.ptr) + b * v.sb + h * v.sh + static_cast<long long>(t) * v.ss + c * 8;
            T* vdp = static_cast<T*>(vd.ptr) + b * vd.sb + h * vd.sh + static_cast<long long>(dst_row0 + t) * vd.ss + c * 8;
            Vec8<T> y;
            y.load(vp);
            y.store(vdp);
        }
    }
}

int launch_rope_append_fused(cudaStream_t s, int dtype, int B, int H, int T, int D, View4 k, View4 v, View4 k_dst, View4 v_dst,
                             int dst_row0, float2* table, const InvFreq& f) {
    if (T <= 0 || B * H <= 0) return VB200_OK;
    const int row_tiles = (T + kRopeRows - 1) / kRopeRows;
    // enough CTAs for about two per SM; every extra (batch, head) chunk repeats the sincosf of its rows
    int chunks = (296 + row_tiles - 1) / row_tiles;
    if (chunks > B * H) chunks = B * H;
    if (chunks < 1) chunks = 1;
    const int bh_per_cta = (B * H + chunks - 1) / chunks;
    chunks = (B * H + bh_per_cta - 1) / bh_per_cta;
    dim3 grid(static_cast<unsigned>(row_tiles), static_cast<unsigned>(chunks));
    switch (dtype) {
        case VB200_F32: rope_append_fused_kernel<float><<<grid, 256, 0, s>>>(B, H, T, D, k, v, k_dst, v_dst, dst_row0, table, f, bh_per_cta); break;
        case VB200_BF16: rope_append_fused_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(B, H, T, D, k, v, k_dst, v_dst, dst_row0, table, f, bh_per_cta); break;
        case VB200_F16: rope_append_fused_kernel<__half><<<grid, 256, 0, s>>>(B, H, T, D, k, v, k_dst, v_dst, dst_row0, table, f, bh_per_cta); break;
        default: return VB200_ERR_UNSUPPORTED;
    }
    note_launch();
    VB200_CUDA_TRY(cudaPeekAtLastError());
    return VB200_OK;
}

int launch_kv_append(cudaStream_t s, int dtype, int B, int H, int T, int D,
                     View4 k, View4 v, View4 k_dst, View4 v_dst, int dst_row0, const float2* table,
                     const InvFreq* inv_freq) {
    InvFreq f{};
    int ca = 0;
    if (inv_freq && !table) { f = *inv_freq; ca = 1; }
    long long total = static_cast<long long>(B) * H * T * (D / 8);
    if (total <= 0) return VB200_OK;
    unsigned grid = static_cast<unsigned>((total + 255) / 256);
    switch (dtype) {
        case VB200_F32:
            kv_append_kernel<float><<<grid, 256, 0, s>>>(B, H, T, D, k, v, k_dst, v_dst, dst_row0, table, f, ca); break;
        case VB200_BF16:
            kv_append_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(B, H, T, D, k, v, k_dst, v_dst, dst_row0, table, f, ca); break;
        case VB200_F16:
            kv_append_kernel<__half><<<grid, 256, 0, s>>>(B, H, T, D, k, v, k_dst, v_dst, dst_row0, table, f, ca); break;
        default: return VB200_ERR_UNSUPPORTED;
    }
    note_launch();
    VB200_CUDA_TRY(cudaPeekAtLastError());
    return VB200_OK;
}

// In-place rotation of x [batch,heads,seq,dim] fp32 by caller-built tables
// cos/sin [seq, dim/2]: the surface of apply_rope_cuda (src/nn/rope.cpp:25-28).
__global__ void apply_rope_f32_kernel(float* __restrict__ x, const float* __restrict__ cos_t,
                                      const float* __restrict__ sin_t, long long rows, int seq, int half) {
    long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= rows * half) return;
    int i = static_cast<int>(idx % half);
    long long row = idx / half;
    int s = static_cast<int>(row % seq);
    float2* p = reinterpret_cast<float2*>(x) + idx;
    float2 xv = *p;
    float2 cs = make_float2(cos_t[static_cast<long long>(s) * half + i], sin_t[static_cast<long long>(s) * half + i]);
    rotate_pair(xv.x, xv.y, cs);
    *p = xv;
}

int launch_apply_rope_f32(cudaStream_t s, float* x, const float* cos_t, const float* sin_t,
                          int batch, int heads, int seq_len, int head_dim) {
    long long rows = static_cast<long long>(batch) * heads * seq_len;
    long long n = rows * (head_dim / 2);
    if (n <= 0) return VB200_OK;
    apply_rope_f32_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(x, cos_t, sin_t, rows, seq_len, head_dim / 2);
    note_launch();
    VB200_CUDA_TRY(cudaPeekAtLastError());
    return VB200_OK;
}

// out[b, qh, s, :] = in[b, qh / n_rep, s, :] (src/ops/attention_ops.cpp:45-55),
// reading the input through its strides.
template <typename T>
__global__ void repeat_kv_kernel(View4 in, T* __restrict__ out, int B, int Hkv, int S, int D, int n_rep) {
    int vecs = D / 8;
    long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    long long total = static_cast<long long>(B) * Hkv * n_rep * S * vecs;
    if (idx >= total) return;
    int c = static_cast<int>(idx % vecs);
    long long r = idx / vecs;
    int s = static_cast<int>(r % S); r /= S;
    int qh = static_cast<int>(r % (Hkv * n_rep));
    int b = static_cast<int>(r / (Hkv * n_rep));
    const T* ip = static_cast<const T*>(in.ptr) + b * in.sb + (qh / n_rep) * in.sh + s * in.ss + c * 8;
    Vec8<T> x;
    x.load(ip);
    x.store(out + idx * 8);
}

int launch_repeat_kv(cudaStream_t s, int dtype, View4 in, void* out, int B, int Hkv, int S, int D, int n_rep) {
    long long total = static_cast<long long>(B) * Hkv * n_rep * S * (D / 8);
    if (total <= 0) return VB200_OK;
    unsigned grid = static_cast<unsigned>((total + 255) / 256);
    switch (dtype) {
        case VB200_F32: repeat_kv_kernel<float><<<grid, 256, 0, s>>>(in, static_cast<float*>(out), B, Hkv, S, D, n_rep); break;
        case VB200_BF16: repeat_kv_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(in, static_cast<__nv_bfloat16*>(out), B, Hkv, S, D, n_rep); break;
        case VB200_F16: repeat_kv_kernel<__half><<<grid, 256, 0, s>>>(in, static_cast<__half*>(out), B, Hkv, S, D, n_rep); break;
        default: return VB200_ERR_UNSUPPORTED;
    }
    note_launch();
    VB200_CUDA_TRY(cudaPeekAtLastError());
    return VB200_OK;
}

}  // namespace vb200
