// Split-KV decode for every shape the two tuned kernels do not take: fp32 caches (the reference's own cache
// format, src/nn/transformer.cpp:40-41), head_dim other than 128 (any multiple of 8 up to 128), any number of
// query heads per KV head, cache rows with a stride.  Same contract, grid (split, kv_head, batch), workspace layout
// and combine kernel as decode_splitkv.cu: RoPE of q and of the new k (src/nn/functional.cpp:424-494), append of the
// new row (KVCache::update, src/nn/transformer.cpp:56-93), attention of the one query row of every head of the group
// over keys [k_begin, k_end) of the split with each K / V row fetched once per KV head, partial (O/l, m, l) per head.
// CUDA cores, fp32 math; written for coverage and correctness (parity 1e-4 in fp32), not tuned: the serving
// formats (16-bit, head_dim 128) never come here.
#include "kernels.h"

namespace vb200 {

namespace {

constexpr int kWarps = 4;
constexpr int kHeadChunk = 8;          // query heads of a group handled per pass over the split's keys
constexpr int kMaxLaneDims = 4;        // lane l owns dims l, l + 32, l + 64, l + 96 (< D <= 128)
constexpr float kLog2eG = 1.4426950408889634f;
constexpr float kLn2G = 0.6931471805599453f;

template <typename T> struct Scalar;
template <> struct Scalar<float> {
    __device__ static float load(const float* p) { return *p; }
    __device__ static void store(float* p, float x) { *p = x; }
};
template <> struct Scalar<__nv_bfloat16> {
    __device__ static float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    __device__ static void store(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }
};
template <> struct Scalar<__half> {
    __device__ static float load(const __half* p) { return __half2float(*p); }
    __device__ static void store(__half* p, float x) { *p = __float2half_rn(x); }
};

template <typename T>
__global__ void __launch_bounds__(kWarps * 32) decode_generic_kernel(DecodeParams p) {
    const int D = p.D, nrep = p.Hq / p.Hkv;
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    extern __shared__ float smem_f[];
    float* q_sm = smem_f;                              // [nrep][D] rotated queries, pre-scaled by scale * log2(e)
    float* newk = q_sm + nrep * D;                     // [D] rotated new key (fp32)
    float* newv = newk + D;                            // [D] new value
    float* mrg = newv + D;                             // [kWarps][kHeadChunk][D + 2] per-warp partials of a head chunk

    const StepLen sl = step_length(p, b);
    const int len = sl.len, total = sl.total;
    const int k_begin = split * p.chunk;
    if (split == 0 && kvh == 0 && tid == 0) {
        reinterpret_cast<int*>(p.workspace)[b] = sl.header();
        if (sl.overflow) atomicCAS(p.status, 0, (2 << 24) | (b & 0xFFFFFF));
    }
    if (k_begin >= total) return;
    const int k_end = min(len, k_begin + p.chunk);
    const bool owns_new = sl.append && (len / p.chunk == split);

    // ---- prologue: q (all heads of the group) and the new k through shared memory, rotated there ----
    const float pos = __int2float_rn(p.q_positions ? p.q_positions[b] : static_cast<int>(p.pos_offset) + len);
    const float qscale = p.scale * kLog2eG;
    const T* qg = static_cast<const T*>(p.q.ptr) + b * p.q.sb + static_cast<long long>(kvh) * nrep * p.q.sh;
    for (int i = tid; i < nrep * (D / 2); i += kWarps * 32) {
        const int h = i / (D / 2), pr = i % (D / 2);
        float x0 = Scalar<T>::load(qg + h * p.q.sh + 2 * pr), x1 = Scalar<T>::load(qg + h * p.q.sh + 2 * pr + 1);
        if (p.rope) {
            float sn, cs;
            sincosf(pos * p.inv_freq.v[pr], &sn, &cs);
            const float t1 = __fmul_rn(x0, cs), t2 = __fmul_rn(x1, sn), t3 = __fmul_rn(x0, sn), t4 = __fmul_rn(x1, cs);
            x0 = __fsub_rn(t1, t2); x1 = __fadd_rn(t3, t4);
        }
        q_sm[h * D + 2 * pr] = x0 * qscale;
        q_sm[h * D + 2 * pr + 1] = x1 * qscale;
    }
    T* kc = static_cast<T*>(p.k_cache.ptr) + b * p.k_cache.sb + kvh * p.k_cache.sh;
    T* vc = static_cast<T*>(p.v_cache.ptr) + b * p.v_cache.sb + kvh * p.v_cache.sh;
    if (owns_new) {
        const T* kn = static_cast<const T*>(p.k_new.ptr) + b * p.k_new.sb + kvh * p.k_new.sh;
        const T* vn = static_cast<const T*>(p.v_new.ptr) + b * p.v_new.sb + kvh * p.v_new.sh;
        for (int pr = tid; pr < D / 2; pr += kWarps * 32) {
            float x0 = Scalar<T>::load(kn + 2 * pr), x1 = Scalar<T>::load(kn + 2 * pr + 1);
            if (p.rope) {
                float sn, cs;
                sincosf(pos * p.inv_freq.v[pr], &sn, &cs);
                const float t1 = __fmul_rn(x0, cs), t2 = __fmul_rn(x1, sn), t3 = __fmul_rn(x0, sn), t4 = __fmul_rn(x1, cs);
                x0 = __fsub_rn(t1, t2); x1 = __fadd_rn(t3, t4);
            }
            newk[2 * pr] = x0; newk[2 * pr + 1] = x1;               // scored at full precision in this step
            const float v0 = Scalar<T>::load(vn + 2 * pr), v1 = Scalar<T>::load(vn + 2 * pr + 1);
            newv[2 * pr] = v0; newv[2 * pr + 1] = v1;
            // the cache row (owns_new implies len < cache_cap)
            Scalar<T>::store(kc + static_cast<long long>(len) * p.k_cache.ss + 2 * pr, x0);
            Scalar<T>::store(kc + static_cast<long long>(len) * p.k_cache.ss + 2 * pr + 1, x1);
            Scalar<T>::store(vc + static_cast<long long>(len) * p.v_cache.ss + 2 * pr, v0);
            Scalar<T>::store(vc + static_cast<long long>(len) * p.v_cache.ss + 2 * pr + 1, v1);
        }
    }
    __syncthreads();

    float* wsp = p.workspace + p.ws_header;
    for (int h0 = 0; h0 < nrep; h0 += kHeadChunk) {
        const int nh = min(kHeadChunk, nrep - h0);
        float qv[kHeadChunk][kMaxLaneDims], acc[kHeadChunk][kMaxLaneDims], m[kHeadChunk], l[kHeadChunk];
#pragma unroll
        for (int h = 0; h < kHeadChunk; ++h) {
            m[h] = -INFINITY; l[h] = 0.f;
#pragma unroll
            for (int i = 0; i < kMaxLaneDims; ++i) {
                const int d = lane + 32 * i;
                qv[h][i] = (h < nh && d < D) ? q_sm[(h0 + h) * D + d] : 0.f;
                acc[h][i] = 0.f;
            }
        }
        // one key at a time per warp; the new token (a row in shared memory) is the last "key" of the split that owns it
        const int n_keys = (k_end - k_begin) + (owns_new ? 1 : 0);
        for (int kk = warp; kk < n_keys; kk += kWarps) {
            const bool is_new = kk >= k_end - k_begin;
            float kvv[kMaxLaneDims], vvv[kMaxLaneDims];
#pragma unroll
            for (int i = 0; i < kMaxLaneDims; ++i) {
                const int d = lane + 32 * i;
                if (d < D) {
                    if (is_new) { kvv[i] = newk[d]; vvv[i] = newv[d]; }
                    else {
                        kvv[i] = Scalar<T>::load(kc + static_cast<long long>(k_begin + kk) * p.k_cache.ss + d);
                        vvv[i] = Scalar<T>::load(vc + static_cast<long long>(k_begin + kk) * p.v_cache.ss + d);
                    }
                } else { kvv[i] = 0.f; vvv[i] = 0.f; }
            }
#pragma unroll
            for (int h = 0; h < kHeadChunk; ++h) {
                if (h >= nh) break;
                float s = 0.f;
#pragma unroll
                for (int i = 0; i < kMaxLaneDims; ++i) s = fmaf(qv[h][i], kvv[i], s);
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);       // score in log2 units
                const float m_new = fmaxf(m[h], s);
                const float alpha = (m[h] == -INFINITY) ? 0.f : exp2f(m[h] - m_new);
                const float pj = exp2f(s - m_new);
                l[h] = l[h] * alpha + pj;
                m[h] = m_new;
#pragma unroll
                for (int i = 0; i < kMaxLaneDims; ++i) acc[h][i] = fmaf(pj, vvv[i], acc[h][i] * alpha);
            }
        }
        // ---- merge the warps, write this split's partial rows of the head chunk ----
        __syncthreads();                                   // (mrg is reused between head chunks)
#pragma unroll
        for (int h = 0; h < kHeadChunk; ++h) {
            if (h >= nh) break;
            float* row = mrg + (warp * kHeadChunk + h) * (D + 2);
#pragma unroll
            for (int i = 0; i < kMaxLaneDims; ++i) {
                const int d = lane + 32 * i;
                if (d < D) row[d] = acc[h][i];
            }
            if (lane == 0) { row[D] = m[h]; row[D + 1] = l[h]; }
        }
        __syncthreads();
        for (int i = tid; i < nh * D; i += kWarps * 32) {
            const int h = i / D, d = i % D;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) M = fmaxf(M, mrg[(w * kHeadChunk + h) * (D + 2) + D]);
            float L = 0.f, a = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                const float* row = mrg + (w * kHeadChunk + h) * (D + 2);
                const float wgt = (row[D] == -INFINITY) ? 0.f : exp2f(row[D] - M);
                L += row[D + 1] * wgt;
                a += row[d] * wgt;
            }
            float* out = wsp + ((static_cast<long long>(b) * p.Hkv + kvh) * p.num_splits + split) * nrep * (D + 2) + (h0 + h) * (D + 2);
            out[d] = a / L;
            if (d == 0) { out[D] = M * kLn2G; out[D + 1] = L; }
        }
    }
}

}  // namespace

size_t decode_generic_smem(const DecodeParams& p) {
    const int nrep = p.Hq / p.Hkv;
    return sizeof(float) * (static_cast<size_t>(nrep) * p.D + 2 * p.D + static_cast<size_t>(kWarps) * kHeadChunk * (p.D + 2));
}

// Launches the split kernel; the caller follows with the common combine kernel.
int launch_decode_generic_split(cudaStream_t s, const DecodeParams& p) {
    if (p.D % 8 != 0 || p.D > 128) return set_detail(VB200_ERR_UNSUPPORTED, "decode: head_dim must be a multiple of 8 and <= 128");
    const size_t smem = decode_generic_smem(p);
    if (smem > 48 * 1024) return set_detail(VB200_ERR_UNSUPPORTED, "decode: too many query heads per KV head for the generic kernel");
    dim3 grid(p.num_splits, p.Hkv, p.B);
    switch (p.dtype) {
        case VB200_F32: decode_generic_kernel<float><<<grid, kWarps * 32, smem, s>>>(p); break;
        case VB200_BF16: decode_generic_kernel<__nv_bfloat16><<<grid, kWarps * 32, smem, s>>>(p); break;
        case VB200_F16: decode_generic_kernel<__half><<<grid, kWarps * 32, smem, s>>>(p); break;
        default: return VB200_ERR_UNSUPPORTED;
    }
    note_launch();
    VB200_CUDA_TRY(cudaPeekAtLastError());
    return VB200_OK;
}

}  // namespace vb200
