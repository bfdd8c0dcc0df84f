// Sequence-sharded decode: exchange of the per-rank partial results (O/l, m, l) and their
// log-sum-exp merge in ONE kernel over NVLink peer memory -- each rank stores its partial rows
// straight into every peer's receive slots (plain peer stores, no TMA, no multicast), raises a
// per-CTA flag there, waits (bounded) for the flags of all ranks in its own buffer and merges.
// It stands in for "all-gather, then vb200_lse_combine": one launch, no collective library call, no
// host wait between the two.  The merge algebra is the online-softmax recurrence of
// src/ops/flash_attention.cpp:309-345 applied across shards.
//
// Exchange buffer of one rank (zeroed once by the caller, then owned by this kernel):
//   [0, 256)                     counter[kMaxCtas]      step number each CTA used last
//   [4096, 4096 + 2*W*64*4)      flag[parity][src][cta] step number src's CTA `cta` published
//   [kSlotBase, ...)             slot[parity][src][rows*(D+2)] fp32
// Two parities: a rank can be at most one step ahead of a peer (it needs the peer's flag of step s
// to finish step s), so step s+2 never overwrites a slot a peer is still reading for step s.
#include "kernels.h"

namespace vb200 {
namespace {

constexpr int kMaxCtas = 64;
constexpr int kRowsPerCta = 4;
constexpr int kThreads = 256;
constexpr size_t kFlagBase = 4096;
constexpr size_t kSlotBase = 4096 + 2 * VB200_EXCHANGE_MAX_WORLD * kMaxCtas * 4;      // 69632, a multiple of 128

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
exchange_combine_kernel(ExchangeParams p) {
    const int c = blockIdx.x, tid = threadIdx.x;
    const int W = p.world, D = p.D, rec = p.D + 2;
    const long long r0 = static_cast<long long>(c) * p.rows_per_cta;
    const long long r1 = min(p.rows, r0 + p.rows_per_cta);
    char* self = static_cast<char*>(p.peers[p.rank]);
    uint32_t* counter = reinterpret_cast<uint32_t*>(self) + c;
    __shared__ uint32_t s_step;
    __shared__ int s_ok;
    if (tid == 0) { s_step = p.step ? p.step : *counter + 1; s_ok = 1; }
    __syncthreads();
    const uint32_t step = s_step;
    const int parity = static_cast<int>(step & 1);
    const size_t slot_floats = static_cast<size_t>(p.rows) * rec;

    // ---- push this CTA's rows of the local partial into slot[parity][rank] of every rank ----
    const long long n2 = (r1 - r0) * rec / 2;                       // (D + 2) is even: whole float2s
    const float2* src = reinterpret_cast<const float2*>(p.partial + r0 * rec);
    for (int k = 0; k < W; ++k) {
        const int peer = (p.rank + 1 + k) % W;                      // start with the neighbour: ranks do not all hit rank 0 first
        float2* dst = reinterpret_cast<float2*>(static_cast<char*>(p.peers[peer]) + kSlotBase) +
                      (static_cast<size_t>(parity) * W + p.rank) * slot_floats / 2 + r0 * rec / 2;
        for (long long i = tid; i < n2; i += kThreads) dst[i] = src[i];
    }
    __threadfence_system();
    __syncthreads();
    if (tid < W) {
        uint32_t* flag = reinterpret_cast<uint32_t*>(static_cast<char*>(p.peers[tid]) + kFlagBase) +
                         (static_cast<size_t>(parity) * VB200_EXCHANGE_MAX_WORLD + p.rank) * kMaxCtas + c;
        st_release_sys(flag, step);
    }

    // ---- wait (bounded) for every rank's rows of this CTA ----
    if (tid < W) {
        const uint32_t* flag = reinterpret_cast<const uint32_t*>(self + kFlagBase) +
                               (static_cast<size_t>(parity) * VB200_EXCHANGE_MAX_WORLD + tid) * kMaxCtas + c;
        const long long t0 = clock64();
        bool ok = false;
        for (unsigned it = 0;; ++it) {
            if (static_cast<int>(ld_acquire_sys(flag) - step) >= 0) { ok = true; break; }
            if ((it & 63) == 63 && clock64() - t0 > p.timeout_cycles) break;
        }
        if (!ok) {
            s_ok = 0;
            atomicCAS(p.status, 0, (3 << 24) | (tid << 8) | 0x71);      // which rank never arrived
        }
    }
    __syncthreads();
    if (tid == 0) *counter = step;
    if (!s_ok) return;

    // ---- merge: m* = max m_r, l* = sum l_r e^{m_r - m*}, O* = sum O_r l_r e^{m_r - m*} / l* ----
    const float* slots = reinterpret_cast<const float*>(self + kSlotBase) + static_cast<size_t>(parity) * W * slot_floats;
    for (long long row = r0; row < r1; ++row) {
        const float* base = slots + row * rec;
        float M = -INFINITY;
        for (int r = 0; r < W; ++r) M = fmaxf(M, __ldcg(base + r * slot_floats + D));
        float L = 0.f;
        for (int d = tid; d < D; d += kThreads) {
            float acc = 0.f, l = 0.f;
            for (int r = 0; r < W; ++r) {
                const float mr = __ldcg(base + r * slot_floats + D);
                const float w = (mr == -INFINITY) ? 0.f : expf(mr - M) * __ldcg(base + r * slot_floats + D + 1);
                l += w;
                acc += w * __ldcg(base + r * slot_floats + d);
            }
            L = l;
            static_cast<T*>(p.out)[row * D + d] = Elem<T>::from_f(acc / l);
        }
        if (p.lse && tid == 0) {                                 // thread 0 ran d = 0, so L holds the row's l*
            p.lse[row] = M + logf(L);
        }
    }
}

}  // namespace

size_t exchange_buffer_bytes(int world, long long rows, int D) {
    return kSlotBase + static_cast<size_t>(2) * world * rows * (D + 2) * sizeof(float);
}

int launch_exchange_combine(cudaStream_t s, ExchangeParams p) {
    long long ctas = (p.rows + kRowsPerCta - 1) / kRowsPerCta;
    p.rows_per_cta = kRowsPerCta;
    if (ctas > kMaxCtas) {
        ctas = kMaxCtas;
        p.rows_per_cta = (p.rows + kMaxCtas - 1) / kMaxCtas;
        ctas = (p.rows + p.rows_per_cta - 1) / p.rows_per_cta;
    }
    if (p.timeout_cycles <= 0) p.timeout_cycles = kWaitCycles;
    switch (p.dtype) {
        case VB200_BF16: exchange_combine_kernel<__nv_bfloat16><<<static_cast<unsigned>(ctas), kThreads, 0, s>>>(p); break;
        case VB200_F16: exchange_combine_kernel<__half><<<static_cast<unsigned>(ctas), kThreads, 0, s>>>(p); break;
        default: return set_detail(VB200_ERR_UNSUPPORTED, "exchange_combine: dtype must be bf16 or fp16");
    }
    note_launch();
    VB200_CUDA_TRY(cudaPeekAtLastError());
    return VB200_OK;
}

}  // namespace vb200
