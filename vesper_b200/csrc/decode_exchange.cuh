// The exchange protocol of sequence-sharded decode, shared by the stand-alone kernel (decode_exchange.cu) and
// the tail of the split-KV decode kernel (decode_gqa_mma.cu) that runs it without a second launch.
//
// Exchange buffer of one rank (zeroed once by the caller, then owned by these kernels):
//   [0, 256)                     counter[kXMaxCtas]     call number each exchanging CTA used last
//   [1024, 1280)                 ticket[kXMaxCtas]      CTAs of a (batch, kv_head) that have delivered their split (fused tail)
//   [4096, 4096 + 2*W*64*4)      flag[parity][src][cta] call number src's CTA `cta` published
//   [kXSlotBase, ...)            slot[parity][src][rows*(D+2)] fp32
// Two parities: a rank can be at most one call ahead of a peer (it needs the peer's flag of call s to finish
// call s), so call s+2 never overwrites a slot a peer is still reading for call s.
#pragma once

#include "kernels.h"

namespace vb200 {

constexpr int kXMaxCtas = 64;
constexpr size_t kXTicketBase = 1024;
constexpr size_t kXFlagBase = 4096;
constexpr size_t kXSlotBase = 4096 + 2 * VB200_EXCHANGE_MAX_WORLD * kXMaxCtas * 4;      // 69632, a multiple of 128

#ifdef __CUDACC__
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// One exchanging CTA (index c, owner of rows [r0, r1) of the partial records): stores its rows of this rank's
// records `src` (row r0 first; global or shared memory) into slot[parity][rank] of every rank with plain peer
// stores, publishes its flag there, waits -- bounded by p.timeout_cycles -- for the flags of all ranks in its own
// buffer and merges:  m* = max m_r,  l* = sum l_r e^{m_r - m*},  O* = sum O_r l_r e^{m_r - m*} / l*
// (the online-softmax recurrence of src/ops/flash_attention.cpp:309-345 across shards).  `sync` synchronises the
// kNT participating threads (tid in [0, kNT)); s_step / s_ok are shared-memory scratch words.  On expiry the
// output is left untouched and the status word names the rank that never arrived.
// `scratch` (shared memory, 16-byte aligned, `scratch_floats` long; may be null): when all ranks' rows of this CTA fit,
// they are fetched there in one round of asynchronous copies and merged from shared memory instead of in two dependent
// rounds of L2 loads per row (needs r0 * (D + 2) * 4 and rows * (D + 2) * 4 to be multiples of 16 bytes).
template <typename T, int kNT, typename Sync>
__device__ __forceinline__ void exchange_rows(const ExchangeParams& p, int c, long long r0, long long r1, const float* src,
                                              int tid, uint32_t* s_step, int* s_ok, Sync sync,
                                              float* scratch = nullptr, int scratch_floats = 0) {
    const int W = p.world, D = p.D, rec = p.D + 2;
    char* self = static_cast<char*>(p.peers[p.rank]);
    uint32_t* counter = reinterpret_cast<uint32_t*>(self) + c;
    if (tid == 0) { *s_step = p.step ? p.step : *counter + 1; *s_ok = 1; }
    sync();
    const uint32_t step = *s_step;
    const int parity = static_cast<int>(step & 1);
    const size_t slot_floats = static_cast<size_t>(p.rows) * rec;

    // ---- push ----
    const long long n2 = (r1 - r0) * rec / 2;                       // (D + 2) is even: whole float2s
    const float2* src2 = reinterpret_cast<const float2*>(src);
    for (int k = 0; k < W; ++k) {
        const int peer = (p.rank + 1 + k) % W;                      // start with the neighbour: ranks do not all hit rank 0 first
        float2* dst = reinterpret_cast<float2*>(static_cast<char*>(p.peers[peer]) + kXSlotBase) +
                      (static_cast<size_t>(parity) * W + p.rank) * slot_floats / 2 + r0 * rec / 2;
        for (long long i = tid; i < n2; i += kNT) dst[i] = src2[i];
    }
    // all threads' peer stores, then the CTA barrier, then the release store of the flag by a few threads: the release
    // is cumulative over what the barrier ordered before it, so no thread needs a system-wide fence of its own
    // (measured at ~5 us per call when all 128 threads issued one)
    sync();
    if (tid < W) {
        uint32_t* flag = reinterpret_cast<uint32_t*>(static_cast<char*>(p.peers[tid]) + kXFlagBase) +
                         (static_cast<size_t>(parity) * VB200_EXCHANGE_MAX_WORLD + p.rank) * kXMaxCtas + c;
        st_release_sys(flag, step);
    }

    // ---- wait (bounded) for every rank's rows of this CTA ----
    if (tid < W) {
        const uint32_t* flag = reinterpret_cast<const uint32_t*>(self + kXFlagBase) +
                               (static_cast<size_t>(parity) * VB200_EXCHANGE_MAX_WORLD + tid) * kXMaxCtas + c;
        const long long t0 = clock64();
        bool ok = false;
        for (unsigned it = 0;; ++it) {
            if (static_cast<int>(ld_acquire_sys(flag) - step) >= 0) { ok = true; break; }
            if ((it & 63) == 63 && clock64() - t0 > p.timeout_cycles) break;
        }
        if (!ok) {
            *s_ok = 0;
            atomicCAS(p.status, 0, (3 << 24) | (tid << 8) | 0x71);      // which rank never arrived
        }
    }
    sync();
    if (tid == 0) *counter = step;
    if (!*s_ok) return;

    // ---- merge: one warp per row (rows of the CTA dealt round-robin), a lane owns dim pairs lane, lane + 32, ... ----
    // Two dependent rounds of L2 loads per row (the maxima, then everything else), all ranks' loads of a round in flight
    // together: the merge is latency-bound, so the rounds are what counts.
    const float* slots = reinterpret_cast<const float*>(self + kXSlotBase) + static_cast<size_t>(parity) * W * slot_floats;
    const int warp = tid >> 5, lane = tid & 31;
    const int nrows = static_cast<int>(r1 - r0);
    const int row_floats = nrows * rec;
    if (scratch != nullptr && static_cast<long long>(W) * row_floats <= scratch_floats && (row_floats % 4) == 0 &&
        ((r0 * rec) % 4) == 0 && (slot_floats % 4) == 0) {
        const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(scratch));
        const int per_rank = row_floats / 4;                            // 16-byte pieces per rank
        for (int i = tid; i < W * per_rank; i += kNT) {
            const int r = i / per_rank, j = i % per_rank;
            const float4* g = reinterpret_cast<const float4*>(slots + r * slot_floats + r0 * rec) + j;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + i * 16), "l"(g) : "memory");
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        sync();
        for (int rr = warp; rr < nrows; rr += kNT / 32) {
            const float* base = scratch + rr * rec;                     // rank r's copy of the row: base + r * row_floats
            float M = -INFINITY;
            for (int r = 0; r < W; ++r) M = fmaxf(M, base[r * row_floats + D]);
            float L = 0.f;
            for (int d2 = lane; d2 < D / 2; d2 += 32) {
                float2 acc = make_float2(0.f, 0.f);
                float l = 0.f;
                for (int r = 0; r < W; ++r) {
                    const float2 ml = *reinterpret_cast<const float2*>(base + r * row_floats + D);
                    const float2 o = reinterpret_cast<const float2*>(base + r * row_floats)[d2];
                    const float w = (ml.x == -INFINITY) ? 0.f : expf(ml.x - M) * ml.y;
                    l += w;
                    acc.x += w * o.x; acc.y += w * o.y;
                }
                L = l;
                reinterpret_cast<uint32_t*>(static_cast<T*>(p.out) + (r0 + rr) * D)[d2] = Elem<T>::pack2(acc.x / l, acc.y / l);
            }
            if (p.lse && lane == 0) p.lse[r0 + rr] = M + logf(L);
        }
        return;
    }
    for (long long row = r0 + warp; row < r1; row += kNT / 32) {
        const float* base = slots + row * rec;
        float M = -INFINITY;
        for (int r = 0; r < W; ++r) M = fmaxf(M, __ldcg(base + r * slot_floats + D));
        float L = 0.f;
        for (int d2 = lane; d2 < D / 2; d2 += 32) {
            float2 acc = make_float2(0.f, 0.f);
            float l = 0.f;
            for (int r = 0; r < W; ++r) {
                const float2 ml = __ldcg(reinterpret_cast<const float2*>(base + r * slot_floats + D));
                const float2 o = __ldcg(reinterpret_cast<const float2*>(base + r * slot_floats) + d2);
                const float w = (ml.x == -INFINITY) ? 0.f : expf(ml.x - M) * ml.y;
                l += w;
                acc.x += w * o.x; acc.y += w * o.y;
            }
            L = l;
            reinterpret_cast<uint32_t*>(static_cast<T*>(p.out) + row * D)[d2] = Elem<T>::pack2(acc.x / l, acc.y / l);
        }
        if (p.lse && lane == 0) p.lse[row] = M + logf(L);        // lane 0 ran d2 = 0, so L holds the row's l*
    }
}
#endif  // __CUDACC__

}  // namespace vb200
