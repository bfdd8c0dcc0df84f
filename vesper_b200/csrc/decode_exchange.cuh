// The exchange protocol of sequence-sharded decode, shared by the stand-alone kernel (decode_exchange.cu) and
// the tail of the split-KV decode kernel (decode_gqa_mma.cu) that runs it without a second launch.
//
// Exchange buffer of one rank (zeroed once by the caller, then owned by these kernels):
//   [0, 256)                     counter[kXMaxCtas]     call number each exchanging CTA used last
//   [1024, 1280)                 ticket[kXMaxCtas]      CTAs of a (batch, kv_head) that have delivered their split (fused tail)
//   [kXSlotBase, ...)            slot[parity][src][rows*(D+2)] of 8-byte words {fp32 value, call number}
//   (the bytes between 1280 and kXSlotBase are not used)
// Every value travels with the call number in ONE 8-byte store (single-copy atomic, also across NVLink): the receiver
// takes a word when its number matches, so there is no separate flag, no release fence on the sender and no acquire
// round trip on the receiver.  Two parities: a rank can be at most one call ahead of a peer (it needs the peer's words
// of call s to finish call s), so call s+2 never overwrites a slot a peer is still reading for call s; a slot's stale
// words carry the number s-2 (or 0), never s.  Calls are numbered per exchanging CTA, and the two users of this
// protocol cut the rows into CTAs differently: a buffer belongs to ONE of them (the numbers of the in-kernel form carry
// bit 31, so a buffer shared by mistake ends in the bounded wait's error, not in a wrong result).
#pragma once

#include "kernels.h"

namespace vb200 {

constexpr int kXMaxCtas = 64;
constexpr size_t kXTicketBase = 1024;
constexpr size_t kXSlotBase = 4096 + 2 * VB200_EXCHANGE_MAX_WORLD * kXMaxCtas * 4;      // 69632, a multiple of 128

#ifdef __CUDACC__
__device__ __forceinline__ void st_word(uint2* p, float v, uint32_t step) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(step) : "memory");
}
__device__ __forceinline__ uint2 ld_word(const uint2* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

// One exchanging CTA (index c, owner of rows [r0, r1) of the partial records): stores its rows of this rank's
// records `src` (row r0 first; global or shared memory) into slot[parity][rank] of every rank with plain peer
// stores, waits -- bounded by p.timeout_cycles -- until the same rows of every rank have landed in its own buffer and
// merges:  m* = max m_r,  l* = sum l_r e^{m_r - m*},  O* = sum O_r l_r e^{m_r - m*} / l*
// (the online-softmax recurrence of src/ops/flash_attention.cpp:309-345 across shards).  `sync` synchronises the
// kNT participating threads (tid in [0, kNT)); s_step / s_ok are shared-memory scratch words.  On expiry the
// output is left untouched and the status word names a rank whose words never arrived.
// `scratch` (shared memory, 16-byte aligned, `scratch_floats` long; may be null): when all ranks' words of this CTA
// fit, they are fetched there in one round of asynchronous copies and checked and merged from shared memory.
template <typename T, int kNT, typename Sync>
__device__ __forceinline__ void exchange_rows(const ExchangeParams& p, int c, long long r0, long long r1, const float* src,
                                              int tid, uint32_t* s_step, int* s_ok, Sync sync,
                                              float* scratch = nullptr, int scratch_floats = 0, uint32_t tag_bit = 0) {
    const int W = p.world, D = p.D, rec = p.D + 2;
    char* self = static_cast<char*>(p.peers[p.rank]);
    uint32_t* counter = reinterpret_cast<uint32_t*>(self) + c;
    if (tid == 0) { *s_step = p.step ? p.step : *counter + 1; *s_ok = 1; }
    sync();
    const uint32_t call = *s_step;
    const int parity = static_cast<int>(call & 1);
    const uint32_t step = (call & 0x7FFFFFFFu) | tag_bit;           // the number the words carry
    const size_t slot_words = static_cast<size_t>(p.rows) * rec;
    const int nrows = static_cast<int>(r1 - r0);
    const int n = nrows * rec;                                      // words of this CTA per rank

    // ---- push ----
    for (int k = 0; k < W; ++k) {
        const int peer = (p.rank + 1 + k) % W;                      // start with the neighbour: ranks do not all hit rank 0 first
        uint2* dst = reinterpret_cast<uint2*>(static_cast<char*>(p.peers[peer]) + kXSlotBase) +
                     (static_cast<size_t>(parity) * W + p.rank) * slot_words + r0 * rec;
        for (int i = tid; i < n; i += kNT) st_word(dst + i, src[i], step);
    }

    // ---- receive (bounded) ----
    const uint2* mine = reinterpret_cast<const uint2*>(self + kXSlotBase) + static_cast<size_t>(parity) * W * slot_words + r0 * rec;
    const long long t0 = clock64();
    const bool staged = scratch != nullptr && static_cast<long long>(W) * n * 2 <= scratch_floats && (n % 2) == 0 &&
                        ((r0 * rec) % 2) == 0 && (slot_words % 2) == 0;
    const uint2* words = nullptr;                                   // where the merge reads rank r's words: words + r * stride
    size_t stride = 0;
    if (staged) {
        // a hint first (the last word of every rank's block), then everything in one round of 16-byte copies; every
        // word's number is checked in shared memory and the round repeated in the rare case that a block was still landing
        if (tid < W) {
            const uint2* last = mine + tid * slot_words + (n - 1);
            for (unsigned it = 0; ld_word(last).y != step; ++it)
                if ((it & 63) == 63 && clock64() - t0 > p.timeout_cycles) {
                    *s_ok = 0;
                    atomicCAS(p.status, 0, (3 << 24) | (tid << 8) | 0x71);      // which rank never arrived
                    break;
                }
        }
        sync();
        uint2* sw = reinterpret_cast<uint2*>(scratch);
        const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(scratch));
        const int per_rank = n / 2;                                 // 16-byte pieces per rank
        while (*s_ok) {
            for (int i = tid; i < W * per_rank; i += kNT) {
                const int r = i / per_rank, j = i % per_rank;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + i * 16), "l"(mine + r * slot_words + 2 * j) : "memory");
            }
            asm volatile("cp.async.wait_all;" ::: "memory");
            if (tid == 0) *s_step = 0;                              // (the call number is in a register by now) 1: a word was missing
            sync();
            int late = -1;
            for (int i = tid; i < W * n; i += kNT)
                if (sw[i].y != step) late = i / n;
            if (late >= 0) *s_step = 1;
            sync();
            if (*s_step == 0) break;
            if (late >= 0 && clock64() - t0 > p.timeout_cycles) {
                *s_ok = 0;
                atomicCAS(p.status, 0, (3 << 24) | (late << 8) | 0x72);
            }
            sync();
        }
        words = sw;
        stride = static_cast<size_t>(n);
    } else {
        // every thread waits for its share of the words (all in flight at once), then the merge reads them again
        for (int i0 = tid; i0 < W * n && *s_ok; i0 += kNT * 16) {
            bool all = false;
            for (unsigned it = 0; !all; ++it) {
                all = true;
#pragma unroll
                for (int u = 0; u < 16; ++u) {
                    const int i = i0 + u * kNT;
                    if (i < W * n && ld_word(mine + (i / n) * slot_words + (i % n)).y != step) all = false;
                }
                if (!all && (it & 15) == 15 && clock64() - t0 > p.timeout_cycles) {
                    *s_ok = 0;
                    atomicCAS(p.status, 0, (3 << 24) | (((i0 / n) & 0xFF) << 8) | 0x73);
                    break;
                }
            }
        }
        words = mine;
        stride = slot_words;
    }
    sync();
    if (tid == 0) *counter = call;
    if (!*s_ok) return;

    // ---- merge: one warp per row (rows of the CTA dealt round-robin), a lane owns dim pairs lane, lane + 32, ... ----
    const int warp = tid >> 5, lane = tid & 31;
    // (words in this rank's buffer are read past the L1, which peer stores do not keep coherent)
    auto value = [staged](const uint2* w) { return __uint_as_float(staged ? w->x : __ldcg(reinterpret_cast<const unsigned int*>(w))); };
    for (int rr = warp; rr < nrows; rr += kNT / 32) {
        const uint2* base = words + rr * rec;                       // rank r's copy of the row: base + r * stride
        float M = -INFINITY;
        for (int r = 0; r < W; ++r) M = fmaxf(M, value(base + r * stride + D));
        float L = 0.f;
        for (int d2 = lane; d2 < D / 2; d2 += 32) {
            float2 acc = make_float2(0.f, 0.f);
            float l = 0.f;
            for (int r = 0; r < W; ++r) {
                const float mr = value(base + r * stride + D), lr = value(base + r * stride + D + 1);
                const float o0 = value(base + r * stride + 2 * d2), o1 = value(base + r * stride + 2 * d2 + 1);
                const float w = (mr == -INFINITY) ? 0.f : expf(mr - M) * lr;
                l += w;
                acc.x += w * o0; acc.y += w * o1;
            }
            L = l;
            reinterpret_cast<uint32_t*>(static_cast<T*>(p.out) + (r0 + rr) * D)[d2] = Elem<T>::pack2(acc.x / l, acc.y / l);
        }
        if (p.lse && lane == 0) p.lse[r0 + rr] = M + logf(L);        // lane 0 ran d2 = 0, so L holds the row's l*
    }
}
#endif  // __CUDACC__

}  // namespace vb200
