// Split-KV decode: one new token per sequence attends to its (ragged) KV cache.
//
// Bandwidth-bound by design: every K and V row is read from HBM exactly once
// per KV head (the Hq/Hkv query heads of a group share the fetch -- the
// grouped indexing kv_head = q_head / n_rep of src/ops/attention_ops.cpp:47
// without materialising repeat_kv), streamed by 1-D bulk async copies into a
// shared-memory ring, with fp32 dot products and accumulation on CUDA cores.
// RoPE of the new q/k (src/nn/functional.cpp:424-494) and the append of the
// new k/v row (KVCache::update, src/nn/transformer.cpp:56-93) are fused in.
//
// Grid (split, kv_head, batch).  A CTA owns keys [split*chunk, (split+1)*chunk)
// of one (batch, kv_head) and emits a partial (O/l, m, l) per query head; the
// combine kernel merges the splits with the log-sum-exp algebra of
// src/ops/flash_attention.cpp:309-345.
#include "kernels.h"

namespace vb200 {

namespace {

constexpr int kTile = 64;        // keys per pipeline stage (K 16 KB + V 16 KB)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;   // log2 units: rescale O only when the max grows by > 2^8

// Sum 16 values across the 16 lanes of a group: afterwards lane g (0..15)
// holds the total of vals[g] in vals[0].  15 shuffles instead of 64.
__device__ __forceinline__ float group16_reduce_scatter(float (&vals)[16], int l16) {
#pragma unroll
    for (int off = 8, n = 16; off >= 1; off >>= 1, n >>= 1) {
        bool upper = (l16 & off) != 0;
#pragma unroll
        for (int i = 0; i < n / 2; ++i) {
            float send = upper ? vals[i] : vals[i + n / 2];
            float keep = upper ? vals[i + n / 2] : vals[i];
            vals[i] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, off);
        }
    }
    return vals[0];
}

template <typename T, int NREP>
struct WarpState {
    float2 q[NREP][4];    // rotated q * scale * log2(e), this lane's 8 dims as 4 pairs
    float2 o[NREP][4];    // unnormalised output accumulator
    float m;              // running reference max (log2 units) of this lane's head
    float l;              // partial sum of p for this lane's (head, key slot)
};

// Process `nkeys` consecutive rows of a K buffer and a V buffer in shared
// memory (row = 128 elements of T).  Rows are dealt to the participating warps
// in slices of 2*KB keys (KB = 16/NREP keys per half-warp group and batch);
// `wslot` in [0, nwslots).  The loop trip count is warp-uniform (both
// half-warps run the same iterations; rows past nkeys are masked) because the
// body uses full-warp shuffles.  All multiply-adds are packed fp32x2.
// KF32: the K rows are fp32 (used for the new token, whose rotated key is
// scored at full precision in the step that appends it).
template <typename T, int NREP, bool KF32 = false>
__device__ __forceinline__ void process_rows(WarpState<T, NREP>& st, const void* ksm_raw, const T* vsm, int nkeys,
                                             int wslot, int nwslots, int lane, float* pbuf /* [16] per group */) {
    constexpr int KB = 16 / NREP;
    const int l16 = lane & 15;
    const int my_k = l16 / NREP;
    for (int wbase = wslot * 2 * KB; wbase < nkeys; wbase += nwslots * 2 * KB) {
        const int base = wbase + (lane >> 4) * KB;
        float vals[16];
#pragma unroll
        for (int kk = 0; kk < KB; ++kk) {
            int key = base + kk;
            float2 kf[4];
            if constexpr (KF32) {
                float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
                if (key < nkeys) {
                    const float* kp = static_cast<const float*>(ksm_raw) + key * 128 + l16 * 8;
                    a0 = *reinterpret_cast<const float4*>(kp); a1 = *reinterpret_cast<const float4*>(kp + 4);
                }
                kf[0] = make_float2(a0.x, a0.y); kf[1] = make_float2(a0.z, a0.w);
                kf[2] = make_float2(a1.x, a1.y); kf[3] = make_float2(a1.z, a1.w);
            } else {
                uint4 raw = make_uint4(0, 0, 0, 0);
                if (key < nkeys) raw = *reinterpret_cast<const uint4*>(static_cast<const T*>(ksm_raw) + key * 128 + l16 * 8);
                const uint32_t* u = &raw.x;
#pragma unroll
                for (int i = 0; i < 4; ++i) kf[i] = Elem<T>::unpack2(u[i]);
            }
#pragma unroll
            for (int h = 0; h < NREP; ++h) {
                float2 a = __fmul2_rn(st.q[h][0], kf[0]);
#pragma unroll
                for (int i = 1; i < 4; ++i) a = __ffma2_rn(st.q[h][i], kf[i], a);
                vals[kk * NREP + h] = a.x + a.y;
            }
        }
        float s = group16_reduce_scatter(vals, l16);       // score (log2 units) of (key my_k, head my_h)
        if (base + my_k >= nkeys) s = -INFINITY;

        float bm = s;                                       // max over the batch's keys for my head
#pragma unroll
        for (int off = NREP; off < 16; off <<= 1) bm = fmaxf(bm, __shfl_xor_sync(0xFFFFFFFFu, bm, off));
        bool grow = bm > st.m + kRescaleThreshold;          // includes the first batch (m = -inf)
        if (__any_sync(0xFFFFFFFFu, grow)) {
            float m_new = grow ? bm : st.m;
            float alpha = (st.m == -INFINITY) ? 0.f : fast_exp2(st.m - m_new);
            st.l *= alpha;
            st.m = m_new;
#pragma unroll
            for (int h = 0; h < NREP; ++h) {
                // lane h of the group holds head h (key slot 0)
                float ah = __shfl_sync(0xFFFFFFFFu, alpha, (threadIdx.x & 16) + h);
                const float2 ah2 = make_float2(ah, ah);
#pragma unroll
                for (int i = 0; i < 4; ++i) st.o[h][i] = __fmul2_rn(st.o[h][i], ah2);
            }
        }
        float p = (s == -INFINITY) ? 0.f : fast_exp2(s - st.m);
        st.l += p;
        pbuf[l16] = p;
        __syncwarp();
#pragma unroll
        for (int kk = 0; kk < KB; ++kk) {
            int key = base + kk;
            if (key < nkeys) {
                uint4 raw = *reinterpret_cast<const uint4*>(vsm + key * 128 + l16 * 8);
                float2 vf[4];
                const uint32_t* u = &raw.x;
#pragma unroll
                for (int i = 0; i < 4; ++i) vf[i] = Elem<T>::unpack2(u[i]);
                float ph[NREP];
                if constexpr (NREP == 8) {
                    float4 x = *reinterpret_cast<const float4*>(pbuf + kk * 8), y = *reinterpret_cast<const float4*>(pbuf + kk * 8 + 4);
                    ph[0] = x.x; ph[1] = x.y; ph[2] = x.z; ph[3] = x.w; ph[4] = y.x; ph[5] = y.y; ph[6] = y.z; ph[7] = y.w;
                } else if constexpr (NREP == 4) {
                    float4 x = *reinterpret_cast<const float4*>(pbuf + kk * 4);
                    ph[0] = x.x; ph[1] = x.y; ph[2] = x.z; ph[3] = x.w;
                } else if constexpr (NREP == 2) {
                    float2 x = *reinterpret_cast<const float2*>(pbuf + kk * 2);
                    ph[0] = x.x; ph[1] = x.y;
                } else {
                    ph[0] = pbuf[kk];
                }
#pragma unroll
                for (int h = 0; h < NREP; ++h) {
                    const float2 p2 = make_float2(ph[h], ph[h]);
#pragma unroll
                    for (int i = 0; i < 4; ++i) st.o[h][i] = __ffma2_rn(p2, vf[i], st.o[h][i]);
                }
            }
        }
        __syncwarp();
    }
}

template <int CW, int kStages>
struct __align__(16) DecodeSmem {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    int abort_flag;
    int pad[3];
};

// Bytes of dynamic shared memory up to (not including) the cluster-merge receive area, a multiple of 16.
template <typename T, int NREP, int CW, int kStages>
__host__ __device__ constexpr int decode_base_smem() {
    return (kStages * 2 * kTile * 128 * static_cast<int>(sizeof(T)) + 128 * static_cast<int>(sizeof(float)) + 128 * static_cast<int>(sizeof(T)) +
            2 * CW * 16 * static_cast<int>(sizeof(float)) + static_cast<int>(sizeof(DecodeSmem<CW, kStages>)) + 15) & ~15;
}

// Dynamic shared memory layout (D = 128, 16-bit T):
//   [0, kStages * 2 * kTile * 256)   K/V ring: stage s -> K at s*32 KB, V at s*32 KB + 16 KB
//   then the new token's rotated key (fp32) and value, the per-group p buffers, DecodeSmem.
// CW = consumer warps (one more warp streams the tiles); kStages = ring depth;
// MINB = CTAs per SM the register allocation is sized for.
template <typename T, int NREP, int CW, int kStages, int MINB>
__global__ void __launch_bounds__((CW + 1) * 32, MINB) decode_splitkv_kernel(DecodeParams p) {
    constexpr int D = 128;
    constexpr int kRowBytes = D * sizeof(T);
    constexpr int kStageBytes = 2 * kTile * kRowBytes;
    constexpr int kNewBytes = D * sizeof(float) + kRowBytes;
    constexpr int kGroups = 2 * CW;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    T* ring = reinterpret_cast<T*>(smem_raw);
    float* newk = reinterpret_cast<float*>(smem_raw + kStages * kStageBytes);   // rotated new key, fp32 [128]
    T* newv = reinterpret_cast<T*>(smem_raw + kStages * kStageBytes + kNewBytes - kRowBytes);   // new value [128]
    float* pbuf_all = reinterpret_cast<float*>(smem_raw + kStages * kStageBytes + kNewBytes);   // [kGroups][16]
    DecodeSmem<CW, kStages>* sm = reinterpret_cast<DecodeSmem<CW, kStages>*>(smem_raw + kStages * kStageBytes + kNewBytes + kGroups * 16 * sizeof(float));
    // cluster merge (only when every CTA streams at most one tile, so ring stage 1 is never loaded): the receive area
    // [splits][NREP][D + 2] floats lives in stage 1 -- no extra shared memory, and free from the start of the kernel
    static_assert(kStages >= 2, "the receive area takes the second ring stage");
    float* rx = reinterpret_cast<float*>(smem_raw + kStageBytes);

    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, l16 = lane & 15;

    // cluster merge: first phase of the cluster barrier, arrived at once and waited for only before the first access to
    // the leader's shared memory (every CTA of the cluster must have started by then; by that time it long has)
    if (p.cluster_merge && gridDim.x > 1) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    // launched with the programmatic-dependent-launch attribute: q / k_new / v_new and the length array
    // may come from the kernel just before this one
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const StepLen sl = step_length(p, b);                           // cached keys before this token, and whether it fits
    const int len = sl.len, total = sl.total;
    const int k_begin = split * p.chunk;
    if (split == 0 && kvh == 0 && threadIdx.x == 0) {
        // what this step used, for the combine kernel (stable even when seq_lens advances)
        reinterpret_cast<int*>(p.workspace)[b] = sl.header();
        if (sl.overflow) atomicCAS(p.status, 0, (2 << 24) | (b & 0xFFFFFF));
    }
    // let the combine kernel's blocks be scheduled as soon as every CTA of this grid has started
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const bool nothing = k_begin >= total;                          // no key for this split
    if (nothing && !p.cluster_merge) return;                        // (a cluster member stays for the cluster barriers)
    const int k_end = min(len, k_begin + p.chunk);                  // cached keys [k_begin, k_end)
    const bool owns_new = !nothing && sl.append && (len / p.chunk == split);
    const int ntiles = (!nothing && k_end > k_begin) ? (k_end - k_begin + kTile - 1) / kTile : 0;
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&sm->full[s], 1); mbar_init(&sm->empty[s], CW); }
        sm->abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    const WaitCtx abort_flag{&sm->abort_flag, p.status};

    const T* kc = static_cast<const T*>(p.k_cache.ptr) + b * p.k_cache.sb + kvh * p.k_cache.sh;
    const T* vc = static_cast<const T*>(p.v_cache.ptr) + b * p.v_cache.sb + kvh * p.v_cache.sh;

    if (warp == CW) {
        // ---------------- producer: one lane streams K/V tiles ----------------
        if (lane == 0) {
            for (int t = 0; t < ntiles; ++t) {
                int s = t % kStages;
                if (t >= kStages && !mbar_wait(&sm->empty[s], ((t / kStages) - 1) & 1, abort_flag, 0x10)) break;
                int row0 = k_begin + t * kTile;
                int nk = min(kTile, k_end - row0);
                uint32_t bytes = static_cast<uint32_t>(nk) * kRowBytes;
                mbar_arrive_expect_tx(&sm->full[s], 2 * bytes);
                unsigned char* dst = smem_raw + s * kStageBytes;
                bulk_load(dst, kc + static_cast<long long>(row0) * D, bytes, &sm->full[s]);
                bulk_load(dst + kTile * kRowBytes, vc + static_cast<long long>(row0) * D, bytes, &sm->full[s]);
            }
        }
    } else {
        // ---------------- consumers ----------------
        WarpState<T, NREP> st;
        st.m = -INFINITY; st.l = 0.f;
#pragma unroll
        for (int h = 0; h < NREP; ++h)
#pragma unroll
            for (int i = 0; i < 4; ++i) st.o[h][i] = make_float2(0.f, 0.f);

        // rotation angles of the query / new token for this lane's 4 pairs
        float cs[4], sn[4];
        if (p.rope) {
            float pos = __int2float_rn(p.q_positions ? p.q_positions[b] : static_cast<int>(p.pos_offset) + len);
#pragma unroll
            for (int i = 0; i < 4; ++i) sincosf(pos * p.inv_freq.v[l16 * 4 + i], &sn[i], &cs[i]);
        }
        const float qscale = p.scale * kLog2e;
#pragma unroll
        for (int h = 0; h < NREP; ++h) {
            const T* qp = static_cast<const T*>(p.q.ptr) + b * p.q.sb + (kvh * NREP + h) * p.q.sh + l16 * 8;
            uint4 raw = *reinterpret_cast<const uint4*>(qp);
            const uint32_t* u = &raw.x;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float2 t = Elem<T>::unpack2(u[i]);
                if (p.rope) {
                    float t1 = __fmul_rn(t.x, cs[i]), t2 = __fmul_rn(t.y, sn[i]);
                    float t3 = __fmul_rn(t.x, sn[i]), t4 = __fmul_rn(t.y, cs[i]);
                    t.x = __fsub_rn(t1, t2); t.y = __fadd_rn(t3, t4);
                }
                st.q[h][i] = make_float2(t.x * qscale, t.y * qscale);
            }
        }

        // new token: rotate k, stage k/v in shared memory, write the cache row
        if (owns_new && warp == 0 && lane < 16) {
            const T* kn = static_cast<const T*>(p.k_new.ptr) + b * p.k_new.sb + kvh * p.k_new.sh + l16 * 8;
            const T* vn = static_cast<const T*>(p.v_new.ptr) + b * p.v_new.sb + kvh * p.v_new.sh + l16 * 8;
            uint4 kraw = *reinterpret_cast<const uint4*>(kn);
            uint4 vraw = *reinterpret_cast<const uint4*>(vn);
            {
                // this step scores the new key in fp32; the cache gets its 16-bit rounding
                uint32_t* u = &kraw.x;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float2 t = Elem<T>::unpack2(u[i]);
                    if (p.rope) {
                        float t1 = __fmul_rn(t.x, cs[i]), t2 = __fmul_rn(t.y, sn[i]);
                        float t3 = __fmul_rn(t.x, sn[i]), t4 = __fmul_rn(t.y, cs[i]);
                        t.x = __fsub_rn(t1, t2); t.y = __fadd_rn(t3, t4);
                        u[i] = Elem<T>::pack2(t.x, t.y);
                    }
                    newk[l16 * 8 + 2 * i] = t.x;
                    newk[l16 * 8 + 2 * i + 1] = t.y;
                }
            }
            *reinterpret_cast<uint4*>(newv + l16 * 8) = vraw;
            {   // owns_new implies len < cache_cap: step_length refuses the append otherwise, whatever seq_lens holds
                T* kdst = const_cast<T*>(kc) + static_cast<long long>(len) * D + l16 * 8;
                T* vdst = const_cast<T*>(vc) + static_cast<long long>(len) * D + l16 * 8;
                *reinterpret_cast<uint4*>(kdst) = kraw;
                *reinterpret_cast<uint4*>(vdst) = vraw;
            }
        }

        const int group = warp * 2 + (lane >> 4);
        float* pbuf = pbuf_all + group * 16;
        bool ok = true;
        for (int t = 0; t < ntiles && ok; ++t) {
            int s = t % kStages;
            ok = mbar_wait(&sm->full[s], (t / kStages) & 1, abort_flag, 0x20);
            if (!ok) break;
            const T* ksm = ring + static_cast<size_t>(s) * (kStageBytes / sizeof(T));
            const T* vsm = ksm + kTile * D;
            int nk = min(kTile, k_end - (k_begin + t * kTile));
            process_rows<T, NREP>(st, ksm, vsm, nk, warp, CW, lane, pbuf);
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm->empty[s]);
        }
        if (owns_new && warp == 0) {
            __syncwarp();
            // one extra key: lands in half-warp 0's slot, half-warp 1 sees only masked rows
            process_rows<T, NREP, true>(st, newk, newv, 1, 0, 1, lane, pbuf);
        }

        // ---- merge the half-warp groups of the CTA through shared memory (the ring is free now) ----
        float l = st.l;
#pragma unroll
        for (int off = NREP; off < 16; off <<= 1) l += __shfl_xor_sync(0xFFFFFFFFu, l, off);
        asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");   // all consumers done with the ring
        float* go = reinterpret_cast<float*>(smem_raw);                             // [kGroups][NREP][128]
        float* gm = go + kGroups * NREP * 128;                                      // [kGroups][NREP]
        float* gl = gm + kGroups * NREP;                                            // [kGroups][NREP]
        if (l16 < NREP) { gm[group * NREP + l16] = st.m; gl[group * NREP + l16] = l; }
#pragma unroll
        for (int h = 0; h < NREP; ++h) {
            float4* dst = reinterpret_cast<float4*>(go + (group * NREP + h) * 128 + l16 * 8);
            dst[0] = make_float4(st.o[h][0].x, st.o[h][0].y, st.o[h][1].x, st.o[h][1].y);
            dst[1] = make_float4(st.o[h][2].x, st.o[h][2].y, st.o[h][3].x, st.o[h][3].y);
        }
        asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");

        // thread d (0..127) finishes dim d of every head
        if (tid < 128) {
            const int d = tid;
            float* wsp = p.workspace + p.ws_header;   // after the per-sequence length slots
            const int nsplits = p.num_splits;
#pragma unroll
            for (int h = 0; h < NREP; ++h) {
                float M = -INFINITY;
#pragma unroll
                for (int g = 0; g < kGroups; ++g) M = fmaxf(M, gm[g * NREP + h]);
                float L = 0.f, acc = 0.f;
#pragma unroll
                for (int g = 0; g < kGroups; ++g) {
                    float mg = gm[g * NREP + h];
                    float w = (mg == -INFINITY) ? 0.f : fast_exp2(mg - M);
                    L += gl[g * NREP + h] * w;
                    acc += go[(g * NREP + h) * 128 + d] * w;
                }
                if (p.cluster_merge) {
                    // this split's row of the receive area, in this CTA's own shared memory (the leader's is final)
                    if (!nothing) {
                        float* own = rx + (split * NREP + h) * (D + 2);
                        own[d] = acc;
                        if (d == 0) { own[D] = M; own[D + 1] = L; }
                    }
                } else {
                    float* out = wsp + ((static_cast<long long>(b) * p.Hkv + kvh) * nsplits + split) * NREP * (D + 2) + h * (D + 2);
                    out[d] = acc / L;
                    if (d == 0) { out[D] = M * kLn2; out[D + 1] = L; }
                }
            }
        }
    }

    if (p.cluster_merge) {
        // The splits of this (batch, kv_head) are one cluster: every member forwards its per-head (acc, m, l) into the
        // leader's receive area (ring stage 1, never loaded here, so nobody waits for the leader's ring to drain); after the
        // cluster barrier the leader merges them in split order and writes the final rows -- no combine kernel, no
        // workspace trip.
        const unsigned nsp = gridDim.x;
        if (nsp > 1) {
            __syncwarp();
            asm volatile("barrier.cluster.wait.aligned;" ::: "memory");           // phase 1: every member is running
            if (split != 0 && !nothing && tid < 128) {
                // each thread forwards what it wrote itself: column tid of every head (thread 0 also m and l)
                uint32_t dst;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(dst) : "r"(smem_u32(rx + split * NREP * (D + 2))), "r"(0));
                const float* own = rx + split * NREP * (D + 2);
#pragma unroll
                for (int h = 0; h < NREP; ++h) {
                    const uint32_t a = dst + h * (D + 2) * 4;
                    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(a + tid * 4), "f"(own[h * (D + 2) + tid]) : "memory");
                    if (tid == 0) {
                        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(a + D * 4), "f"(own[h * (D + 2) + D]) : "memory");
                        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(a + (D + 1) * 4), "f"(own[h * (D + 2) + D + 1]) : "memory");
                    }
                }
            }
            __syncwarp();
            asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");   // phase 2: the rows are in the leader's memory
            asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        } else {
            __syncthreads();
        }
        if (split == 0 && tid < 128) {
            const int d = tid;
            // members without keys stored nothing: splits beyond the sequence are a suffix
            const unsigned nvalid = min(nsp, static_cast<unsigned>((total + p.chunk - 1) / p.chunk));
#pragma unroll
            for (int h = 0; h < NREP; ++h) {
                float M = -INFINITY;
                for (unsigned r = 0; r < nvalid; ++r) M = fmaxf(M, rx[(r * NREP + h) * (D + 2) + D]);
                float L = 0.f, acc = 0.f;
                for (unsigned r = 0; r < nvalid; ++r) {
                    const float* pr = rx + (r * NREP + h) * (D + 2);
                    const float mr = pr[D];
                    const float w = (mr == -INFINITY) ? 0.f : fast_exp2(mr - M);
                    L += pr[D + 1] * w;
                    acc += pr[d] * w;
                }
                const int hq = kvh * NREP + h;
                const float o = (total > 0) ? acc / L : 0.f;
                static_cast<T*>(p.o.ptr)[b * p.o.sb + hq * p.o.sh + d] = Elem<T>::from_f(o);
                if (p.lse && d == 0) p.lse[static_cast<long long>(b) * p.Hq + hq] = M * kLn2 + logf(L);
            }
        }
    }
}

// One block per (q_head, batch): merge the valid splits.  512 threads = 4 groups of 128
// (thread d of a group owns output dim d); each group takes a quarter of the splits.
constexpr int kCombineGroups = 4;

template <typename T>
__global__ void __launch_bounds__(128 * kCombineGroups) decode_combine_kernel(DecodeParams p) {
    const int D = p.D;                                   // <= 128: thread d of a group owns dim d, the others idle
    __shared__ float s_red[kCombineGroups * 32];
    __shared__ float s_acc[kCombineGroups][128];
    __shared__ float s_l[kCombineGroups];
    const int hq = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, d = tid & 127, grp = tid >> 7;
    const int nrep = p.Hq / p.Hkv, kvh = hq / nrep, h = hq % nrep;
    // Launched with programmatic stream serialization: the blocks may become resident while the
    // split kernel drains; nothing of its output is touched before this wait returns.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int hdr = reinterpret_cast<const int*>(p.workspace)[b];
    const int total = StepLen::header_total(hdr);                    // keys this step attended to (new token included)
    const bool appended = StepLen::header_appended(hdr);
    const int nsp = min((total + p.chunk - 1) / p.chunk, p.num_splits);
    const float* base = p.workspace + p.ws_header +
                        ((static_cast<long long>(b) * p.Hkv + kvh) * p.num_splits) * nrep * (D + 2) + h * (D + 2);
    const long long sstride = static_cast<long long>(nrep) * (D + 2);

    // global max over the splits
    float M = -INFINITY;
    for (int s = tid; s < nsp; s += blockDim.x) M = fmaxf(M, base[s * sstride + D]);
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xFFFFFFFFu, M, o));
    if ((tid & 31) == 0) s_red[tid >> 5] = M;
    __syncthreads();
    M = s_red[0];
#pragma unroll
    for (int i = 1; i < kCombineGroups * 4; ++i) M = fmaxf(M, s_red[i]);

    // each group accumulates its quarter of the splits (rows of 128 floats: coalesced)
    const int per = (nsp + kCombineGroups - 1) / kCombineGroups;
    const int s_lo = grp * per, s_hi = min(nsp, s_lo + per);
    float L = 0.f, acc = 0.f;
#pragma unroll 4
    for (int s = s_lo; s < s_hi; ++s) {
        const float* row = base + s * sstride;
        float w = expf(row[D] - M) * row[D + 1];
        L += w;
        if (d < D) acc += w * row[d];
    }
    s_acc[grp][d] = acc;
    if (d == 0) s_l[grp] = L;
    __syncthreads();
    if (grp != 0) return;
    acc = 0.f; L = 0.f;
#pragma unroll
    for (int g = 0; g < kCombineGroups; ++g) { acc += s_acc[g][d]; L += s_l[g]; }

    float o = (nsp > 0) ? acc / L : 0.f;
    if (p.partial_out) {
        float* po = p.partial_out + (static_cast<long long>(b) * p.Hq + hq) * (D + 2);
        if (d < D) po[d] = o;
        if (d == 0) { po[D] = M; po[D + 1] = L; }
    } else {
        T* og = static_cast<T*>(p.o.ptr) + b * p.o.sb + hq * p.o.sh;
        if (d < D) og[d] = Elem<T>::from_f(o);
        if (p.lse && d == 0) p.lse[static_cast<long long>(b) * p.Hq + hq] = M + logf(L);
    }
    // a full sequence (token not appended) keeps its length
    if (hq == 0 && d == 0 && p.seq_lens && appended && p.advance_lens) p.seq_lens[b] = total;
}

// partials [R, rows, D+2] -> out [rows, D], lse [rows]
template <typename T>
__global__ void lse_combine_kernel(const float* __restrict__ partials, int R, long long rows, int D,
                                   T* __restrict__ out, float* __restrict__ lse) {
    long long row = blockIdx.x;
    int d = threadIdx.x;
    const long long rstride = rows * (D + 2);
    const float* base = partials + row * (D + 2);
    float M = -INFINITY;
    for (int r = 0; r < R; ++r) M = fmaxf(M, base[r * rstride + D]);
    float L = 0.f, acc = 0.f;
    for (int r = 0; r < R; ++r) {
        float mr = base[r * rstride + D];
        float w = (mr == -INFINITY) ? 0.f : expf(mr - M) * base[r * rstride + D + 1];
        L += w;
        if (d < D) acc += w * base[r * rstride + d];
    }
    if (d < D) out[row * D + d] = Elem<T>::from_f(acc / L);
    if (lse && d == 0) lse[row] = M + logf(L);
}

template <typename T>
int launch_combine(cudaStream_t s, const DecodeParams& p) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(p.Hq, p.B);
    cfg.blockDim = dim3(128 * kCombineGroups);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    VB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, decode_combine_kernel<T>, p));
    note_launch();
    VB200_CUDA_TRY(cudaPeekAtLastError());
    return VB200_OK;
}

// every shape the tuned kernels do not take (decode_generic.cu), then the common combine
template <typename T>
int launch_decode_generic(cudaStream_t s, const DecodeParams& p) {
    if (p.fused_exchange) return set_detail(VB200_ERR_UNSUPPORTED, "decode + exchange in one launch needs 16-bit caches with head_dim 128");
    profile_mark_begin(s);
    if (int rc = launch_decode_generic_split(s, p)) return rc;
    profile_mark_end(s);
    return launch_combine<T>(s, p);
}

constexpr int kMaxClusterSplits = 16;   // cluster sizes above 8 need the non-portable cluster size attribute

template <typename T, int NREP>
int launch_decode_t(cudaStream_t s, const DecodeParams& p) {
    constexpr int D = 128;
    // Measured on B200: 4 consumer warps per CTA beat 6 and 8 (fewer keys per warp and tile, costlier
    // merge); for groups of up to 4 query heads three CTAs per SM with a 2-deep ring are fastest
    // (128 registers suffice), 8-head groups need ~170 registers: two CTAs per SM, 3-deep ring.
    constexpr int CW = 4;
    constexpr int kStages = (NREP <= 4) ? 2 : 3;
    constexpr int MINB = (NREP <= 4) ? 3 : 2;
    // Groups of 8 heads are compute-bound on CUDA cores and always take the warp-MMA split kernel; groups of 4
    // take it when a CTA streams at least 256 keys (measured: 5.7 vs 5.3 TB/s on 1-8 K contexts) and the
    // CUDA-core kernel below that, where its lighter prologue wins (3 us per call at 600-key contexts).
    bool use_mma = false, need_combine = true;
    if constexpr (NREP == 8) use_mma = true;
    if constexpr (NREP == 4) use_mma = p.chunk >= 256 || p.fused_exchange;
    if (p.fused_exchange) {
        // the exchange runs as the tail of the warp-MMA split kernel: no combine launch
        if (!use_mma) return set_detail(VB200_ERR_UNSUPPORTED, "decode + exchange in one launch needs 4 or 8 query heads per KV head");
        need_combine = false;
    }
    if (use_mma) {
        if constexpr (NREP == 4 || NREP == 8) {
            profile_mark_begin(s);
            if (int rc = launch_decode_gqa_mma_split<T, NREP>(s, p)) return rc;
        }
    } else if constexpr (NREP != 8) {       // (the CUDA-core kernel is never the choice for 8-head groups)
        constexpr size_t kBaseSmem = decode_base_smem<T, NREP, CW, kStages>();
        constexpr size_t kRxRow = NREP * (D + 2) * sizeof(float);                       // one split's (acc, m, l) per head
        static_assert(2 * CW * NREP * 128 * 4 + 2 * 2 * CW * NREP * 4 <= 2 * kTile * 128 * sizeof(T), "merge buffers must fit in the first ring stage (the second may hold the cluster receive area)");
        static thread_local bool configured[64] = {};      // per device ordinal: the attribute belongs to the device's context
        int dev = 0;
        VB200_CUDA_TRY(cudaGetDevice(&dev));
        if (dev < 0 || dev >= 64) return set_detail(VB200_ERR_NO_DEVICE, "device ordinal out of range");
    if (!configured[dev]) {
            VB200_CUDA_TRY(cudaFuncSetAttribute(decode_splitkv_kernel<T, NREP, CW, kStages, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                static_cast<int>(kBaseSmem)));
            VB200_CUDA_TRY(cudaFuncSetAttribute(decode_splitkv_kernel<T, NREP, CW, kStages, MINB>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
            configured[dev] = true;
        }
        // Up to 16 one-tile splits per (batch, kv_head): they run as one thread-block cluster that merges its partials
        // through distributed shared memory and writes the final rows -- the combine kernel and the workspace round
        // trip drop out.  Not when the caller wants the partial record or the length array advanced (the combine
        // kernel does that after every CTA of the grid has read the lengths), nor when a CTA streams more than one
        // tile (the receive area is the ring's second stage).
        DecodeParams q = p;
        constexpr size_t kStageBytesHost = 2 * kTile * D * sizeof(T);
        q.cluster_merge = (!p.partial_out && !(p.seq_lens && p.advance_lens && p.append) && p.num_splits <= kMaxClusterSplits &&
                           p.chunk <= kTile && p.num_splits * kRxRow <= kStageBytesHost) ? 1 : 0;
        dim3 grid(p.num_splits, p.Hkv, p.B);
        if (q.cluster_merge && p.num_splits > 8) {
            // a size above the portable 8 must fit one GPC of this device: asked once per size
            static thread_local int fits[kMaxClusterSplits + 1] = {};   // 0 unknown, 1 yes, -1 no
            static thread_local int fits_dev = -1;
            if (fits_dev != dev) { for (int& f : fits) f = 0; fits_dev = dev; }
            if (fits[p.num_splits] == 0) {
                cudaLaunchConfig_t probe{};
                probe.gridDim = grid;
                probe.blockDim = dim3((CW + 1) * 32);
                probe.dynamicSmemBytes = kBaseSmem;
                cudaLaunchAttribute pa[1];
                pa[0].id = cudaLaunchAttributeClusterDimension;
                pa[0].val.clusterDim.x = static_cast<unsigned>(p.num_splits);
                pa[0].val.clusterDim.y = 1;
                pa[0].val.clusterDim.z = 1;
                probe.attrs = pa;
                probe.numAttrs = 1;
                int n_clusters = 0;
                cudaError_t e = cudaOccupancyMaxActiveClusters(&n_clusters, decode_splitkv_kernel<T, NREP, CW, kStages, MINB>, &probe);
                if (e != cudaSuccess) { (void)cudaGetLastError(); n_clusters = 0; }
                fits[p.num_splits] = n_clusters > 0 ? 1 : -1;
            }
            if (fits[p.num_splits] < 0) q.cluster_merge = 0;
        }
        need_combine = !q.cluster_merge;
        const size_t smem = kBaseSmem;
        profile_mark_begin(s);
        {
            cudaLaunchConfig_t cfg{};
            cfg.gridDim = grid;
            cfg.blockDim = dim3((CW + 1) * 32);
            cfg.dynamicSmemBytes = smem;
            cfg.stream = s;
            cudaLaunchAttribute attr[2];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            int n_attr = 1;
            if (q.cluster_merge && p.num_splits > 1) {
                attr[1].id = cudaLaunchAttributeClusterDimension;
                attr[1].val.clusterDim.x = static_cast<unsigned>(p.num_splits);
                attr[1].val.clusterDim.y = 1;
                attr[1].val.clusterDim.z = 1;
                n_attr = 2;
            }
            cfg.attrs = attr;
            cfg.numAttrs = n_attr;
            VB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, decode_splitkv_kernel<T, NREP, CW, kStages, MINB>, q));
        }
    }
    profile_mark_end(s);
    note_launch();
    VB200_CUDA_TRY(cudaPeekAtLastError());
    if (need_combine) {
        if (int rc = launch_combine<T>(s, p)) return rc;
    }
    VB200_CUDA_TRY(cudaPeekAtLastError());
    return VB200_OK;
}

template <typename T>
int launch_decode_nrep(cudaStream_t s, const DecodeParams& p) {
    switch (p.Hq / p.Hkv) {
        case 1: return launch_decode_t<T, 1>(s, p);
        case 2: return launch_decode_t<T, 2>(s, p);
        case 4: return launch_decode_t<T, 4>(s, p);
        case 8: return launch_decode_t<T, 8>(s, p);
        default: return launch_decode_generic<T>(s, p);        // other group sizes
    }
}

}  // namespace

int decode_tile_keys() { return kTile; }

int launch_decode(cudaStream_t s, const DecodeParams& p) {
    // the tuned kernels: 16-bit caches, head_dim 128, contiguous cache rows (a tile is one bulk copy / TMA box)
    const bool tuned = p.D == 128 && p.dtype != VB200_F32 && p.k_cache.ss == p.D && p.v_cache.ss == p.D;
    if (p.dtype == VB200_BF16) return tuned ? launch_decode_nrep<__nv_bfloat16>(s, p) : launch_decode_generic<__nv_bfloat16>(s, p);
    if (p.dtype == VB200_F16) return tuned ? launch_decode_nrep<__half>(s, p) : launch_decode_generic<__half>(s, p);
    if (p.dtype == VB200_F32) return launch_decode_generic<float>(s, p);
    return set_detail(VB200_ERR_UNSUPPORTED, "decode: unknown dtype");
}

int launch_lse_combine(cudaStream_t s, const float* partials, int R, long long rows, int D,
                       int dtype, void* out, float* lse) {
    if (rows <= 0) return VB200_OK;
    if (D > 1024) return VB200_ERR_UNSUPPORTED;
    int threads = ((D + 31) / 32) * 32;
    unsigned grid = static_cast<unsigned>(rows);
    switch (dtype) {
        case VB200_BF16: lse_combine_kernel<__nv_bfloat16><<<grid, threads, 0, s>>>(partials, R, rows, D, static_cast<__nv_bfloat16*>(out), lse); break;
        case VB200_F16: lse_combine_kernel<__half><<<grid, threads, 0, s>>>(partials, R, rows, D, static_cast<__half*>(out), lse); break;
        default: return VB200_ERR_UNSUPPORTED;
    }
    note_launch();
    VB200_CUDA_TRY(cudaPeekAtLastError());
    return VB200_OK;
}

}  // namespace vb200
