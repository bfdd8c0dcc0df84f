// y = x W^T for bf16 activations x[M,K] and bf16 weights W[N,K] (the layout of the reference's
// nn::Linear::weight, src/nn/linear.cpp:19, whose forward is matmul(input, weight.transpose(0,1)),
// src/nn/linear.cpp:41-48) on the sm_100a tensor cores, fp32 accumulation in TMEM.
//
// Two kernels share the TMA / tcgen05 plumbing:
//   linear_wide_kernel    M > 16 (prompt processing).  Persistent CTAs walk 128 x 256 output tiles;
//                         x rows are the UMMA M operand, W rows the N operand; 4-stage TMA ring,
//                         two TMEM accumulators so the epilogue of one tile overlaps the next mainloop.
//   linear_skinny_kernel  M <= 16 (one token per sequence).  The product is weight-bandwidth bound,
//                         so the roles swap: 128 W rows are the UMMA M operand and the (zero padded)
//                         16 token rows the N operand; K is split over the CTAs of a thread-block
//                         cluster, which reduce their partial tiles through distributed shared
//                         memory in a fixed order (deterministic) before the leader's epilogue.
// Epilogues (fused, per output element): store bf16 | store fp32 | fp32 accumulate into the residual
// stream | SwiGLU over interleaved (gate, up) weight rows -> bf16 (src/nn/swiglu.cpp:36-48,
// ops::silu_mul src/ops/elementwise.cpp:1297-1328).
#include "kernels.h"

#include <cuda.h>
#include <cstdio>

namespace vb200 {
namespace {

constexpr int kBK = 64;                 // K elements per stage = one 128-byte swizzle row
constexpr int kTileA = 128;             // rows of the UMMA M operand
constexpr int kThreads = 192;           // warp 0: TMA producer, warp 1: MMA issuer, warps 2-5: epilogue
constexpr int kABytes = kTileA * kBK * 2;

struct LinearMaps {
    CUtensorMap a;   // UMMA M operand rows
    CUtensorMap b;   // UMMA N operand rows
};

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        : : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
// After an expired wait the CTA leaves early while bulk copies it issued may still be landing in
// its shared memory: stay resident for a bounded time (far longer than a copy takes) before exiting.
__device__ __forceinline__ void abort_linger(volatile int* abort_flag) {
    if (*abort_flag && threadIdx.x == 0) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {}
    }
    __syncthreads();
}
// 32-byte global accesses (sm_100): half as many store instructions per row segment as 16-byte ones.  The
// interface promises 16-byte alignment only, so a segment that is not 32-byte aligned goes as two halves.
__device__ __forceinline__ void st_global_v8(void* ptr, const uint32_t (&w)[8]) {
    if ((reinterpret_cast<uintptr_t>(ptr) & 31) == 0) {
        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                     ::"l"(ptr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
    } else {
        uint4* p4 = static_cast<uint4*>(ptr);
        p4[0] = make_uint4(w[0], w[1], w[2], w[3]);
        p4[1] = make_uint4(w[4], w[5], w[6], w[7]);
    }
}
__device__ __forceinline__ void ld_global_v8(const void* ptr, uint32_t (&w)[8]) {
    if ((reinterpret_cast<uintptr_t>(ptr) & 31) == 0) {
        asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                     : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]) : "l"(ptr) : "memory");
    } else {
        const uint4* p4 = static_cast<const uint4*>(ptr);
        const uint4 a = p4[0], b = p4[1];
        w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
    }
}
__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + __expf(-g)); }

// One output element group of the wide kernel: 32 consecutive columns of one row.
template <int EPI>
__device__ __forceinline__ void store_row32(const LinearParams& p, int row, int col0, uint32_t (&acc)[32]) {
    if (p.row_scale != nullptr) {                // deferred RMSNorm: this row's 1/rms
        const float rs = __ldg(p.row_scale + row);
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = __float_as_uint(__uint_as_float(acc[j]) * rs);
    }
    if (p.bias != nullptr) {                     // nn::Linear's bias (src/nn/linear.cpp:44-46)
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) acc[j] = __float_as_uint(__uint_as_float(acc[j]) + __ldg(p.bias + col0 + j));
    }
    if (EPI == VB200_EPI_SWIGLU) {
        // columns (2j, 2j+1) = (gate_j, up_j) -> out[row, col0/2 + j]
        __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(row) * p.ldo + (col0 >> 1);
        const int n_out = min(16, (p.N - col0) >> 1);
        uint32_t packed[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float a0 = silu_f(__uint_as_float(acc[4 * j])) * __uint_as_float(acc[4 * j + 1]);
            float a1 = silu_f(__uint_as_float(acc[4 * j + 2])) * __uint_as_float(acc[4 * j + 3]);
            packed[j] = Elem<__nv_bfloat16>::pack2(a0, a1);
        }
        if (n_out == 16) {
            st_global_v8(out, packed);
        } else {
            for (int j = 0; j < n_out; ++j) {
                const uint32_t u = packed[j >> 1];
                reinterpret_cast<uint16_t*>(out)[j] = static_cast<uint16_t>((j & 1) ? (u >> 16) : (u & 0xFFFF));
            }
        }
        return;
    }
    const int n_valid = min(32, p.N - col0);
    if (EPI == VB200_EPI_BF16) {
        __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(row) * p.ldo + col0;
        if (n_valid == 32) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                uint32_t w8[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) w8[e] = Elem<__nv_bfloat16>::pack2(__uint_as_float(acc[16 * j + 2 * e]), __uint_as_float(acc[16 * j + 2 * e + 1]));
                st_global_v8(out + 16 * j, w8);
            }
        } else {
            for (int j = 0; j < n_valid; ++j) out[j] = __float2bfloat16_rn(__uint_as_float(acc[j]));
        }
    } else {
        float* out = static_cast<float*>(p.out) + static_cast<long long>(row) * p.ldo + col0;
        if (n_valid == 32) {
            uint32_t hres[4][8];
            if (EPI == VB200_EPI_ADD_F32) {                     // all four 32-byte loads of the residual in flight at once
#pragma unroll
                for (int j = 0; j < 4; ++j) ld_global_v8(out + 8 * j, hres[j]);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t w8[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    float v = __uint_as_float(acc[8 * j + e]);
                    if (EPI == VB200_EPI_ADD_F32) v += __uint_as_float(hres[j][e]);
                    w8[e] = __float_as_uint(v);
                    acc[8 * j + e] = w8[e];                     // the new residual value, for the scaled copy below
                }
                st_global_v8(out + 8 * j, w8);
            }
        } else {
            for (int j = 0; j < n_valid; ++j) {
                float v = __uint_as_float(acc[j]);
                if (EPI == VB200_EPI_ADD_F32) v += out[j];
                out[j] = v;
                acc[j] = __float_as_uint(v);
            }
        }
        if (EPI == VB200_EPI_ADD_F32 && p.scaled_copy != nullptr) {
            __nv_bfloat16* cp = static_cast<__nv_bfloat16*>(p.scaled_copy) + static_cast<long long>(row) * p.N + col0;
            if (n_valid == 32) {
                const float4* g4 = reinterpret_cast<const float4*>(p.copy_scale + col0);
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    uint32_t w8[8];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float4 gw = __ldg(g4 + 4 * j + e);
                        w8[2 * e] = Elem<__nv_bfloat16>::pack2(__uint_as_float(acc[16 * j + 4 * e]) * gw.x, __uint_as_float(acc[16 * j + 4 * e + 1]) * gw.y);
                        w8[2 * e + 1] = Elem<__nv_bfloat16>::pack2(__uint_as_float(acc[16 * j + 4 * e + 2]) * gw.z, __uint_as_float(acc[16 * j + 4 * e + 3]) * gw.w);
                    }
                    st_global_v8(cp + 16 * j, w8);
                }
            } else {
                for (int j = 0; j < n_valid; ++j) cp[j] = __float2bfloat16_rn(__uint_as_float(acc[j]) * __ldg(p.copy_scale + col0 + j));
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Wide kernel: out[m, n] = sum_k x[m,k] W[n,k], tiles of 128 rows (m) x BN columns (n).
// ------------------------------------------------------------------------------------------------
template <int BN>
struct WideCfg {
    static constexpr int kStages = 4;
    static constexpr int kBBytes = BN * kBK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBarOffset = kStages * kStageBytes;
    static constexpr int kSmemBytes = kBarOffset + 256 + 1024;      // barriers + slack for 1024-byte alignment
    static constexpr int kTmemCols = 2 * BN;                        // two accumulators
    static_assert(kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "TMEM allocation is a power of two <= 512");
};

template <int BN, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
linear_wide_kernel(const __grid_constant__ LinearMaps maps, LinearParams p) {
    using C = WideCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::kBarOffset);
    uint64_t* empty = full + C::kStages;
    uint64_t* acc_full = empty + C::kStages;      // [2]
    uint64_t* acc_empty = acc_full + 2;           // [2]
    uint64_t* drain = acc_empty + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tiles = (p.M + kTileA - 1) / kTileA;
    const int n_tiles = (p.N + BN - 1) / BN;
    const int tiles = m_tiles * n_tiles;
    const int k_blocks = (p.K + kBK - 1) / kBK;
    const WaitCtx ctx{abort_flag, p.status};

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < C::kStages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
        mbar_init(drain, 1);
        mbar_fence_init();
        tma_prefetch_desc(&maps.a);
        tma_prefetch_desc(&maps.b);
    }
    if (warp == 1) { tmem_alloc(tmem_slot, C::kTmemCols); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // the next kernel in the stream may be scheduled now (it waits for this grid to finish before it reads
    // anything); the activations may come from the kernel launched just before this one
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            for (int t = blockIdx.x; t < tiles && !*abort_flag; t += gridDim.x) {
                const int mt = t % m_tiles, nt = t / m_tiles;   // consecutive CTAs share a W tile through L2
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % C::kStages;
                    if (it >= C::kStages && !mbar_wait(&empty[s], ((it / C::kStages) - 1) & 1, ctx, 0x41)) break;
                    uint8_t* st = smem + s * C::kStageBytes;
                    mbar_arrive_expect_tx(&full[s], C::kStageBytes);
                    tma_load_2d(st, &maps.a, &full[s], kb * kBK, mt * kTileA);
                    tma_load_2d(st + kABytes, &maps.b, &full[s], kb * kBK, nt * BN);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_f16(1, 0, 0, kTileA, BN);
            uint32_t it = 0, tile_no = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++tile_no) {
                const int buf = tile_no & 1;
                if (tile_no >= 2) ok = mbar_wait(&acc_empty[buf], ((tile_no >> 1) - 1) & 1, ctx, 0x42);
                if (!ok) break;
                tc_fence_after();
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % C::kStages;
                    if (!mbar_wait(&full[s], (it / C::kStages) & 1, ctx, 0x43)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + s * C::kStageBytes), b_addr = a_addr + kABytes;
#pragma unroll
                    for (int kk = 0; kk < kBK / 16; ++kk) {
                        umma_ss(tmem_base + buf * BN, make_smem_desc_sw128(a_addr + kk * 32, 16, 1024),
                                make_smem_desc_sw128(b_addr + kk * 32, 16, 1024), idesc, (kb | kk) ? 1u : 0u);
                    }
                    umma_commit(&empty[s]);           // the stage is free once these MMAs have read it
                }
                if (ok) umma_commit(&acc_full[buf]);
            }
            // drain: no MMA may be in flight when TMEM is freed (also on the abort path)
            umma_commit(drain);
            mbar_wait(drain, 0, ctx, 0x44);
        }
    } else {
        const int quarter = warp & 3;                 // TMEM lanes this warp may read
        uint32_t tile_no = 0;
        for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++tile_no) {
            const int mt = t % m_tiles, nt = t / m_tiles;
            const int buf = tile_no & 1;
            if (!mbar_wait_warp(&acc_full[buf], (tile_no >> 1) & 1, ctx, 0x45)) break;
            tc_fence_after();
            const int row = mt * kTileA + quarter * 32 + lane;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t acc[32];
                tmem_ld32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN + c * 32, acc);
                tmem_ld_wait();
                const int col0 = nt * BN + c * 32;
                if (row < p.M && col0 < p.N) store_row32<EPI>(p, row, col0, acc);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, C::kTmemCols);
    abort_linger(abort_flag);
}

// ------------------------------------------------------------------------------------------------
// Skinny kernel: out[m, n] = sum_k x[m,k] W[n,k] for m < MT <= 64.  One CTA = 128 W rows x one K slice;
// the `splits` CTAs of a cluster hold the K slices of the same 128 rows.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

template <int MT>
struct SkinnyCfg {
    static constexpr int kStages = 6;
    static constexpr int kBBytes = MT * kBK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kRingBytes = kStages * kStageBytes;
    static constexpr int kBarOffset = kRingBytes;
    static constexpr int kSmemBytes = kBarOffset + 256 + 1024;
    static constexpr int kTmemCols = MT < 32 ? 32 : MT;
    static constexpr int kPeerBytes = MT * kTileA * 4;                   // one peer's partial tile, fp32
    static constexpr int kMaxSplits = (1 + kRingBytes / kPeerBytes) < 8 ? (1 + kRingBytes / kPeerBytes) : 8;
};

template <int MT, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
linear_skinny_kernel(const __grid_constant__ LinearMaps maps, LinearParams p, int splits) {
    using C = SkinnyCfg<MT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::kBarOffset);
    uint64_t* empty = full + C::kStages;
    uint64_t* acc_full = empty + C::kStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = splits > 1 ? cluster_rank() : 0;
    const int nt = blockIdx.x / splits;
    const int k_blocks = (p.K + kBK - 1) / kBK;
    const int kb_per = (k_blocks + splits - 1) / splits;
    const int kb0 = static_cast<int>(rank) * kb_per;
    const int nkb = max(0, min(k_blocks, kb0 + kb_per) - kb0);
    const WaitCtx ctx{abort_flag, p.status};
    __shared__ float s_inv_rms[MT];

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < C::kStages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
        mbar_init(acc_full, 1);
        mbar_fence_init();
        tma_prefetch_desc(&maps.a);
        tma_prefetch_desc(&maps.b);
    }
    if (warp == 1) { tmem_alloc(tmem_slot, C::kTmemCols); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Programmatic dependent launch: the next kernel of the stream may be scheduled as soon as every CTA of
    // this grid is here, and this grid was scheduled while its predecessor was still running.  Weights do
    // not depend on the predecessor, so their first ring of TMA loads goes out BEFORE griddepcontrol.wait
    // and streams while the predecessor finishes; only the activation loads and the epilogue's global
    // accesses wait for it.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    float acc[MT];
#pragma unroll
    for (int j = 0; j < MT; ++j) acc[j] = 0.0f;

    if (warp == 0) {
        if (lane == 0) {
            const int pre = min(nkb, C::kStages);
            for (int i = 0; i < pre; ++i) {
                mbar_arrive_expect_tx(&full[i], C::kStageBytes);
                tma_load_2d(smem + i * C::kStageBytes, &maps.a, &full[i], (kb0 + i) * kBK, nt * kTileA);     // 128 W rows
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int i = 0; i < pre; ++i)
                tma_load_2d(smem + i * C::kStageBytes + kABytes, &maps.b, &full[i], (kb0 + i) * kBK, 0);      // the token rows (zero filled past M)
            for (int i = pre; i < nkb; ++i) {
                const int s = i % C::kStages;
                if (!mbar_wait(&empty[s], ((i / C::kStages) - 1) & 1, ctx, 0x51)) break;
                uint8_t* st = smem + s * C::kStageBytes;
                mbar_arrive_expect_tx(&full[s], C::kStageBytes);
                tma_load_2d(st, &maps.a, &full[s], (kb0 + i) * kBK, nt * kTileA);
                tma_load_2d(st + kABytes, &maps.b, &full[s], (kb0 + i) * kBK, 0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_f16(1, 0, 0, kTileA, MT);
            for (int i = 0; i < nkb; ++i) {
                const int s = i % C::kStages;
                if (!mbar_wait(&full[s], (i / C::kStages) & 1, ctx, 0x52)) break;
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem + s * C::kStageBytes), b_addr = a_addr + kABytes;
#pragma unroll
                for (int kk = 0; kk < kBK / 16; ++kk) {
                    umma_ss(tmem_base, make_smem_desc_sw128(a_addr + kk * 32, 16, 1024),
                            make_smem_desc_sw128(b_addr + kk * 32, 16, 1024), idesc, (i | kk) ? 1u : 0u);
                }
                umma_commit(&empty[s]);
            }
            umma_commit(acc_full);       // completes once every MMA above has finished (also after a break)
        }
    } else {
        const int quarter = warp & 3;
        asm volatile("griddepcontrol.wait;" ::: "memory");      // before any global access of the epilogue
        if (p.rms_rows != nullptr && rank == 0) {
            // deferred RMSNorm: 1/rms of the token rows, computed while the weights stream (these warps are idle
            // until the accumulator is complete); one warp per row, every load of a 2048-column chunk in flight
            const int m_count = min(p.M, MT), nv = p.rms_dim / 4;
            for (int j = warp - 2; j < m_count; j += 4) {
                const float4* hr = reinterpret_cast<const float4*>(p.rms_rows + static_cast<long long>(j) * p.rms_ld);
                float ss = 0.f;
                for (int c0 = 0; c0 < nv; c0 += 512) {
                    float4 v[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int c = c0 + lane + 32 * i;
                        v[i] = c < nv ? __ldcg(hr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (int i = 0; i < 16; ++i) ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
                if (lane == 0) s_inv_rms[j] = 1.0f / sqrtf(ss / static_cast<float>(p.rms_dim) + p.rms_eps);
            }
        }
        // wait even when this slice is empty: the commit above always arrives
        if (mbar_wait_warp(acc_full, 0, ctx, 0x53) && nkb > 0) {
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < MT / 16; ++c) {
                uint32_t r[16];
                tmem_ld16(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + c * 16, r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[c * 16 + j] = __uint_as_float(r[j]);
            }
        }
        tc_fence_before();
    }

    if (splits > 1) {
        // (1) every CTA of the cluster has finished reading its ring, so the leader's ring can hold the partials
        cluster_sync_all();
        if (warp >= 2 && rank != 0) {
            const int row = (warp & 3) * 32 + lane;
            const uint32_t base = map_to_rank(smem_u32(smem), 0) + (rank - 1) * C::kPeerBytes + row * 4;
#pragma unroll
            for (int j = 0; j < MT; ++j) st_cluster_f32(base + j * (kTileA * 4), acc[j]);
        }
        // (2) partials are visible in the leader's shared memory
        cluster_sync_all();
        if (warp >= 2 && rank == 0) {
            const int row = (warp & 3) * 32 + lane;
            const float* red = reinterpret_cast<const float*>(smem);
            for (int r = 1; r < splits; ++r) {           // fixed order: bit-reproducible
#pragma unroll
                for (int j = 0; j < MT; ++j) acc[j] += red[((r - 1) * MT + j) * kTileA + row];
            }
        }
    }

    if (warp >= 2 && rank == 0) {
        const int n = nt * kTileA + (warp & 3) * 32 + lane;
        const int m_count = min(p.M, MT);
        if (p.rms_rows != nullptr) {
            asm volatile("bar.sync 2, 128;" ::: "memory");       // s_inv_rms written by the four epilogue warps
#pragma unroll
            for (int j = 0; j < MT; ++j) acc[j] *= (j < m_count ? s_inv_rms[j] : 0.f);
        }
        if (p.bias != nullptr && n < p.N) {
            const float bv = __ldg(p.bias + n);
#pragma unroll
            for (int j = 0; j < MT; ++j) acc[j] += bv;
        }
        if (EPI == VB200_EPI_SWIGLU) {
            __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
#pragma unroll
            for (int j = 0; j < MT; ++j) {
                const float other = __shfl_xor_sync(0xFFFFFFFFu, acc[j], 1);     // odd lanes hold the `up` rows
                if (j < m_count && !(lane & 1) && n + 1 < p.N)
                    out[static_cast<long long>(j) * p.ldo + (n >> 1)] = __float2bfloat16_rn(silu_f(acc[j]) * other);
            }
        } else if (n < p.N) {
#pragma unroll
            for (int j = 0; j < MT; ++j) {
                if (j >= m_count) break;
                const long long idx = static_cast<long long>(j) * p.ldo + n;
                if (EPI == VB200_EPI_BF16) static_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16_rn(acc[j]);
                else if (EPI == VB200_EPI_F32) static_cast<float*>(p.out)[idx] = acc[j];
                else {
                    const float hv = static_cast<float*>(p.out)[idx] + acc[j];
                    static_cast<float*>(p.out)[idx] = hv;
                    if (p.scaled_copy != nullptr)
                        static_cast<__nv_bfloat16*>(p.scaled_copy)[static_cast<long long>(j) * p.N + n] = __float2bfloat16_rn(hv * __ldg(p.copy_scale + n));
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, C::kTmemCols);
    abort_linger(abort_flag);
}

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess) return nullptr;
        if (qres != cudaDriverEntryPointSuccess) return nullptr;
        return reinterpret_cast<EncodeTiledFn>(ptr);
    }();
    return fn;
}

// rows x K bf16 matrix with row stride ld (elements) -> 2-D map (K, rows), box [64][box_rows], 128-byte swizzle;
// reads past either extent return zeros.
int make_map_2d(CUtensorMap* m, const void* ptr, long long rows, long long K, long long ld, int box_rows) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return set_detail(VB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        static thread_local char buf[96];
        snprintf(buf, sizeof(buf), "cuTensorMapEncodeTiled (linear) failed with CUresult %d", static_cast<int>(r));
        return set_detail(VB200_ERR_CUDA, buf);
    }
    return VB200_OK;
}

// Raises the dynamic shared memory limit of one kernel instantiation once per device and thread;
// `configured` is the caller's (per instantiation) thread-local array of 64 markers, one per device ordinal.
template <typename Kernel>
int set_smem_once(Kernel kernel, int bytes, bool* configured) {
    int dev = 0;
    VB200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return set_detail(VB200_ERR_NO_DEVICE, "device ordinal out of range");
    if (!configured[dev]) {
        VB200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
        configured[dev] = true;
    }
    return VB200_OK;
}

int sm_count(int* sms) {
    int dev = 0;
    VB200_CUDA_TRY(cudaGetDevice(&dev));
    VB200_CUDA_TRY(cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, dev));
    return VB200_OK;
}

template <int BN, int EPI>
int launch_wide(cudaStream_t s, const LinearParams& p) {
    using C = WideCfg<BN>;
    LinearMaps maps;
    if (int rc = make_map_2d(&maps.a, p.x, p.M, p.K, p.ldx, kTileA)) return rc;
    if (int rc = make_map_2d(&maps.b, p.w, p.N, p.K, p.ldw, BN)) return rc;
    auto kernel = linear_wide_kernel<BN, EPI>;
    static thread_local bool configured[64] = {};
    if (int rc = set_smem_once(kernel, C::kSmemBytes, configured)) return rc;
    int sms = 0;
    if (int rc = sm_count(&sms)) return rc;
    const int tiles = ((p.M + kTileA - 1) / kTileA) * ((p.N + BN - 1) / BN);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(tiles < sms ? tiles : sms));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    VB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, maps, p));
    note_launch();
    return VB200_OK;
}

int pick_splits(int n_tiles, int k_blocks, int max_splits, int sms) {
    int want = (sms + n_tiles - 1) / n_tiles;            // enough CTAs to touch every SM
    if (want > max_splits) want = max_splits;
    if (want > k_blocks) want = k_blocks;
    if (want < 1) want = 1;
    for (int s = want; s <= max_splits && s <= k_blocks; ++s)
        if (k_blocks % s == 0) return s;                 // equal K slices when a nearby count allows it
    return want;
}

template <int MT, int EPI>
int launch_skinny(cudaStream_t s, const LinearParams& p) {
    using C = SkinnyCfg<MT>;
    LinearMaps maps;
    if (int rc = make_map_2d(&maps.a, p.w, p.N, p.K, p.ldw, kTileA)) return rc;
    if (int rc = make_map_2d(&maps.b, p.x, p.M, p.K, p.ldx, MT)) return rc;
    auto kernel = linear_skinny_kernel<MT, EPI>;
    static thread_local bool configured[64] = {};
    if (int rc = set_smem_once(kernel, C::kSmemBytes, configured)) return rc;
    int sms = 0;
    if (int rc = sm_count(&sms)) return rc;
    const int n_tiles = (p.N + kTileA - 1) / kTileA;
    const int splits = p.splits > 0 ? (p.splits < C::kMaxSplits ? p.splits : C::kMaxSplits)
                                    : pick_splits(n_tiles, (p.K + kBK - 1) / kBK, C::kMaxSplits, sms);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(n_tiles * splits));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    int n_attr = 1;
    if (splits > 1) {
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = static_cast<unsigned>(splits);
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        n_attr = 2;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    VB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, maps, p, splits));
    note_launch();
    return VB200_OK;
}

template <int EPI>
int launch_epi(cudaStream_t s, const LinearParams& p) {
    if (p.M <= 16) return launch_skinny<16, EPI>(s, p);
    if (p.M <= 32) return launch_skinny<32, EPI>(s, p);
    if (p.M <= 64) return launch_skinny<64, EPI>(s, p);
    return launch_wide<256, EPI>(s, p);
}

}  // namespace

int launch_linear(cudaStream_t s, const LinearParams& p) {
    switch (p.epilogue) {
        case VB200_EPI_BF16: return launch_epi<VB200_EPI_BF16>(s, p);
        case VB200_EPI_F32: return launch_epi<VB200_EPI_F32>(s, p);
        case VB200_EPI_ADD_F32: {
            if (int rc = launch_epi<VB200_EPI_ADD_F32>(s, p)) return rc;
            // the norm of the finished rows is a second launch, chained by programmatic dependent launch.  (Doing it
            // inside the weight-streaming kernel, by the CTA that finishes last, was measured: fence + ticket +
            // a lone CTA re-reading the rows cost 8 us on the decode step's critical path against 3-4 us here.)
            if (p.norm_out) return launch_rms_norm(s, static_cast<const float*>(p.out), p.norm_w, p.norm_out, p.M, p.N, p.norm_eps);
            return VB200_OK;
        }
        case VB200_EPI_SWIGLU: return launch_epi<VB200_EPI_SWIGLU>(s, p);
        default: return set_detail(VB200_ERR_INVALID_ARG, "unknown linear epilogue");
    }
}

}  // namespace vb200
