// bf16 / fp16 attention forward for sm_100a: TMA-staged Q/K/V tiles,
// tcgen05.mma with TMEM accumulators for S = Q K^T and O = P V, online softmax
// in registers (one thread per query row), causal block skipping, GQA by
// head-group indexing, RoPE of the Q tile fused into the prologue.
//
// Math (same as flash_attention_cpu_dispatch, src/ops/flash_attention.cpp:218-364):
//   s_ij = scale * q_i . k_j ;  key j visible to query i iff j <= start_pos + i
//   O_i = sum_j softmax_j(s_ij) v_j ;  LSE_i = ln sum_j exp(s_ij)
//
// CTA = two 128-row query tiles of one (batch, q_head), processed ping-pong so
// the tensor pipe works on one tile while the other is in softmax:
//   warps 0-3   softmax / correction / epilogue of tile 0   (TMEM lanes 0..127)
//   warps 4-7   the same for tile 1
//   warp  8     TMA producer (Q tiles, then the K/V ring)
//   warp  9     tcgen05.mma issuer, TMEM owner
// TMEM (512 columns): S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [384,384+D);
// P (16-bit, packed two per column) overwrites the first 64 columns of its S.
//
// Every wait is bounded (see mbar_wait); on expiry the CTA drains and returns
// with the device status word set.
#include <cstdio>

#include "kernels.h"

namespace vb200 {

namespace {

constexpr int kBlockM = 128;
constexpr int kBlockN = 128;
constexpr int kStages = 4;
constexpr int kSoftmaxThreads = 256;
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kThreads = 320;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;

struct __align__(8) Barriers {
    uint64_t q_full[2], q_ready[2];
    uint64_t kv_full[kStages], kv_empty[kStages];
    uint64_t s_full[2], p_ready[2], o_done[2];
    uint64_t mma_done;
    uint32_t tmem_base;
    int abort_flag;
};

struct TmaMaps {
    CUtensorMap q, k, v;
};

template <int D>
struct Cfg {
    static constexpr int kHalves = D / 64;                       // 64-column (128-byte) boxes per row
    static constexpr int kHalfBytes = 128 * 128;                 // one [128 rows][64 cols] 16-bit box
    static constexpr int kTileBytes = kHalves * kHalfBytes;      // one [128][D] tile
    static constexpr int kSmemBytes = (2 + kStages) * kTileBytes + 1024 /*alignment slack*/ + 256 /*Barriers*/;
};

template <typename T, int D>
__global__ void __launch_bounds__(kThreads, 1)
prefill_sm100_kernel(const __grid_constant__ TmaMaps maps, PrefillParams p) {
    using C = Cfg<D>;
    extern __shared__ unsigned char smem_dyn[];
    // 128B-swizzled tiles need 1024-byte alignment
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    unsigned char* q_smem = smem;                               // 2 tiles
    unsigned char* kv_smem = smem + 2 * C::kTileBytes;          // kStages tiles
    Barriers* bar = reinterpret_cast<Barriers*>(smem + (2 + kStages) * C::kTileBytes);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- work item: heaviest (last) query pairs first ----
    const int n_bh = p.B * p.Hq;
    const int n_pairs = (p.T + 2 * kBlockM - 1) / (2 * kBlockM);
    const int pair = n_pairs - 1 - static_cast<int>(blockIdx.x) / n_bh;
    const int bh = static_cast<int>(blockIdx.x) % n_bh;
    const int b = bh / p.Hq, hq = bh % p.Hq;
    const int hkv = hq / (p.Hq / p.Hkv);

    int r0[2], nblk[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        r0[t] = (2 * pair + t) * kBlockM;
        if (r0[t] >= p.T) { nblk[t] = 0; continue; }
        int kv_end = p.Skv;
        if (p.causal) kv_end = min(p.Skv, p.start_pos + min(r0[t] + kBlockM, p.T));
        nblk[t] = (kv_end + kBlockN - 1) / kBlockN;
    }
    const int nmax = max(nblk[0], nblk[1]);

    // ---- setup ----
    if (warp == kMmaWarp) {
        if (lane == 0) {
            for (int t = 0; t < 2; ++t) {
                mbar_init(&bar->q_full[t], 1); mbar_init(&bar->q_ready[t], kBlockM);
                mbar_init(&bar->s_full[t], 1); mbar_init(&bar->p_ready[t], kBlockM); mbar_init(&bar->o_done[t], 1);
            }
            for (int s = 0; s < kStages; ++s) { mbar_init(&bar->kv_full[s], 1); mbar_init(&bar->kv_empty[s], 1); }
            mbar_init(&bar->mma_done, 1);
            bar->abort_flag = 0;
            mbar_fence_init();
        }
        __syncwarp();
        tmem_alloc(&bar->tmem_base, 512);
        tmem_relinquish();
        tc_fence_before();
    } else if (warp == kProducerWarp && lane == 0) {
        tma_prefetch_desc(&maps.q); tma_prefetch_desc(&maps.k); tma_prefetch_desc(&maps.v);
    }
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bar->tmem_base;
    const WaitCtx abort_flag{&bar->abort_flag, p.status};

    if (warp == kProducerWarp) {
        // =========================== TMA producer ===========================
        if (lane == 0) {
            for (int t = 0; t < 2; ++t) {
                if (nblk[t] == 0) continue;
                mbar_arrive_expect_tx(&bar->q_full[t], C::kTileBytes);
                for (int h = 0; h < C::kHalves; ++h)
                    tma_load_4d(q_smem + t * C::kTileBytes + h * C::kHalfBytes, &maps.q, &bar->q_full[t], h * 64, r0[t], hq, b);
            }
            bool ok = true;
            for (int item = 0; item < 2 * nmax && ok; ++item) {     // item 2j = K_j, 2j+1 = V_j
                const int slot = item % kStages, j = item >> 1;
                if (item >= kStages) ok = mbar_wait(&bar->kv_empty[slot], ((item / kStages) - 1) & 1, abort_flag, 0x100 + item);
                if (!ok) break;
                mbar_arrive_expect_tx(&bar->kv_full[slot], C::kTileBytes);
                const CUtensorMap* m = (item & 1) ? &maps.v : &maps.k;
                for (int h = 0; h < C::kHalves; ++h)
                    tma_load_4d(kv_smem + slot * C::kTileBytes + h * C::kHalfBytes, m, &bar->kv_full[slot], h * 64, j * kBlockN, hkv, b);
            }
        }
    } else if (warp == kMmaWarp) {
        // =========================== MMA issuer ===========================
        if (lane == 0) {
            constexpr uint32_t idesc_qk = make_idesc_f16(Elem<T>::kFormat, 0, 0, kBlockM, kBlockN);
            constexpr uint32_t idesc_pv = make_idesc_f16(Elem<T>::kFormat, 0, 1, kBlockM, D);
            const uint32_t q_addr = smem_u32(q_smem), kv_addr = smem_u32(kv_smem);
            auto tmem_s = [&](int t) { return tmem_base + static_cast<uint32_t>(t * 128); };
            auto tmem_o = [&](int t) { return tmem_base + static_cast<uint32_t>(256 + t * 128); };
            auto issue_qk = [&](int t, int slot) {
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    uint32_t off = (kk >> 2) * C::kHalfBytes + (kk & 3) * 32;
                    uint64_t a = make_smem_desc_sw128(q_addr + t * C::kTileBytes + off, 16, 1024);
                    uint64_t bd = make_smem_desc_sw128(kv_addr + slot * C::kTileBytes + off, 16, 1024);
                    umma_ss(tmem_s(t), a, bd, idesc_qk, kk > 0 ? 1u : 0u);
                }
            };
            auto issue_pv = [&](int t, int slot, bool accumulate) {
#pragma unroll
                for (int kk = 0; kk < kBlockN / 16; ++kk) {
                    // V tile is MN-major for this product: 16 keys = 2048 bytes per step,
                    // second 64-column box one half-tile further (leading offset)
                    uint64_t bd = make_smem_desc_sw128(kv_addr + slot * C::kTileBytes + kk * 2048, C::kHalfBytes, 1024);
                    umma_ts(tmem_o(t), tmem_s(t) + kk * 8, bd, idesc_pv, (accumulate || kk > 0) ? 1u : 0u);
                }
            };
            bool ok = true;
            if (nmax > 0) {
                ok = mbar_wait(&bar->kv_full[0], 0, abort_flag, 0x200);
                for (int t = 0; t < 2 && ok; ++t) {
                    if (nblk[t] == 0) continue;
                    ok = mbar_wait(&bar->q_ready[t], 0, abort_flag, 0x210 + t);
                    if (!ok) break;
                    tc_fence_after();
                    issue_qk(t, 0);
                    umma_commit(&bar->s_full[t]);
                }
                if (ok) umma_commit(&bar->kv_empty[0]);
            }
            for (int j = 0; j < nmax && ok; ++j) {
                const int v_item = 2 * j + 1, k_item = 2 * j + 2;
                const int v_slot = v_item % kStages, k_slot = k_item % kStages;
                ok = mbar_wait(&bar->kv_full[v_slot], (v_item / kStages) & 1, abort_flag, 0x300 + j);
                bool k_ready = false;
                for (int t = 0; t < 2 && ok; ++t) {
                    if (j >= nblk[t]) continue;
                    ok = mbar_wait(&bar->p_ready[t], j & 1, abort_flag, 0x400 + 2 * j + t);
                    if (!ok) break;
                    tc_fence_after();
                    issue_pv(t, v_slot, j > 0);
                    umma_commit(&bar->o_done[t]);
                    if (j + 1 < nblk[t]) {
                        if (!k_ready) {
                            ok = mbar_wait(&bar->kv_full[k_slot], (k_item / kStages) & 1, abort_flag, 0x500 + j);
                            if (!ok) break;
                            tc_fence_after();
                            k_ready = true;
                        }
                        issue_qk(t, k_slot);
                        umma_commit(&bar->s_full[t]);
                    }
                }
                if (!ok) break;
                umma_commit(&bar->kv_empty[v_slot]);
                if (j + 1 < nmax) umma_commit(&bar->kv_empty[k_slot]);
            }
            // everything issued so far has to retire before TMEM is released
            umma_commit(&bar->mma_done);
            mbar_wait(&bar->mma_done, 0, abort_flag, 0x600);
        }
        __syncwarp();
    } else {
        // =========================== softmax / correction / epilogue ===========================
        const int t = warp >> 2;                     // tile of this warpgroup
        const int r = tid & 127;                     // row inside the tile = TMEM lane
        const int row = r0[t] + r;                   // query row in [0, T)
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t s_addr = tmem_base + lane_base + static_cast<uint32_t>(t * 128);
        const uint32_t o_addr = tmem_base + lane_base + static_cast<uint32_t>(256 + t * 128);
        const int n = nblk[t];
        bool ok = true;

        if (n > 0) {
            ok = mbar_wait_warp(&bar->q_full[t], 0, abort_flag, 0x700 + t);
            if (ok && p.q_rope_table != nullptr && row < p.T) {
                // rotate this thread's row of the swizzled Q tile in place
                const float2* tab = p.q_rope_table + static_cast<long long>(row) * (D / 2);
                unsigned char* qrow = q_smem + t * C::kTileBytes + r * 128;
#pragma unroll
                for (int c = 0; c < D / 8; ++c) {
                    uint4* ptr = reinterpret_cast<uint4*>(qrow + (c >> 3) * C::kHalfBytes + (((c & 7) ^ (r & 7)) << 4));
                    uint4 raw = *ptr;
                    uint32_t* u = &raw.x;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float2 x = Elem<T>::unpack2(u[i]);
                        float2 cs = __ldg(tab + c * 4 + i);
                        float t1 = __fmul_rn(x.x, cs.x), t2 = __fmul_rn(x.y, cs.y);
                        float t3 = __fmul_rn(x.x, cs.y), t4 = __fmul_rn(x.y, cs.x);
                        u[i] = Elem<T>::pack2(__fsub_rn(t1, t2), __fadd_rn(t3, t4));
                    }
                    *ptr = raw;
                }
                fence_proxy_async_smem();
            }
            mbar_arrive(&bar->q_ready[t]);
        }

        const float scale_log2 = p.scale * kLog2e;
        float m_ref = -INFINITY, l_sum = 0.f;

        for (int j = 0; j < n && ok; ++j) {
            ok = mbar_wait_warp(&bar->s_full[t], j & 1, abort_flag, 0x800 + 2 * j + t);
            if (!ok) break;
            tc_fence_after();
            uint32_t s[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_ld32(s_addr + c * 32, s[c]);
            tmem_ld_wait();

            const int k0 = j * kBlockN;
            const bool need_mask = (k0 + kBlockN > p.Skv) || (p.causal && (k0 + kBlockN - 1 > p.start_pos + r0[t]));
            if (need_mask) {
                const int limit = p.causal ? min(p.Skv - 1, p.start_pos + row) : p.Skv - 1;   // last visible key
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (k0 + c * 32 + i > limit) s[c][i] = 0xFF800000u;   // -inf
            }
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(s[c][i]));
            const float m_cand = mx * scale_log2;
            const bool grow = m_cand > m_ref + kRescaleThreshold;      // true on the first block
            if (__any_sync(0xFFFFFFFFu, grow)) {
                const float m_new = grow ? m_cand : m_ref;
                const float alpha = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - m_new);
                if (j > 0) {
                    // all PV products issued so far for this tile must have landed in O
                    ok = mbar_wait_warp(&bar->o_done[t], (j - 1) & 1, abort_flag, 0x900 + 2 * j + t);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int c = 0; c < D / 32; ++c) {
                        uint32_t o[32];
                        tmem_ld32(o_addr + c * 32, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st32(o_addr + c * 32, o);
                    }
                    tmem_st_wait();
                }
                l_sum *= alpha;
                m_ref = m_new;
            }
            // p = 2^(s*scale*log2e - m_ref); packed to 16 bit two per column
            float row_sum = 0.f;
            uint32_t pk[2][32];
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float p0 = fast_exp2(fmaf(__uint_as_float(s[c][i]), scale_log2, -m_ref));
                    float p1 = fast_exp2(fmaf(__uint_as_float(s[c][i + 1]), scale_log2, -m_ref));
                    row_sum += p0 + p1;
                    pk[c >> 1][(c & 1) * 16 + (i >> 1)] = Elem<T>::pack2(p0, p1);
                }
            l_sum += row_sum;
            tmem_st32(s_addr, pk[0]);
            tmem_st32(s_addr + 32, pk[1]);
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(&bar->p_ready[t]);
        }

        if (n > 0 && ok) {
            ok = mbar_wait_warp(&bar->o_done[t], (n - 1) & 1, abort_flag, 0xA00 + t);
            if (ok) {
                tc_fence_after();
                const float inv_l = 1.0f / l_sum;
                T* orow = static_cast<T*>(p.o.ptr) + b * p.o.sb + hq * p.o.sh + static_cast<long long>(row) * p.o.ss;
#pragma unroll
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t o[32];
                    tmem_ld32(o_addr + c * 32, o);
                    tmem_ld_wait();
                    if (row < p.T) {
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            uint4 out;
                            out.x = Elem<T>::pack2(__uint_as_float(o[8 * v + 0]) * inv_l, __uint_as_float(o[8 * v + 1]) * inv_l);
                            out.y = Elem<T>::pack2(__uint_as_float(o[8 * v + 2]) * inv_l, __uint_as_float(o[8 * v + 3]) * inv_l);
                            out.z = Elem<T>::pack2(__uint_as_float(o[8 * v + 4]) * inv_l, __uint_as_float(o[8 * v + 5]) * inv_l);
                            out.w = Elem<T>::pack2(__uint_as_float(o[8 * v + 6]) * inv_l, __uint_as_float(o[8 * v + 7]) * inv_l);
                            *reinterpret_cast<uint4*>(orow + c * 32 + v * 8) = out;
                        }
                    }
                }
                if (p.lse != nullptr && row < p.T)
                    p.lse[(static_cast<long long>(b) * p.Hq + hq) * p.T + row] = (m_ref + fast_log2(l_sum)) * kLn2;
            }
        }
    }

    // ---- teardown ----
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// ---- host side: tensor maps and launch ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess) return nullptr;
        if (qres != cudaDriverEntryPointSuccess) return nullptr;
        return reinterpret_cast<EncodeTiledFn>(ptr);
    }();
    return fn;
}

// [B,H,rows,D] view -> 4-D map (D, rows, H, B), box [64 cols][128 rows], 128-byte swizzle.
int make_map(CUtensorMap* m, int dtype, const View4& v, int rows, int H, int B, int D) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return set_detail(VB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(B)};
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(v.ss) * 2, static_cast<cuuint64_t>(v.sh) * 2, static_cast<cuuint64_t>(v.sb) * 2};
    // a dimension of extent 1 may carry any stride; keep it a legal multiple of 16
    for (int i = 0; i < 3; ++i) if (strides[i] == 0) strides[i] = 16;
    cuuint32_t box[4] = {64, 128, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(m, dtype == VB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                     v.ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        static thread_local char buf[96];
        snprintf(buf, sizeof(buf), "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
        return set_detail(VB200_ERR_CUDA, buf);
    }
    return VB200_OK;
}

template <typename T, int D>
int launch_t(cudaStream_t s, const PrefillParams& p) {
    TmaMaps maps;
    if (int rc = make_map(&maps.q, p.dtype, p.q, p.T, p.Hq, p.B, D)) return rc;
    if (int rc = make_map(&maps.k, p.dtype, p.k, p.Skv, p.Hkv, p.B, D)) return rc;
    if (int rc = make_map(&maps.v, p.dtype, p.v, p.Skv, p.Hkv, p.B, D)) return rc;
    static thread_local int configured_dev = -1;
    int dev = 0;
    VB200_CUDA_TRY(cudaGetDevice(&dev));
    if (configured_dev != dev) {
        VB200_CUDA_TRY(cudaFuncSetAttribute(prefill_sm100_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<D>::kSmemBytes));
        configured_dev = dev;
    }
    const int n_pairs = (p.T + 2 * kBlockM - 1) / (2 * kBlockM);
    dim3 grid(static_cast<unsigned>(n_pairs) * p.B * p.Hq);
    profile_mark_begin(s);
    prefill_sm100_kernel<T, D><<<grid, kThreads, Cfg<D>::kSmemBytes, s>>>(maps, p);
    profile_mark_end(s);
    note_launch();
    VB200_CUDA_TRY(cudaPeekAtLastError());
    return VB200_OK;
}

}  // namespace

int launch_prefill_sm100(cudaStream_t s, const PrefillParams& p) {
    if (p.D != 128 && p.D != 64) return set_detail(VB200_ERR_UNSUPPORTED, "bf16/fp16 attention supports head_dim 64 and 128");
    if (p.dtype == VB200_BF16) return p.D == 128 ? launch_t<__nv_bfloat16, 128>(s, p) : launch_t<__nv_bfloat16, 64>(s, p);
    if (p.dtype == VB200_F16) return p.D == 128 ? launch_t<__half, 128>(s, p) : launch_t<__half, 64>(s, p);
    return VB200_ERR_UNSUPPORTED;
}

}  // namespace vb200
