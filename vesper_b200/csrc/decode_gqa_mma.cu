// Split-KV decode for groups of 8 query heads per KV head (Hq / Hkv == 8).
//
// Same contract as decode_splitkv_kernel (grid (split, kv_head, batch), partial (O/l, m, l) per head
// into the workspace, RoPE of q / new k and the cache append fused in), but the two products run on
// the tensor cores with warp-level MMA: on CUDA cores an 8-head group needs 4 fp32 FMAs per KV byte
// and measured compute-bound at ~2.2 TB/s, a third of what HBM delivers; m16n8k16 MMAs (rows = the 8
// heads, zero padded to 16) make the kernel bandwidth-bound again.  As before every K / V row is
// fetched from HBM once per KV head.
//
//   S[head, key]  = Q[head, :] . K[key, :]      A = Q (registers, rotated, bf16/fp16), B = K rows (ldmatrix)
//   O[head, dim] += P[head, key] V[key, dim]    A = P (the S accumulators re-packed), B = V rows (ldmatrix.trans)
// A 64-key tile of K (and of V) arrives as two TMA boxes of [64 keys x 64 dims] with the 128-byte
// swizzle (4-D tensor maps over the cache views, no multicast); ldmatrix applies the same XOR to its row
// addresses, so the eight 16-byte rows of a phase fall into distinct banks.  (Row-by-row 256-byte bulk
// copies into padded rows were tried first: 2 M copies per step saturate the copy engine, 1.9 TB/s.)
#include "decode_exchange.cuh"

#include <cuda.h>
#include <cstdio>

namespace vb200 {

namespace {

constexpr int kTileM = 64;                 // keys per pipeline stage
constexpr int kBoxBytes = kTileM * 128;     // one [64 keys x 64 dims] box: rows of 128 bytes, 16-byte chunks XOR-swizzled by (row & 7)

struct KvMaps {
    CUtensorMap k, v;
};
constexpr float kLog2eM = 1.4426950408889634f;
constexpr float kLn2M = 0.6931471805599453f;
constexpr float kRescaleM = 8.0f;

template <typename T> struct MmaOp;
template <> struct MmaOp<__nv_bfloat16> {
    __device__ static void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};
template <> struct MmaOp<__half> {
    __device__ static void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

template <int CW, int kStages>
struct __align__(16) MmaSmem {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    int abort_flag;
    int pad[3];
};

// Per-warp running state, in MMA fragment layout: this thread owns head h = lane / 4 and, of every
// 8-wide column tile, columns (lane % 4) * 2 + {0, 1}.
struct FragState {
    float o[16][2];     // output accumulator: 16 dim tiles x 2 columns
    float m;            // running reference max of head h (log2 units)
    float l;            // this thread's share of the running sum of head h
};

// CW consumer warps (16 keys of every 64-key tile each) + 1 producer warp.
template <typename T, int NREP, int CW, int kStages, int MINB>
__global__ void __launch_bounds__((CW + 1) * 32, MINB) decode_gqa_mma_kernel(const __grid_constant__ KvMaps maps, DecodeParams p) {
    static_assert(CW * 16 == kTileM, "one 16-key slice per consumer warp");
    constexpr int D = 128;
    static_assert(NREP >= 1 && NREP <= 8, "the heads of a group are rows 0..NREP-1 of the 16-row MMA tile");
    constexpr int kRowBytes = D * 2;
    constexpr int kMatBytes = 2 * kBoxBytes;                 // one K or V tile = two boxes (dims 0-63, 64-127)
    constexpr int kStageBytes = 2 * kMatBytes;
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem_raw = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~static_cast<uintptr_t>(1023));
    float* newk = reinterpret_cast<float*>(smem_raw + kStages * kStageBytes);           // rotated new key, fp32 [128]
    T* newv = reinterpret_cast<T*>(smem_raw + kStages * kStageBytes + D * 4);           // new value [128]
    MmaSmem<CW, kStages>* sm = reinterpret_cast<MmaSmem<CW, kStages>*>(smem_raw + kStages * kStageBytes + D * 4 + kRowBytes);

    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // (nothing below depends on the previous kernel until the wait: the barriers and the tensor maps are set up while it drains)
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&sm->full[s], 1); mbar_init(&sm->empty[s], CW); }
        sm->abort_flag = 0;
        mbar_fence_init();
    } else if (tid == CW * 32) {
        tma_prefetch_desc(&maps.k);
        tma_prefetch_desc(&maps.v);
    }
    __syncthreads();
    asm volatile("griddepcontrol.wait;" ::: "memory");       // q / k_new / v_new / lengths may come from the previous kernel
    const StepLen sl = step_length(p, b);
    const int len = sl.len, total = sl.total;
    const int k_begin = split * p.chunk;
    if (split == 0 && kvh == 0 && threadIdx.x == 0) {
        reinterpret_cast<int*>(p.workspace)[b] = sl.header();
        if (sl.overflow) atomicCAS(p.status, 0, (2 << 24) | (b & 0xFFFFFF));
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (k_begin >= total) return;
    const int k_end = min(len, k_begin + p.chunk);
    const bool owns_new = sl.append && (len / p.chunk == split);
    const int ntiles = (k_end > k_begin) ? (k_end - k_begin + kTileM - 1) / kTileM : 0;

    const WaitCtx ctx{&sm->abort_flag, p.status};
    const T* kc = static_cast<const T*>(p.k_cache.ptr) + b * p.k_cache.sb + kvh * p.k_cache.sh;
    const T* vc = static_cast<const T*>(p.v_cache.ptr) + b * p.v_cache.sb + kvh * p.v_cache.sh;

    if (warp == CW) {
        // ---------------- producer: one lane issues four TMA boxes per tile ----------------
        if (lane == 0) {
            for (int t = 0; t < ntiles; ++t) {
                const int s = t % kStages;
                if (t >= kStages && !mbar_wait(&sm->empty[s], ((t / kStages) - 1) & 1, ctx, 0x18)) break;
                const int row0 = k_begin + t * kTileM;
                unsigned char* dst = smem_raw + s * kStageBytes;
                mbar_arrive_expect_tx(&sm->full[s], kStageBytes);         // rows past the cache capacity arrive as zeros and count too
                tma_load_4d(dst, &maps.k, &sm->full[s], 0, row0, kvh, b);
                tma_load_4d(dst + kBoxBytes, &maps.k, &sm->full[s], 64, row0, kvh, b);
                tma_load_4d(dst + kMatBytes, &maps.v, &sm->full[s], 0, row0, kvh, b);
                tma_load_4d(dst + kMatBytes + kBoxBytes, &maps.v, &sm->full[s], 64, row0, kvh, b);
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    const int hh = lane >> 2, cq = lane & 3;                 // head of this thread, column pair inside an 8-wide tile
    const float qscale = p.scale * kLog2eM;

    // rotated query in A-fragment layout: step ks covers dims [16 ks, 16 ks + 16); this thread holds the
    // pairs (16 ks + 2 cq, +1) and (16 ks + 8 + 2 cq, +1) of head hh -- a register is one RoPE pair
    uint32_t qa[8][2], qlo[8][2];      // q = hi + lo in the 16-bit type: the scores keep fp32-class accuracy in q
    const float pos = __int2float_rn(p.q_positions ? p.q_positions[b] : static_cast<int>(p.pos_offset) + len);
    {
        // The 16 angles a thread needs depend on cq only: the 8 threads that share cq compute two each
        // (thread hh: step ks = hh) and pass them round with shuffles.
        float my_cs[2] = {1.f, 1.f}, my_sn[2] = {0.f, 0.f};
        if (p.rope) {
#pragma unroll
            for (int half = 0; half < 2; ++half) sincosf(pos * p.inv_freq.v[hh * 8 + half * 4 + cq], &my_sn[half], &my_cs[half]);
        }
        const bool live = hh < NREP;                          // rows NREP..7 of the tile are padding as well
        const T* qp = static_cast<const T*>(p.q.ptr) + b * p.q.sb + (kvh * NREP + (live ? hh : 0)) * p.q.sh;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int d0 = ks * 16 + half * 8 + cq * 2;
                const float cs = __shfl_sync(0xFFFFFFFFu, my_cs[half], ks * 4 + cq);
                const float sn = __shfl_sync(0xFFFFFFFFu, my_sn[half], ks * 4 + cq);
                float2 t = Elem<T>::unpack2(*reinterpret_cast<const uint32_t*>(qp + d0));
                const float t1 = __fmul_rn(t.x, cs), t2 = __fmul_rn(t.y, sn), t3 = __fmul_rn(t.x, sn), t4 = __fmul_rn(t.y, cs);
                const float rx = __fsub_rn(t1, t2), ry = __fadd_rn(t3, t4);
                const uint32_t hi = Elem<T>::pack2(rx, ry);
                const float2 hf = Elem<T>::unpack2(hi);
                qa[ks][half] = live ? hi : 0u;
                qlo[ks][half] = live ? Elem<T>::pack2(rx - hf.x, ry - hf.y) : 0u;
            }
        }
    }

    // new token (one warp): rotate k, stage k (fp32) and v in shared memory, write the cache row
    if (owns_new && warp == 0 && lane < 16) {
        const int l16 = lane;
        const T* kn = static_cast<const T*>(p.k_new.ptr) + b * p.k_new.sb + kvh * p.k_new.sh + l16 * 8;
        const T* vn = static_cast<const T*>(p.v_new.ptr) + b * p.v_new.sb + kvh * p.v_new.sh + l16 * 8;
        uint4 kraw = *reinterpret_cast<const uint4*>(kn);
        const uint4 vraw = *reinterpret_cast<const uint4*>(vn);
        uint32_t* u = &kraw.x;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 t = Elem<T>::unpack2(u[i]);
            if (p.rope) {
                float sn, cs;
                sincosf(pos * p.inv_freq.v[l16 * 4 + i], &sn, &cs);
                const float t1 = __fmul_rn(t.x, cs), t2 = __fmul_rn(t.y, sn), t3 = __fmul_rn(t.x, sn), t4 = __fmul_rn(t.y, cs);
                t.x = __fsub_rn(t1, t2); t.y = __fadd_rn(t3, t4);
                u[i] = Elem<T>::pack2(t.x, t.y);
            }
            newk[l16 * 8 + 2 * i] = t.x;          // scored at full precision in this step; the cache gets the rounded row
            newk[l16 * 8 + 2 * i + 1] = t.y;
        }
        *reinterpret_cast<uint4*>(newv + l16 * 8) = vraw;
        // owns_new implies len < cache_cap (step_length refuses the append otherwise)
        *reinterpret_cast<uint4*>(const_cast<T*>(kc) + static_cast<long long>(len) * D + l16 * 8) = kraw;
        *reinterpret_cast<uint4*>(const_cast<T*>(vc) + static_cast<long long>(len) * D + l16 * 8) = vraw;
    }

    FragState st;
    st.m = -INFINITY; st.l = 0.f;
#pragma unroll
    for (int n = 0; n < 16; ++n) { st.o[n][0] = 0.f; st.o[n][1] = 0.f; }
    float pad0 = 0.f, pad1 = 0.f;                 // accumulators of the zero rows 8..15 (stay zero)

    const uint32_t smem_base = smem_u32(smem_raw);
    // ldmatrix lane addressing: lanes 8j..8j+7 supply the row addresses of matrix j
    const int lm_row = lane & 7, lm_mat = lane >> 3;
    for (int t = 0; t < ntiles; ++t) {
        const int s = t % kStages;
        if (!mbar_wait_warp(&sm->full[s], (t / kStages) & 1, ctx, 0x28)) break;
        const int nk = min(kTileM, k_end - (k_begin + t * kTileM));
        const int key0 = warp * 16;                           // this warp's 16-key slice of the tile
        if (key0 < nk) {
            const uint32_t ks_addr = smem_base + s * kStageBytes + key0 * 128;     // row key0 of the dims 0-63 box
            const uint32_t vs_addr = ks_addr + kMatBytes;
            if (key0 + 16 > nk) {
                // ragged last tile: rows past nk hold whatever the cache holds there; P is 0 for them but
                // 0 * NaN would poison O, so their V rows are cleared (a row is 128 bytes in each box)
                unsigned char* vrow = smem_raw + s * kStageBytes + kMatBytes;
                for (int i = lane; i < (key0 + 16 - nk) * 16; i += 32) {
                    const int r = nk + (i >> 4), c = i & 15;
                    *reinterpret_cast<uint4*>(vrow + (c >> 3) * kBoxBytes + r * 128 + (c & 7) * 16) = make_uint4(0, 0, 0, 0);
                }
                __syncwarp();
            }
            // ---- S = Q K^T for 16 keys: two 8-key column tiles ----
            float sc[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) { sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f; }
#pragma unroll
            for (int kp = 0; kp < 4; ++kp) {                  // 32 dims per ldmatrix.x4
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    uint32_t kb[4];
                    // matrices: (keys nt*8.., dims 32kp + 8 lm_mat ..)
                    ldmatrix_x4(kb, ks_addr + (kp >> 1) * kBoxBytes + (nt * 8 + lm_row) * 128 + ((((kp & 1) * 4 + lm_mat) ^ lm_row) << 4));
                    // rows 0-7 of the A tile carry the high halves of q, rows 8-15 (otherwise padding) the low
                    // halves: one MMA yields both partial scores, added below
                    const uint32_t a_lo[4] = {qa[2 * kp][0], qlo[2 * kp][0], qa[2 * kp][1], qlo[2 * kp][1]};
                    const uint32_t a_hi[4] = {qa[2 * kp + 1][0], qlo[2 * kp + 1][0], qa[2 * kp + 1][1], qlo[2 * kp + 1][1]};
                    MmaOp<T>::mma(sc[nt], a_lo, kb[0], kb[1]);
                    MmaOp<T>::mma(sc[nt], a_hi, kb[2], kb[3]);
                }
            }
            // ---- online softmax for head hh over this thread's 4 keys (and its 3 neighbours' 12) ----
            float sv[4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int key = key0 + nt * 8 + cq * 2 + j;
                    sv[nt * 2 + j] = key < nk ? (sc[nt][j] + sc[nt][j + 2]) * qscale : -INFINITY;
                }
            float bm = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
            bm = fmaxf(bm, __shfl_xor_sync(0xFFFFFFFFu, bm, 1));
            bm = fmaxf(bm, __shfl_xor_sync(0xFFFFFFFFu, bm, 2));
            if (bm > st.m + kRescaleM) {                      // uniform over the 4 lanes of a head
                const float alpha = (st.m == -INFINITY) ? 0.f : fast_exp2(st.m - bm);
                st.l *= alpha;
                st.m = bm;
#pragma unroll
                for (int n = 0; n < 16; ++n) { st.o[n][0] *= alpha; st.o[n][1] *= alpha; }
            }
            float pv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { pv[i] = (sv[i] == -INFINITY) ? 0.f : fast_exp2(sv[i] - st.m); st.l += pv[i]; }
            const uint32_t pa[4] = {Elem<T>::pack2(pv[0], pv[1]), 0u, Elem<T>::pack2(pv[2], pv[3]), 0u};
            // ---- O += P V: 16 dim tiles, two per ldmatrix.x4.trans ----
#pragma unroll
            for (int dp = 0; dp < 8; ++dp) {
                uint32_t vb[4];
                // matrices: (keys 8 (lm_mat & 1).., dims 16 dp + 8 (lm_mat >> 1) ..), transposed on load
                ldmatrix_x4_trans(vb, vs_addr + (dp >> 2) * kBoxBytes + ((lm_mat & 1) * 8 + lm_row) * 128 +
                                          ((((dp & 3) * 2 + (lm_mat >> 1)) ^ lm_row) << 4));
                float c0[4] = {st.o[2 * dp][0], st.o[2 * dp][1], pad0, pad1};
                MmaOp<T>::mma(c0, pa, vb[0], vb[1]);
                st.o[2 * dp][0] = c0[0]; st.o[2 * dp][1] = c0[1]; pad0 = c0[2]; pad1 = c0[3];
                float c1[4] = {st.o[2 * dp + 1][0], st.o[2 * dp + 1][1], pad0, pad1};
                MmaOp<T>::mma(c1, pa, vb[2], vb[3]);
                st.o[2 * dp + 1][0] = c1[0]; st.o[2 * dp + 1][1] = c1[1]; pad0 = c1[2]; pad1 = c1[3];
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm->empty[s]);
    }

    // ---- the new token (warp 0): scored in fp32 against the staged row ----
    if (owns_new && warp == 0) {
        __syncwarp();
        // dot of head hh: this thread covers dims cq*32 .. cq*32+31 of q (re-read, rotated again in fp32)
        const T* qp = static_cast<const T*>(p.q.ptr) + b * p.q.sb + (kvh * NREP + (hh < NREP ? hh : 0)) * p.q.sh + cq * 32;
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float2 t = Elem<T>::unpack2(*reinterpret_cast<const uint32_t*>(qp + 2 * i));
            const int d0 = cq * 32 + 2 * i;
            if (p.rope) {
                float sn, cs;
                sincosf(pos * p.inv_freq.v[d0 >> 1], &sn, &cs);
                const float t1 = __fmul_rn(t.x, cs), t2 = __fmul_rn(t.y, sn), t3 = __fmul_rn(t.x, sn), t4 = __fmul_rn(t.y, cs);
                t.x = __fsub_rn(t1, t2); t.y = __fadd_rn(t3, t4);
            }
            dot = fmaf(t.x, newk[d0], dot);
            dot = fmaf(t.y, newk[d0 + 1], dot);
        }
        dot += __shfl_xor_sync(0xFFFFFFFFu, dot, 1);
        dot += __shfl_xor_sync(0xFFFFFFFFu, dot, 2);
        const float s_new = dot * qscale;
        if (s_new > st.m + kRescaleM) {
            const float alpha = (st.m == -INFINITY) ? 0.f : fast_exp2(st.m - s_new);
            st.l *= alpha;
            st.m = s_new;
#pragma unroll
            for (int n = 0; n < 16; ++n) { st.o[n][0] *= alpha; st.o[n][1] *= alpha; }
        }
        const float pn = fast_exp2(s_new - st.m);
        if (cq == 0) st.l += pn;                              // once per head
#pragma unroll
        for (int n = 0; n < 16; ++n) {
            const float2 v2 = Elem<T>::unpack2(*reinterpret_cast<const uint32_t*>(newv + n * 8 + cq * 2));
            st.o[n][0] = fmaf(pn, v2.x, st.o[n][0]);
            st.o[n][1] = fmaf(pn, v2.y, st.o[n][1]);
        }
    }

    // ---- merge the CW warps through shared memory (the ring is free once every consumer is here) ----
    float l = st.l;
    l += __shfl_xor_sync(0xFFFFFFFFu, l, 1);
    l += __shfl_xor_sync(0xFFFFFFFFu, l, 2);
    asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
    float* go = reinterpret_cast<float*>(smem_raw);           // [CW][NREP][128]
    float* gm = go + CW * NREP * 128;                         // [CW][NREP]
    float* gl = gm + CW * NREP;                               // [CW][NREP]
    if (hh < NREP) {
        if (cq == 0) { gm[warp * NREP + hh] = st.m; gl[warp * NREP + hh] = l; }
#pragma unroll
        for (int n = 0; n < 16; ++n)
            *reinterpret_cast<float2*>(go + (warp * NREP + hh) * 128 + n * 8 + cq * 2) = make_float2(st.o[n][0], st.o[n][1]);
    }
    asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
    if (tid < 128) {
        const int d = tid;
        float* wsp = p.workspace + p.ws_header;
#pragma unroll
        for (int h = 0; h < NREP; ++h) {
            float M = -INFINITY;
#pragma unroll
            for (int g = 0; g < CW; ++g) M = fmaxf(M, gm[g * NREP + h]);
            float L = 0.f, acc = 0.f;
#pragma unroll
            for (int g = 0; g < CW; ++g) {
                const float mg = gm[g * NREP + h];
                const float w = (mg == -INFINITY) ? 0.f : fast_exp2(mg - M);
                L += gl[g * NREP + h] * w;
                acc += go[(g * NREP + h) * 128 + d] * w;
            }
            float* out = wsp + ((static_cast<long long>(b) * p.Hkv + kvh) * p.num_splits + split) * NREP * (D + 2) + h * (D + 2);
            out[d] = acc / L;
            if (d == 0) { out[D] = M * kLn2M; out[D + 1] = L; }
        }
    }
    if (!p.fused_exchange) return;

    // ---- sequence-sharded decode in one launch: the CTA that delivers the LAST split of this (batch, kv_head) merges
    // the group's splits and exchanges the merged records with the other ranks (128 consumer threads; the producer
    // warp has left) ----
    float* rec = reinterpret_cast<float*>(smem_raw);          // [NREP][D + 2]: this rank's merged (O/l, m, l) per head
    __shared__ int s_last;
    __shared__ uint32_t s_step;
    __shared__ int s_ok;
    const int unit = b * p.Hkv + kvh;
    const int nvalid = min((total + p.chunk - 1) / p.chunk, p.num_splits);
    // every thread's rows, then (cumulatively, through the CTA barrier) one thread's fence, before the ticket
    asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
    if (tid == 0) {
        __threadfence();
        int* ticket = reinterpret_cast<int*>(static_cast<char*>(p.xchg.peers[p.xchg.rank]) + kXTicketBase) + unit;
        const int t = atomicAdd(ticket, 1);
        s_last = (t == nvalid - 1) ? 1 : 0;
        if (s_last) *ticket = 0;                              // every split has delivered: ready for the next call
    }
    asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
    if (!s_last) return;
    __threadfence();
    constexpr int kRec2 = (D + 2) / 2, kBlk2 = NREP * kRec2, kNT = CW * 32;
    constexpr int kRingBytes = kStages * kStageBytes;
    constexpr int kRecBytes = NREP * (D + 2) * 4, kMiscBytes = 128;
    // splits staged per round: their records (kBlk2 float2 each) and one weight per (head, split) must fit behind rec
    constexpr int kStageCap = ((kRingBytes - kRecBytes - kMiscBytes) / (kBlk2 * 8 + NREP * 4)) & ~3;
    static_assert(kStageCap >= 8 && (NREP * kStageCap * 4) % 16 == 0 && kRecBytes % 16 == 0, "staging layout");
    float* sm_run = rec + NREP * (D + 2);                     // [0,8) running max, [8,16) running sum, [16,24) rescale factor per head
    float* sm_w = sm_run + kMiscBytes / 4;                    // [NREP][kStageCap] merge weights of the staged splits
    float2* stage2 = reinterpret_cast<float2*>(sm_w + NREP * kStageCap);
    {
        // Merge of the group's splits by all 128 threads.  A split's records of the NREP heads are one contiguous
        // block of NREP * (D + 2) floats, viewed as float2 columns: column h * 65 + i (i < 64) holds dims 2i, 2i + 1
        // of head h, column h * 65 + 64 its (m, l).  The rows come from L2, written by other CTAs, at a time when the
        // other groups still stream their keys: a dependent round of loads costs ~2500 cycles, so the records of as many
        // splits as fit (all of them, for the split counts this path plans) are brought into the now idle K/V ring
        // by 16-byte asynchronous copies -- no registers held, every copy in flight at once -- and merged from there;
        // further rounds fold in with the usual rescale.
        constexpr int kCols = (kBlk2 + kNT - 1) / kNT;
        const float2* grp2 = reinterpret_cast<const float2*>(p.workspace + p.ws_header + (static_cast<long long>(unit) * p.num_splits) * NREP * (D + 2));
        float2 acc[kCols];
        int col[kCols], head[kCols];
#pragma unroll
        for (int k = 0; k < kCols; ++k) {
            acc[k] = make_float2(0.f, 0.f);
            const int c = tid + k * kNT;
            const bool use = c < kBlk2 && (c % kRec2) != D / 2;
            col[k] = use ? c : -1;
            head[k] = use ? c / kRec2 : 0;
        }
        if (tid < NREP) { sm_run[tid] = -INFINITY; sm_run[8 + tid] = 0.f; }
        const uint32_t stage_addr = smem_u32(stage2);
        for (int s0 = 0; s0 < nvalid; s0 += kStageCap) {
            const int n = min(kStageCap, nvalid - s0);
            const float4* src4 = reinterpret_cast<const float4*>(grp2 + static_cast<long long>(s0) * kBlk2);
            for (int i = tid; i < n * (kBlk2 / 2); i += kNT)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(stage_addr + i * 16), "l"(src4 + i) : "memory");
            asm volatile("cp.async.wait_all;" ::: "memory");
            asm volatile("bar.sync 1, %0;" ::"n"(kNT) : "memory");
            for (int h = warp; h < NREP; h += CW) {
                float Mc = -INFINITY;
                for (int u = lane; u < n; u += 32) Mc = fmaxf(Mc, stage2[u * kBlk2 + h * kRec2 + D / 2].x);
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) Mc = fmaxf(Mc, __shfl_xor_sync(0xFFFFFFFFu, Mc, o));
                const float Mold = sm_run[h], Mnew = fmaxf(Mold, Mc);
                float Lc = 0.f;
                for (int u = lane; u < n; u += 32) {
                    const float2 ml = stage2[u * kBlk2 + h * kRec2 + D / 2];
                    const float wgt = (ml.x == -INFINITY) ? 0.f : expf(ml.x - Mnew) * ml.y;
                    sm_w[h * kStageCap + u] = wgt;
                    Lc += wgt;
                }
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) Lc += __shfl_xor_sync(0xFFFFFFFFu, Lc, o);
                __syncwarp();
                if (lane == 0) {
                    const float keep = (Mold == -INFINITY) ? 0.f : expf(Mold - Mnew);
                    sm_run[16 + h] = keep;
                    sm_run[8 + h] = sm_run[8 + h] * keep + Lc;
                    sm_run[h] = Mnew;
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kNT) : "memory");
#pragma unroll
            for (int k = 0; k < kCols; ++k) {
                const float keep = sm_run[16 + head[k]];
                acc[k].x *= keep; acc[k].y *= keep;
            }
            for (int u = 0; u < n; ++u) {
#pragma unroll
                for (int k = 0; k < kCols; ++k)
                    if (col[k] >= 0) {
                        const float wgt = sm_w[head[k] * kStageCap + u];
                        const float2 v = stage2[u * kBlk2 + col[k]];
                        acc[k].x += wgt * v.x;
                        acc[k].y += wgt * v.y;
                    }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kNT) : "memory");      // the round is consumed before the next one lands
        }
#pragma unroll
        for (int k = 0; k < kCols; ++k)
            if (col[k] >= 0) {
                const float L = sm_run[8 + head[k]];
                const float inv = L > 0.f ? 1.0f / L : 0.f;
                reinterpret_cast<float2*>(rec)[col[k]] = make_float2(acc[k].x * inv, acc[k].y * inv);
            }
        if (tid < NREP) { rec[tid * (D + 2) + D] = sm_run[tid]; rec[tid * (D + 2) + D + 1] = sm_run[8 + tid]; }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
    const long long r0 = static_cast<long long>(b) * p.Hq + static_cast<long long>(kvh) * NREP;
    // (the staging area is free again: the peers' rows of this group land there for the final merge)
    exchange_rows<T, CW * 32>(p.xchg, unit, r0, r0 + NREP, rec, tid, &s_step, &s_ok,
                              [] { asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory"); },
                              reinterpret_cast<float*>(stage2), kStageCap * kBlk2 * 2, 0x80000000u);
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn kv_encode_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess) return nullptr;
        if (qres != cudaDriverEntryPointSuccess) return nullptr;
        return reinterpret_cast<EncodeTiledFn>(ptr);
    }();
    return fn;
}

// [B,Hkv,cap,128] cache view -> 4-D map (D, rows, Hkv, B), box [64 dims][64 rows], 128-byte swizzle.
int make_kv_map(CUtensorMap* m, int dtype, const View4& v, int rows, int H, int B) {
    EncodeTiledFn enc = kv_encode_fn();
    if (!enc) return set_detail(VB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[4] = {128, static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(B)};
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(v.ss) * 2, static_cast<cuuint64_t>(v.sh) * 2, static_cast<cuuint64_t>(v.sb) * 2};
    for (int i = 0; i < 3; ++i) if (strides[i] == 0) strides[i] = 16;
    cuuint32_t box[4] = {64, kTileM, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(m, dtype == VB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, v.ptr, dims, strides,
                     box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        static thread_local char buf[96];
        snprintf(buf, sizeof(buf), "cuTensorMapEncodeTiled (decode) failed with CUresult %d", static_cast<int>(r));
        return set_detail(VB200_ERR_CUDA, buf);
    }
    return VB200_OK;
}

}  // namespace

// Launches the split kernel; the caller follows with the common combine kernel.
template <typename T, int NREP>
int launch_decode_gqa_mma_split(cudaStream_t s, const DecodeParams& p) {
    constexpr int CW = 4, kStages = 3, MINB = 2;
    constexpr size_t smem = static_cast<size_t>(kStages) * 4 * kBoxBytes + 128 * 4 + 128 * 2 + sizeof(MmaSmem<CW, kStages>) + 1024;
    static_assert(CW * NREP * 128 * 4 + 2 * CW * NREP * 4 <= kStages * 4 * kBoxBytes, "merge buffers must fit in the ring");
    // the maps of this thread's last call, reused while the cache views are unchanged (a decode loop calls with the same
    // caches step after step)
    struct Key {
        int dtype, cap, Hkv, B;
        View4 k, v;
        bool operator==(const Key& x) const {
            auto same = [](const View4& a, const View4& b) { return a.ptr == b.ptr && a.sb == b.sb && a.sh == b.sh && a.ss == b.ss; };
            return dtype == x.dtype && cap == x.cap && Hkv == x.Hkv && B == x.B && same(k, x.k) && same(v, x.v);
        }
    };
    static thread_local Key cached_key{};
    static thread_local KvMaps maps;
    static thread_local bool cached_valid = false;
    const Key key{p.dtype, p.cache_cap, p.Hkv, p.B, p.k_cache, p.v_cache};
    if (!cached_valid || !(cached_key == key)) {
        cached_valid = false;
        if (int rc = make_kv_map(&maps.k, p.dtype, p.k_cache, p.cache_cap, p.Hkv, p.B)) return rc;
        if (int rc = make_kv_map(&maps.v, p.dtype, p.v_cache, p.cache_cap, p.Hkv, p.B)) return rc;
        cached_key = key;
        cached_valid = true;
    }
    auto kernel = decode_gqa_mma_kernel<T, NREP, CW, kStages, MINB>;
    static thread_local bool configured[64] = {};      // per device ordinal: the attribute belongs to the device's context
    int dev = 0;
    VB200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return set_detail(VB200_ERR_NO_DEVICE, "device ordinal out of range");
    if (!configured[dev]) {
        VB200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(p.num_splits, p.Hkv, p.B);
    cfg.blockDim = dim3((CW + 1) * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    VB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, maps, p));
    return VB200_OK;
}
template int launch_decode_gqa_mma_split<__nv_bfloat16, 8>(cudaStream_t, const DecodeParams&);
template int launch_decode_gqa_mma_split<__half, 8>(cudaStream_t, const DecodeParams&);
template int launch_decode_gqa_mma_split<__nv_bfloat16, 4>(cudaStream_t, const DecodeParams&);
template int launch_decode_gqa_mma_split<__half, 4>(cudaStream_t, const DecodeParams&);

}  // namespace vb200

