// bf16 / fp16 attention forward for sm_100a: TMA-staged Q/K/V tiles,
// tcgen05.mma with TMEM accumulators for S = Q K^T and O = P V, online softmax
// in registers (one thread per query row), causal block skipping, GQA by
// head-group indexing, RoPE of the Q tiles fused in (rotated in shared memory
// by two otherwise idle warps while the previous work item computes).
//
// Math (same as flash_attention_cpu_dispatch, src/ops/flash_attention.cpp:218-364):
//   s_ij = scale * q_i . k_j ;  key j visible to query i iff j <= start_pos + i
//   O_i = sum_j softmax_j(s_ij) v_j ;  LSE_i = ln sum_j exp(s_ij)
//
// Persistent kernel, one CTA per SM.  A work item is two adjacent 128-row
// query tiles of one (batch, q_head), processed ping-pong so the tensor pipe
// works on one tile while the other is in softmax.  Items are sorted by work
// (last query rows first) and dealt to the CTAs in snake order.
//   warps 0-3    softmax / correction / epilogue of tile 0   (TMEM lanes 0..127)
//   warps 4-7    the same for tile 1
//   warp  8      TMA producer: Q tiles (3 rotating buffers, so the next item's
//                tiles load while this one computes) and the K/V ring (4 slots)
//   warp  9      tcgen05.mma issuer, TMEM owner
//   warps 10-11  RoPE of freshly loaded Q tiles, in place in swizzled smem
// TMEM (512 columns): S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [384,384+D);
// P (16-bit, packed two per column) overwrites the first 64 columns of its S.
//
// Every wait is bounded (see mbar_wait); on expiry the CTA drains and returns
// with the device status word set.
#include <cstdio>
#include <cstdlib>

#include "kernels.h"

namespace vb200 {

namespace {

constexpr int kBlockM = 128;
constexpr int kBlockN = 128;
constexpr int kStages = 4;        // K/V ring slots
constexpr int kQBufs = 3;         // rotating Q tile buffers
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kRopeWarp0 = 10;    // warps 10, 11
constexpr int kRopeThreads = 64;
constexpr int kThreads = 384;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;
constexpr int kEpiBatch = 2;         // TMEM loads (32 columns each) in flight per wait in the epilogue

// Register split after setmaxnreg: the two softmax warpgroups (one thread per row holds a 128-column score tile)
// take 216 registers per thread, the producer / MMA / RoPE warpgroup 72.
constexpr int kRegSoftmax = 216, kRegOther = 72;
static_assert(kRegSoftmax * 256 + kRegOther * 128 <= 168 * 384, "register budget");

struct __align__(8) Barriers {
    uint64_t q_full[kQBufs], q_rot[kQBufs], q_free[kQBufs];
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
    static constexpr int kSmemBytes = (kQBufs + kStages) * kTileBytes + 1024 /*alignment slack*/ + 256 /*Barriers*/;
};

// One unit of work: two 128-row query tiles that read the same K/V blocks.  With an even number of
// query heads per KV head the two tiles are the SAME rows of two heads of one group: both visit the
// same number of key blocks, so neither softmax warpgroup idles in the last iteration (adjacent row
// tiles of one head differ by one block: 8 of 72 iterations per head wasted at S = 2048).  Otherwise
// (one query head per KV head) they are two adjacent row tiles of one head.
struct Item {
    int b, hq, hq1, hkv;   // hq / hq1: head of tile 0 / tile 1
    int r0[2];      // first query row of each tile
    int nblk[2];    // key blocks each tile visits (0: tile not present)
    int nmax;
};

__host__ __device__ __forceinline__ bool pair_by_heads(const PrefillParams& p) {
    return (p.Hq / p.Hkv) % 2 == 0;
}
// number of (batch, head or head pair) columns and of row steps of the item grid
__host__ __device__ __forceinline__ int item_cols(const PrefillParams& p) { return pair_by_heads(p) ? p.B * (p.Hq / 2) : p.B * p.Hq; }
__host__ __device__ __forceinline__ int item_rows(const PrefillParams& p) {
    return pair_by_heads(p) ? (p.T + kBlockM - 1) / kBlockM : (p.T + 2 * kBlockM - 1) / (2 * kBlockM);
}

__device__ __forceinline__ Item get_item(const PrefillParams& p, int it, int n_bh, int n_pairs) {
    Item w;
    const int pair = n_pairs - 1 - it / n_bh;      // heaviest (last) query rows first
    const int bh = it % n_bh;
    const bool by_heads = pair_by_heads(p);
    if (by_heads) {
        w.b = bh / (p.Hq / 2);
        w.hq = 2 * (bh % (p.Hq / 2));
        w.hq1 = w.hq + 1;
    } else {
        w.b = bh / p.Hq;
        w.hq = bh % p.Hq;
        w.hq1 = w.hq;
    }
    w.hkv = w.hq / (p.Hq / p.Hkv);
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        w.r0[t] = by_heads ? pair * kBlockM : (2 * pair + t) * kBlockM;
        if (w.r0[t] >= p.T) { w.nblk[t] = 0; continue; }
        int kv_end = p.Skv;
        if (p.causal) kv_end = min(p.Skv, p.start_pos + min(w.r0[t] + kBlockM, p.T));
        w.nblk[t] = (kv_end + kBlockN - 1) / kBlockN;
    }
    w.nmax = max(w.nblk[0], w.nblk[1]);
    return w;
}

// Snake dealing of the sorted items: round r gives CTA c item r*G + c (even r)
// or r*G + G-1-c (odd r), which evens out the per-CTA totals.  -1: none.
__device__ __forceinline__ int item_of_round(int round, int n_items) {
    const int G = gridDim.x, c = blockIdx.x;
    const int idx = round * G + ((round & 1) ? (G - 1 - c) : c);
    return idx < n_items ? idx : -1;
}

template <int N> __device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

// kExactRope selects how the RoPE warps get a query row's angles: false = table seed every kRopeSeed
// steps + angle-addition recurrence (prompts whose last position is <= 16384), true = every row from
// the table.  A template parameter, not a run-time branch: the extra loop in one kernel body changed
// the register allocation of the whole kernel and cost the common case 5-8 %.
template <typename T, int D, bool kExactRope>
__global__ void __launch_bounds__(kThreads, 1)
prefill_sm100_kernel(const __grid_constant__ TmaMaps maps, PrefillParams p) {
    using C = Cfg<D>;
    extern __shared__ unsigned char smem_dyn[];
    // 128B-swizzled tiles need 1024-byte alignment
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    unsigned char* q_smem = smem;                                   // kQBufs tiles
    unsigned char* kv_smem = smem + kQBufs * C::kTileBytes;         // kStages tiles
    Barriers* bar = reinterpret_cast<Barriers*>(smem + (kQBufs + kStages) * C::kTileBytes);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_bh = item_cols(p);
    const int n_pairs = item_rows(p);
    const int n_items = n_bh * n_pairs;
    const int n_rounds = (n_items + gridDim.x - 1) / gridDim.x;
    const bool rope = p.q_rope_table != nullptr;

    // ---- setup ----
    if (warp == kMmaWarp) {
        if (lane == 0) {
            for (int b = 0; b < kQBufs; ++b) {
                mbar_init(&bar->q_full[b], 1); mbar_init(&bar->q_rot[b], kRopeThreads); mbar_init(&bar->q_free[b], 1);
            }
            for (int t = 0; t < 2; ++t) {
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

    if (warp >= 8) {
        // the data-movement / issue / RoPE warpgroup needs few registers; the softmax warpgroups take them
        reg_dec<kRegOther>();
        if (warp == kProducerWarp) {
            // =========================== TMA producer ===========================
            if (lane == 0) {
                int kv_item = 0;                 // running index into the K/V ring over all work items
                int q_seq = 0;                   // running index of Q tiles -> buffer q_seq % 3
                bool ok = true;
                auto load_q = [&](const Item& w, int t) {
                    if (w.nblk[t] == 0 || !ok) return;
                    const int b = q_seq % kQBufs, use = q_seq / kQBufs;
                    // the tile that used this buffer before must have had its last QK issued and retired
                    if (use > 0) ok = mbar_wait(&bar->q_free[b], (use - 1) & 1, abort_flag, 0x110 + b);
                    if (!ok) return;
                    ++q_seq;
                    mbar_arrive_expect_tx(&bar->q_full[b], C::kTileBytes);
#pragma unroll
                    for (int h = 0; h < C::kHalves; ++h)
                        tma_load_4d(q_smem + b * C::kTileBytes + h * C::kHalfBytes, &maps.q, &bar->q_full[b], h * 64, w.r0[t], t ? w.hq1 : w.hq, w.b);
                };
                int round = 0;
                int idx = -1;
                while (round < n_rounds && (idx = item_of_round(round, n_items)) < 0) ++round;
                Item w;
                if (idx >= 0) { w = get_item(p, idx, n_bh, n_pairs); load_q(w, 0); load_q(w, 1); }
                while (idx >= 0 && ok) {
                    // look one item ahead so its first Q tile streams in (and gets rotated) during this item
                    int round2 = round + 1, idx2 = -1;
                    while (round2 < n_rounds && (idx2 = item_of_round(round2, n_items)) < 0) ++round2;
                    Item wn;
                    if (idx2 >= 0) { wn = get_item(p, idx2, n_bh, n_pairs); load_q(wn, 0); }
                    for (int x = 0; x < 2 * w.nmax && ok; ++x, ++kv_item) {     // x = 2j: K_j, 2j+1: V_j
                        const int slot = kv_item % kStages;
                        if (kv_item >= kStages) ok = mbar_wait(&bar->kv_empty[slot], ((kv_item / kStages) - 1) & 1, abort_flag, 0x100);
                        if (!ok) break;
                        mbar_arrive_expect_tx(&bar->kv_full[slot], C::kTileBytes);
                        const CUtensorMap* m = (x & 1) ? &maps.v : &maps.k;
#pragma unroll
                        for (int h = 0; h < C::kHalves; ++h)
                            tma_load_4d(kv_smem + slot * C::kTileBytes + h * C::kHalfBytes, m, &bar->kv_full[slot], h * 64, (x >> 1) * kBlockN, w.hkv, w.b);
                    }
                    // the second tile of the next item reuses the buffer this item's first tile frees
                    if (idx2 >= 0) load_q(wn, 1);
                    idx = idx2; round = round2; w = wn;
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
                auto issue_qk = [&](int t, int qbuf, int slot) {
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        uint32_t off = (kk >> 2) * C::kHalfBytes + (kk & 3) * 32;
                        uint64_t a = make_smem_desc_sw128(q_addr + qbuf * C::kTileBytes + off, 16, 1024);
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
                int kv_item = 0, q_seq = 0;
                int blk0 = 0, blk1 = 0;          // running count of score tiles per query tile (barrier phases)
                bool ok = true;
                for (int round = 0; round < n_rounds && ok; ++round) {
                    const int idx = item_of_round(round, n_items);
                    if (idx < 0) continue;
                    const Item w = get_item(p, idx, n_bh, n_pairs);
                    int qbuf[2] = {0, 0};
                    const int k0_slot = kv_item % kStages;
                    ok = mbar_wait(&bar->kv_full[k0_slot], (kv_item / kStages) & 1, abort_flag, 0x200);
#pragma unroll
                    for (int t = 0; t < 2; ++t) {
                        if (w.nblk[t] == 0 || !ok) continue;
                        qbuf[t] = q_seq % kQBufs;
                        const int ph = (q_seq / kQBufs) & 1;
                        ++q_seq;
                        // S of this tile is free: every PV of the previous item was issued before this point
                        ok = mbar_wait(rope ? &bar->q_rot[qbuf[t]] : &bar->q_full[qbuf[t]], ph, abort_flag, 0x210 + t);
                        if (!ok) continue;
                        tc_fence_after();
                        issue_qk(t, qbuf[t], k0_slot);
                        umma_commit(&bar->s_full[t]);
                        if (w.nblk[t] == 1) umma_commit(&bar->q_free[qbuf[t]]);
                    }
                    if (!ok) break;
                    umma_commit(&bar->kv_empty[k0_slot]);
                    for (int j = 0; j < w.nmax && ok; ++j) {
                        const int v_item = kv_item + 2 * j + 1, k_item = kv_item + 2 * j + 2;
                        const int v_slot = v_item % kStages, k_slot = k_item % kStages;
                        ok = mbar_wait(&bar->kv_full[v_slot], (v_item / kStages) & 1, abort_flag, 0x300);
                        bool k_ready = false;
#pragma unroll
                        for (int t = 0; t < 2; ++t) {
                            if (j >= w.nblk[t] || !ok) continue;
                            int& blk = t ? blk1 : blk0;
                            ok = mbar_wait(&bar->p_ready[t], blk & 1, abort_flag, 0x400 + t);
                            if (!ok) continue;
                            ++blk;
                            tc_fence_after();
                            issue_pv(t, v_slot, j > 0);
                            umma_commit(&bar->o_done[t]);
                            if (j + 1 < w.nblk[t]) {
                                if (!k_ready) {
                                    ok = mbar_wait(&bar->kv_full[k_slot], (k_item / kStages) & 1, abort_flag, 0x500);
                                    if (!ok) continue;
                                    tc_fence_after();
                                    k_ready = true;
                                }
                                issue_qk(t, qbuf[t], k_slot);
                                umma_commit(&bar->s_full[t]);
                                if (j + 2 == w.nblk[t]) umma_commit(&bar->q_free[qbuf[t]]);   // last QK of this tile
                            }
                        }
                        if (!ok) break;
                        umma_commit(&bar->kv_empty[v_slot]);
                        if (j + 1 < w.nmax) umma_commit(&bar->kv_empty[k_slot]);
                    }
                    kv_item += 2 * w.nmax;
                }
                // everything issued so far has to retire before TMEM is released
                umma_commit(&bar->mma_done);
                mbar_wait(&bar->mma_done, 0, abort_flag, 0x600);
            }
            __syncwarp();
        } else if (rope) {
            // =========================== RoPE of the Q tiles ===========================
            // 2 warps; warp w owns rows [64w, 64w+64) of each tile.  A step handles two rows: lane l
            // takes 16-byte chunk (l & 15) of row 2*step + (l >> 4), so the (cos,sin) table reads of a
            // warp are two contiguous 512-byte rows and the swizzled smem accesses are conflict-free.
            const int rw = warp - kRopeWarp0;
            const int c = lane & 15;                          // 16-byte chunk of the row (D = 128: 16 chunks)
            constexpr int kRopeSeed = 8;                      // steps (of two rows) between exact table reads
            float step_c[4], step_s[4];                       // rotation by two positions for this lane's 4 pairs
#pragma unroll
            for (int e = 0; e < 4; ++e) sincosf(2.0f * p.inv_freq.v[(c * 4 + e) & (kMaxHalfDim - 1)], &step_s[e], &step_c[e]);
            int q_seq = 0;
            bool ok = true;
            for (int round = 0; round < n_rounds && ok; ++round) {
                const int idx = item_of_round(round, n_items);
                if (idx < 0) continue;
                const Item w = get_item(p, idx, n_bh, n_pairs);
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    if (w.nblk[t] == 0 || !ok) continue;
                    const int b = q_seq % kQBufs, ph = (q_seq / kQBufs) & 1;
                    ++q_seq;
                    ok = mbar_wait_warp(&bar->q_full[b], ph, abort_flag, 0x700 + b);
                    if (!ok) continue;
                    if (c < D / 8) {
                        unsigned char* qtile = q_smem + b * C::kTileBytes + (c >> 3) * C::kHalfBytes;
                        // A lane walks rows r, r+2, r+4, ... of its chunk.  The (cos,sin) of a row come from
                        // the exact table every kRopeSeed steps and from a rotation by 2*f in between
                        // (angle-addition recurrence), which cuts the table traffic by kRopeSeed.
                        const int r_first = rw * 64 + (lane >> 4);
                        float4 seed0, seed1;
                        {
                            const int row = min(w.r0[t] + r_first, p.T - 1);
                            const float4* tab = reinterpret_cast<const float4*>(p.q_rope_table + static_cast<long long>(row) * (D / 2)) + c * 2;
                            seed0 = __ldg(tab); seed1 = __ldg(tab + 1);
                        }
                        if constexpr (kExactRope) {
                            // far positions: the reference's fp32 angle pos*f is itself rounded to ~6e-8*pos,
                            // which the recurrence does not reproduce -- every row reads the table there
#pragma unroll 2
                            for (int st = 0; st < 32; ++st) {
                                const int r = r_first + 2 * st;
                                const int rowx = min(w.r0[t] + r, p.T - 1);
                                const float4* tabx = reinterpret_cast<const float4*>(p.q_rope_table + static_cast<long long>(rowx) * (D / 2)) + c * 2;
                                const float4 a0 = __ldg(tabx), a1 = __ldg(tabx + 1);
                                const float csx[4] = {a0.x, a0.z, a1.x, a1.z}, snx[4] = {a0.y, a0.w, a1.y, a1.w};
                                uint4* ptr = reinterpret_cast<uint4*>(qtile + r * 128 + (((c & 7) ^ (r & 7)) << 4));
                                uint4 raw = *ptr;
                                uint32_t* u = &raw.x;
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    float2 x = Elem<T>::unpack2(u[e]);
                                    float t1 = __fmul_rn(x.x, csx[e]), t2 = __fmul_rn(x.y, snx[e]);
                                    float t3 = __fmul_rn(x.x, snx[e]), t4 = __fmul_rn(x.y, csx[e]);
                                    u[e] = Elem<T>::pack2(__fsub_rn(t1, t2), __fadd_rn(t3, t4));
                                }
                                *ptr = raw;
                            }
                        } else
#pragma unroll 1
                        for (int s0 = 0; s0 < 32; s0 += kRopeSeed) {
                            float cs[4] = {seed0.x, seed0.z, seed1.x, seed1.z};
                            float sn[4] = {seed0.y, seed0.w, seed1.y, seed1.w};
                            if (s0 + kRopeSeed < 32) {             // prefetch the next exact seed
                                const int row = min(w.r0[t] + r_first + 2 * (s0 + kRopeSeed), p.T - 1);
                                const float4* tab = reinterpret_cast<const float4*>(p.q_rope_table + static_cast<long long>(row) * (D / 2)) + c * 2;
                                seed0 = __ldg(tab); seed1 = __ldg(tab + 1);
                            }
#pragma unroll
                            for (int i = 0; i < kRopeSeed; ++i) {
                                const int r = r_first + 2 * (s0 + i);
                                uint4* ptr = reinterpret_cast<uint4*>(qtile + r * 128 + (((c & 7) ^ (r & 7)) << 4));
                                uint4 raw = *ptr;
                                uint32_t* u = &raw.x;
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    float2 x = Elem<T>::unpack2(u[e]);
                                    float t1 = __fmul_rn(x.x, cs[e]), t2 = __fmul_rn(x.y, sn[e]);
                                    float t3 = __fmul_rn(x.x, sn[e]), t4 = __fmul_rn(x.y, cs[e]);
                                    u[e] = Elem<T>::pack2(__fsub_rn(t1, t2), __fadd_rn(t3, t4));
                                    // advance this pair's angle by two positions
                                    const float cn = fmaf(cs[e], step_c[e], -sn[e] * step_s[e]);
                                    sn[e] = fmaf(sn[e], step_c[e], cs[e] * step_s[e]);
                                    cs[e] = cn;
                                }
                                *ptr = raw;                     // rows past T are zero: rotating them is harmless
                            }
                        }
                    }
                    fence_proxy_async_smem();        // generic-proxy writes -> visible to the tensor core's smem reads
                    mbar_arrive(&bar->q_rot[b]);
                }
            }
        }
    } else {
        // =========================== softmax / correction / epilogue ===========================
        reg_inc<kRegSoftmax>();
        const int t = warp >> 2;                     // tile of this warpgroup
        const int r = tid & 127;                     // row inside the tile = TMEM lane
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t s_addr = tmem_base + lane_base + static_cast<uint32_t>(t * 128);
        const uint32_t o_addr = tmem_base + lane_base + static_cast<uint32_t>(256 + t * 128);
        const float scale_log2 = p.scale * kLog2e;
        int g = 0;                                   // running count of score tiles of this query tile
        bool ok = true;

        for (int round = 0; round < n_rounds && ok; ++round) {
            const int idx = item_of_round(round, n_items);
            if (idx < 0) continue;
            const Item w = get_item(p, idx, n_bh, n_pairs);
            const int n = t ? w.nblk[1] : w.nblk[0];
            if (n == 0) continue;
            const int tile_r0 = t ? w.r0[1] : w.r0[0];
            const int row = tile_r0 + r;             // query row in [0, T)

            float m_ref = -INFINITY, l_sum = 0.f;
            for (int j = 0; j < n; ++j, ++g) {
                ok = mbar_wait_warp(&bar->s_full[t], g & 1, abort_flag, 0x800 + t);
                if (!ok) break;
                tc_fence_after();
                uint32_t s[4][32];
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_ld32(s_addr + c * 32, s[c]);
                tmem_ld_wait();

                const int k0 = j * kBlockN;
                const bool need_mask = (k0 + kBlockN > p.Skv) || (p.causal && (k0 + kBlockN - 1 > p.start_pos + tile_r0));
                if (need_mask) {
                    const int limit = p.causal ? min(p.Skv - 1, p.start_pos + row) : p.Skv - 1;   // last visible key
#pragma unroll
                    for (int c = 0; c < 4; ++c)
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (k0 + c * 32 + i > limit) s[c][i] = 0xFF800000u;   // -inf
                }
                // row max: 8 independent chains of 3-input max (one thread owns the whole row)
                float mx8[8];
#pragma unroll
                for (int a = 0; a < 8; ++a) mx8[a] = -INFINITY;
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        mx8[(i >> 1) & 7] = fmaxf(mx8[(i >> 1) & 7], fmaxf(__uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1])));
                    }
                const float mx = fmaxf(fmax3(mx8[0], mx8[1], mx8[2]), fmaxf(fmax3(mx8[3], mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
                const float m_cand = mx * scale_log2;
                const bool grow = m_cand > m_ref + kRescaleThreshold;      // true on the first block of an item
                if (__any_sync(0xFFFFFFFFu, grow)) {
                    const float m_new = grow ? m_cand : m_ref;
                    const float alpha = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - m_new);
                    if (j > 0) {
                        // all PV products issued so far for this tile must have landed in O
                        ok = mbar_wait_warp(&bar->o_done[t], (g - 1) & 1, abort_flag, 0x900 + t);
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
                float2 rs[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
                const float2 sc2 = make_float2(scale_log2, scale_log2), nm2 = make_float2(-m_ref, -m_ref);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t pk[32];
#pragma unroll
                    for (int cc = 0; cc < 2; ++cc) {
                        const int c = 2 * half + cc;
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            // packed fp32x2: one FMA and one add per pair of columns
                            const float2 e = __ffma2_rn(make_float2(__uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1])), sc2, nm2);
                            const float2 pp = make_float2(fast_exp2(e.x), fast_exp2(e.y));
                            rs[(i >> 1) & 3] = __fadd2_rn(rs[(i >> 1) & 3], pp);
                            pk[cc * 16 + (i >> 1)] = Elem<T>::pack2(pp.x, pp.y);
                        }
                    }
                    tmem_st32(s_addr + half * 32, pk);
                }
                l_sum += ((rs[0].x + rs[0].y) + (rs[1].x + rs[1].y)) + ((rs[2].x + rs[2].y) + (rs[3].x + rs[3].y));
                tmem_st_wait();
                tc_fence_before();
                mbar_arrive(&bar->p_ready[t]);
            }
            if (!ok) break;

            // ---- epilogue of this item: O / l -> global, LSE ----
            ok = mbar_wait_warp(&bar->o_done[t], (g - 1) & 1, abort_flag, 0xA00 + t);
            if (!ok) break;
            tc_fence_after();
            const float inv_l = 1.0f / l_sum;
            const int hq_t = t ? w.hq1 : w.hq;
            T* orow = static_cast<T*>(p.o.ptr) + w.b * p.o.sb + hq_t * p.o.sh + static_cast<long long>(row) * p.o.ss;
            const bool o32 = (reinterpret_cast<uintptr_t>(orow) & 31) == 0;     // every segment offset below is a multiple of 32 bytes
#pragma unroll
            for (int c = 0; c < D / 32; c += kEpiBatch) {
                uint32_t o[kEpiBatch][32];
#pragma unroll
                for (int h2 = 0; h2 < kEpiBatch; ++h2)
                    if (c + h2 < D / 32) tmem_ld32(o_addr + (c + h2) * 32, o[h2]);
                tmem_ld_wait();
                if (row < p.T) {
#pragma unroll
                    for (int h2 = 0; h2 < kEpiBatch; ++h2) {
                        if (c + h2 >= D / 32) break;
#pragma unroll
                        for (int v = 0; v < 2; ++v) {
                            uint32_t w8[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e)
                                w8[e] = Elem<T>::pack2(__uint_as_float(o[h2][16 * v + 2 * e]) * inv_l, __uint_as_float(o[h2][16 * v + 2 * e + 1]) * inv_l);
                            if (o32) {
                                asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                                             ::"l"(orow + (c + h2) * 32 + v * 16), "r"(w8[0]), "r"(w8[1]), "r"(w8[2]), "r"(w8[3]), "r"(w8[4]), "r"(w8[5]),
                                               "r"(w8[6]), "r"(w8[7]) : "memory");
                            } else {                     // the interface promises 16-byte alignment only
                                uint4* o4 = reinterpret_cast<uint4*>(orow + (c + h2) * 32 + v * 16);
                                o4[0] = make_uint4(w8[0], w8[1], w8[2], w8[3]);
                                o4[1] = make_uint4(w8[4], w8[5], w8[6], w8[7]);
                            }
                        }
                    }
                }
            }
            // O has been read out: the next item's first PV (issued only after this thread's next
            // p_ready arrival) may overwrite it
            tc_fence_before();
            if (p.lse != nullptr && row < p.T)
                p.lse[(static_cast<long long>(w.b) * p.Hq + hq_t) * p.T + row] = (m_ref + fast_log2(l_sum)) * kLn2;
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

// The three maps of the last call of this thread, reused while the views they describe are unchanged (a serving loop
// calls with the same buffers step after step; encoding costs a few microseconds of host time per map).
struct MapKey {
    int dtype, D, B, Hq, Hkv, T, Skv;
    View4 q, k, v;
    bool operator==(const MapKey& x) const {
        auto same = [](const View4& a, const View4& b) { return a.ptr == b.ptr && a.sb == b.sb && a.sh == b.sh && a.ss == b.ss; };
        return dtype == x.dtype && D == x.D && B == x.B && Hq == x.Hq && Hkv == x.Hkv && T == x.T && Skv == x.Skv && same(q, x.q) &&
               same(k, x.k) && same(v, x.v);
    }
};

template <typename T, int D, bool kExactRope>
int launch_t(cudaStream_t s, const PrefillParams& p) {
    static thread_local MapKey cached_key{};
    static thread_local TmaMaps maps;
    static thread_local bool cached_valid = false;
    const MapKey key{p.dtype, D, p.B, p.Hq, p.Hkv, p.T, p.Skv, p.q, p.k, p.v};
    if (!cached_valid || !(cached_key == key)) {
        cached_valid = false;
        if (int rc = make_map(&maps.q, p.dtype, p.q, p.T, p.Hq, p.B, D)) return rc;
        if (int rc = make_map(&maps.k, p.dtype, p.k, p.Skv, p.Hkv, p.B, D)) return rc;
        if (int rc = make_map(&maps.v, p.dtype, p.v, p.Skv, p.Hkv, p.B, D)) return rc;
        cached_key = key;
        cached_valid = true;
    }
    static thread_local bool configured[64] = {};      // per device ordinal: the attribute belongs to the device's context
    int dev = 0;
    VB200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return set_detail(VB200_ERR_NO_DEVICE, "device ordinal out of range");
    if (!configured[dev]) {
        VB200_CUDA_TRY(cudaFuncSetAttribute(prefill_sm100_kernel<T, D, kExactRope>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<D>::kSmemBytes));
        configured[dev] = true;
    }
    const int n_items = item_rows(p) * item_cols(p);
    int sms = 0;
    VB200_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    // persistent: one CTA per SM walks the work items (heaviest first, round-robin)
    dim3 grid(static_cast<unsigned>(n_items < sms ? n_items : sms));
    profile_mark_begin(s);
    prefill_sm100_kernel<T, D, kExactRope><<<grid, kThreads, Cfg<D>::kSmemBytes, s>>>(maps, p);
    profile_mark_end(s);
    note_launch();
    note_prefill_kernel("prefill_sm100_kernel");
    VB200_CUDA_TRY(cudaPeekAtLastError());
    return VB200_OK;
}

}  // namespace


// Which of the two tensor-core kernels runs a head_dim-128 call: the single-CTA kernel of this file, unless
// VB200_PREFILL_KERNEL=pair in the environment (read once per process) asks for the two-SM kernel
// (prefill_pair_sm100.cu), which is correct but measured slower at every shape tried.
static bool use_pair_kernel(const PrefillParams& p) {
    static const int forced = []() {
        const char* e = getenv("VB200_PREFILL_KERNEL");
        if (!e) return -1;
        return (e[0] == 'p' || e[0] == 'P') ? 1 : 0;
    }();
    if (p.D != 128) return false;
    return forced == 1;      // the single-CTA kernel is the faster one at every measured shape; the pair kernel is opt-in
}

int launch_prefill_sm100(cudaStream_t s, const PrefillParams& p) {
    if (p.D != 128 && p.D != 64) return set_detail(VB200_ERR_UNSUPPORTED, "bf16/fp16 attention supports head_dim 64 and 128");
    if (use_pair_kernel(p)) return launch_prefill_pair_sm100(s, p);
    // past position 16384 the fp32 angle pos*f of the reference is itself coarse (~6e-8*pos) and only a
    // per-row table read reproduces it
    const bool exact = p.q_rope_table != nullptr && p.start_pos + p.T > 16384;
    if (p.dtype == VB200_BF16) {
        if (p.D == 128) return exact ? launch_t<__nv_bfloat16, 128, true>(s, p) : launch_t<__nv_bfloat16, 128, false>(s, p);
        return exact ? launch_t<__nv_bfloat16, 64, true>(s, p) : launch_t<__nv_bfloat16, 64, false>(s, p);
    }
    if (p.dtype == VB200_F16) {
        if (p.D == 128) return exact ? launch_t<__half, 128, true>(s, p) : launch_t<__half, 128, false>(s, p);
        return exact ? launch_t<__half, 64, true>(s, p) : launch_t<__half, 64, false>(s, p);
    }
    return VB200_ERR_UNSUPPORTED;
}

}  // namespace vb200
