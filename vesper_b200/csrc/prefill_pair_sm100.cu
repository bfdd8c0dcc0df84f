// bf16 / fp16 attention forward for head_dim 128 on sm_100a, two SMs per work item: a cluster of two CTAs runs
// every product as ONE tcgen05.mma.cta_group::2 of M = 256 query rows (128 per CTA) against a key / value block
// of which each CTA holds HALF in its shared memory (the K rows 64c .. 64c+63 of the block for S = Q K^T, the V
// columns 64c .. 64c+63 for O += P V).  Per SM that halves the shared-memory traffic of the B operand and the
// L2 -> SM fill traffic of K / V, which is what bounds the single-CTA kernel (prefill_sm100.cu: A and B of a
// 128 x 128 x 16 product both from shared memory need 128 B/clk, the shared-memory limit).
//
// Math (flash_attention_cpu_dispatch, src/ops/flash_attention.cpp:218-364):
//   s_ij = scale * q_i . k_j ;  key j visible to query i iff j <= start_pos + i
//   O_i = sum_j softmax_j(s_ij) v_j ;  LSE_i = ln sum_j exp(s_ij)
//
// A work item is FOUR 128-row query tiles that read the same K / V blocks -- two per CTA -- e.g. the same rows of
// the four query heads of a GQA group.  Persistent: cluster x of the grid walks items x, x + G, ... in snake order,
// heaviest (last rows) first.  Roles per CTA (384 threads):
//   warps 0-3 / 4-7  softmax, correction and epilogue of this CTA's tile 0 / 1 (one thread per row = TMEM lane)
//   warp  8          TMA producer: this CTA's Q tiles (3 rotating buffers) and its halves of K and V (4-slot ring)
//   warp  9          TMEM owner; in the leader CTA (cluster rank 0) also the ONLY issuer of tcgen05.mma
//   warps 10-11      RoPE of freshly loaded Q tiles, in place in swizzled shared memory
// Hand-overs: the leader's MMA thread waits on barriers in ITS shared memory that both CTAs feed -- the K / V
// "full" barrier receives the transaction bytes of both CTAs' TMA loads (cp.async.bulk.tensor with .cta_group::2
// naming the leader's barrier; no multicast anywhere), the "Q rotated" and "P ready" barriers receive remote
// mbarrier arrivals -- and signals back with tcgen05.commit multicast to the same barrier in both CTAs.
// TMEM per CTA (512 columns): S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P (16-bit) overwrites the first
// 64 columns of its S.  The epilogue stages the O tile in shared memory and writes it with TMA stores.
//
// Every wait is bounded (mbar_wait); on expiry the CTA drains and returns with the device status word set.
#include <cstdio>

#include "kernels.h"

namespace vb200 {

namespace {

constexpr int kBlockM = 128;           // query rows per tile
constexpr int kBlockN = 128;           // keys per block
constexpr int kD = 128;                // head_dim of this kernel
constexpr int kStages = 4;             // ring slots, each HALF a K or V block (16 KB)
constexpr int kQBufs = 3;
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kRopeWarp0 = 10;
constexpr int kThreads = 384;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;
constexpr int kRegSoftmax = 216, kRegOther = 72;
static_assert(kRegSoftmax * 256 + kRegOther * 128 <= 168 * 384, "register budget");

constexpr int kBoxBytes = 128 * 128;                 // [128 rows][64 cols] 16-bit box, 128-byte rows, 128B swizzle
constexpr int kTileBytes = 2 * kBoxBytes;            // one [128][128] tile (Q, or the O staging area)
constexpr int kSlotBytes = kBoxBytes;                // half a K block (2 boxes of [64 rows][64 cols]) or half a V block (1 box)
constexpr int kSmemBytes = kQBufs * kTileBytes + kStages * kSlotBytes + 2 * kTileBytes + 1024 + 256;

struct __align__(8) Barriers {
    uint64_t q_full[kQBufs];            // local: this CTA's Q tile landed
    uint64_t q_rot[kQBufs];             // leader: both CTAs' Q tiles rotated (or just loaded), 4 warp arrivals
    uint64_t q_free[kQBufs];            // both (multicast commit): last QK^T of the tile retired
    uint64_t kv_full[kStages];          // leader: both halves of the slot landed
    uint64_t kv_empty[kStages];         // both (multicast commit)
    uint64_t s_full[2];                 // both (multicast commit)
    uint64_t p_ready[2];                // leader: 8 warp arrivals (4 per CTA)
    uint64_t o_done[2];                 // both (multicast commit)
    uint64_t mma_done;                  // both (multicast commit)
    uint64_t epi_done[2];               // local: the 128 rows of a staged O tile are written (128 arrivals)
    uint32_t tmem_base;
    int abort_flag;
};

struct PairMaps {
    CUtensorMap q, k, v, o;
};

// How the four tiles of an item are laid over (head, row tile): A = four heads of a group, B = two heads x two
// adjacent row tiles, C = four adjacent row tiles of one head.
__host__ __device__ __forceinline__ int item_mode(const PrefillParams& p) {
    const int n_rep = p.Hq / p.Hkv;
    return (n_rep % 4 == 0) ? 0 : (n_rep % 2 == 0) ? 1 : 2;
}
__host__ __device__ __forceinline__ int item_cols(const PrefillParams& p) {
    const int m = item_mode(p);
    return p.B * (m == 0 ? p.Hq / 4 : m == 1 ? p.Hq / 2 : p.Hq);
}
__host__ __device__ __forceinline__ int item_rows(const PrefillParams& p) {
    const int m = item_mode(p);
    const int span = kBlockM * (m == 0 ? 1 : m == 1 ? 2 : 4);
    return (p.T + span - 1) / span;
}

struct Item {
    int b, hkv;
    int hq[2];       // head of this CTA's tile 0 / 1
    int r0[2];       // first query row of each tile (may be >= T: the tile is then computed on zero rows and not stored)
    int n;           // key blocks EVERY tile of the item steps through (the longest tile's count; the others see masked blocks)
};

__device__ __forceinline__ Item get_item(const PrefillParams& p, int it, int n_cols, int n_rows, int cta) {
    Item w;
    const int pr = n_rows - 1 - it / n_cols;       // heaviest (last) query rows first
    const int col = it % n_cols;
    const int mode = item_mode(p);
    int last_r0;
    if (mode == 0) {
        const int g = col % (p.Hq / 4);
        w.b = col / (p.Hq / 4);
        w.hq[0] = 4 * g + 2 * cta; w.hq[1] = w.hq[0] + 1;
        w.r0[0] = w.r0[1] = pr * kBlockM;
        last_r0 = pr * kBlockM;
    } else if (mode == 1) {
        const int g = col % (p.Hq / 2);
        w.b = col / (p.Hq / 2);
        w.hq[0] = 2 * g; w.hq[1] = 2 * g + 1;
        w.r0[0] = w.r0[1] = (2 * pr + cta) * kBlockM;
        last_r0 = (2 * pr + 1) * kBlockM;
    } else {
        w.b = col / p.Hq;
        w.hq[0] = w.hq[1] = col % p.Hq;
        w.r0[0] = (4 * pr + 2 * cta) * kBlockM; w.r0[1] = w.r0[0] + kBlockM;
        last_r0 = (4 * pr + 3) * kBlockM;
    }
    w.hkv = w.hq[0] / (p.Hq / p.Hkv);
    int kv_end = p.Skv;
    if (p.causal) kv_end = min(p.Skv, p.start_pos + min(last_r0 + kBlockM, p.T));
    w.n = (kv_end + kBlockN - 1) / kBlockN;
    return w;
}

// Snake dealing over the clusters of the grid.  -1: none.
__device__ __forceinline__ int item_of_round(int round, int n_items, int cluster, int n_clusters) {
    const int idx = round * n_clusters + ((round & 1) ? (n_clusters - 1 - cluster) : cluster);
    return idx < n_items ? idx : -1;
}

template <int N> __device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

// ---- cluster / cta_group::2 helpers ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of `local` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// Bounded wait with cluster-scope acquire (the barrier is fed by the peer CTA as well).
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, const WaitCtx& ctx, int where) {
    const uint32_t addr = smem_u32(bar);
    uint32_t ok = 0;
    long long t0 = 0;
    for (uint32_t it = 0;; ++it) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.b32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return true;
        if ((it & 0xFF) == 0xFF) {
            if (*ctx.abort_flag) return false;
            const long long now = clock64();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitCycles) {
                *ctx.abort_flag = 1;
                atomicCAS(ctx.status, 0, (1 << 24) | where);
                return false;
            }
        }
    }
}

// 4-D tiled TMA load whose completion bytes go to a barrier that may live in the peer CTA (`bar_cluster_addr` is a
// shared::cluster address); the destination is this CTA's own shared memory.  No multicast.
__device__ __forceinline__ void tma_load_4d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr,
                                                 int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        : : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr),
            "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
// 4-D tiled TMA store shared -> global (rows / columns outside the tensor are clipped), as one bulk group.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, const void* smem_src, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
        : : "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem, both CTAs] (+)= A[smem desc, each CTA its 128 rows] * B[smem desc, each CTA its half of N]
__device__ __forceinline__ void umma2_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        : : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// the same with A from each CTA's TMEM
__device__ __forceinline__ void umma2_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        : : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the barrier at this shared-memory offset in BOTH CTAs once every MMA issued so far has completed
__device__ __forceinline__ void umma2_commit(uint64_t* bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(both) : "memory");
}

template <typename T, bool kExactRope>
__global__ void __launch_bounds__(kThreads, 1)
prefill_pair_kernel(const __grid_constant__ PairMaps maps, PrefillParams p) {
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    unsigned char* q_smem = smem;                                        // kQBufs tiles
    unsigned char* kv_smem = q_smem + kQBufs * kTileBytes;               // kStages half-block slots
    unsigned char* o_smem = kv_smem + kStages * kSlotBytes;              // 2 staging tiles (one per softmax warpgroup)
    Barriers* bar = reinterpret_cast<Barriers*>(o_smem + 2 * kTileBytes);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t cta = cluster_ctarank();                              // 0 = leader (issues the MMAs), 1 = peer
    const bool leader = cta == 0;
    const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
    const int n_cols = item_cols(p), n_rows = item_rows(p);
    const int n_items = n_cols * n_rows;
    const int n_rounds = (n_items + n_clusters - 1) / n_clusters;
    const bool rope = p.q_rope_table != nullptr;

    // ---- setup ----
    if (warp == kMmaWarp) {
        if (lane == 0) {
            for (int b = 0; b < kQBufs; ++b) { mbar_init(&bar->q_full[b], 1); mbar_init(&bar->q_rot[b], 4); mbar_init(&bar->q_free[b], 1); }
            for (int t = 0; t < 2; ++t) {
                mbar_init(&bar->s_full[t], 1); mbar_init(&bar->p_ready[t], 8); mbar_init(&bar->o_done[t], 1); mbar_init(&bar->epi_done[t], kBlockM);
            }
            for (int s = 0; s < kStages; ++s) { mbar_init(&bar->kv_full[s], 1); mbar_init(&bar->kv_empty[s], 1); }
            mbar_init(&bar->mma_done, 1);
            bar->abort_flag = 0;
            mbar_fence_init();
        }
        __syncwarp();
        tmem_alloc2(&bar->tmem_base, 512);
        tmem_relinquish2();
        tc_fence_before();
    } else if (warp == kProducerWarp && lane == 0) {
        tma_prefetch_desc(&maps.q); tma_prefetch_desc(&maps.k); tma_prefetch_desc(&maps.v); tma_prefetch_desc(&maps.o);
    }
    __syncthreads();
    // both CTAs' barriers exist and both TMEM allocations are done before anything crosses the pair
    cluster_arrive();
    cluster_wait();
    tc_fence_after();
    const uint32_t tmem_base = bar->tmem_base;
    const WaitCtx abort_flag{&bar->abort_flag, p.status};

    if (warp >= 8) {
        reg_dec<kRegOther>();
        if (warp == kProducerWarp) {
            // =========================== TMA producer (each CTA: its Q tiles, its halves of K and V) ===========================
            if (lane == 0) {
                int kv_item = 0, q_seq = 0;
                bool ok = true;
                uint32_t kv_full_leader[kStages];
#pragma unroll
                for (int s = 0; s < kStages; ++s) kv_full_leader[s] = map_to_cta(smem_u32(&bar->kv_full[s]), 0);
                auto load_q = [&](const Item& w, int t) {
                    if (!ok) return;
                    const int b = q_seq % kQBufs, use = q_seq / kQBufs;
                    if (use > 0) ok = mbar_wait(&bar->q_free[b], (use - 1) & 1, abort_flag, 0x110 + b);
                    if (!ok) return;
                    ++q_seq;
                    mbar_arrive_expect_tx(&bar->q_full[b], kTileBytes);
                    // rows at or past T (an absent tile, a ragged last tile) arrive as zeros
                    tma_load_4d(q_smem + b * kTileBytes, &maps.q, &bar->q_full[b], 0, w.r0[t], w.hq[t], w.b);
                    tma_load_4d(q_smem + b * kTileBytes + kBoxBytes, &maps.q, &bar->q_full[b], 64, w.r0[t], w.hq[t], w.b);
                };
                int round = 0, idx = -1;
                while (round < n_rounds && (idx = item_of_round(round, n_items, cluster_id, n_clusters)) < 0) ++round;
                Item w;
                if (idx >= 0) { w = get_item(p, idx, n_cols, n_rows, cta); load_q(w, 0); load_q(w, 1); }
                while (idx >= 0 && ok) {
                    int round2 = round + 1, idx2 = -1;
                    while (round2 < n_rounds && (idx2 = item_of_round(round2, n_items, cluster_id, n_clusters)) < 0) ++round2;
                    Item wn;
                    if (idx2 >= 0) { wn = get_item(p, idx2, n_cols, n_rows, cta); load_q(wn, 0); }
                    for (int x = 0; x < 2 * w.n && ok; ++x, ++kv_item) {        // x = 2j: K_j, 2j+1: V_j
                        const int slot = kv_item % kStages;
                        if (kv_item >= kStages) ok = mbar_wait(&bar->kv_empty[slot], ((kv_item / kStages) - 1) & 1, abort_flag, 0x100);
                        if (!ok) break;
                        // the leader's barrier collects the bytes of both CTAs' halves
                        if (leader) mbar_arrive_expect_tx(&bar->kv_full[slot], 2 * kSlotBytes);
                        unsigned char* dst = kv_smem + slot * kSlotBytes;
                        const int key0 = (x >> 1) * kBlockN;
                        if ((x & 1) == 0) {
                            // K: this CTA's 64 keys of the block, all 128 dims, as two [64 rows][64 cols] boxes
                            tma_load_4d_pair(dst, &maps.k, kv_full_leader[slot], 0, key0 + 64 * static_cast<int>(cta), w.hkv, w.b);
                            tma_load_4d_pair(dst + kSlotBytes / 2, &maps.k, kv_full_leader[slot], 64, key0 + 64 * static_cast<int>(cta), w.hkv, w.b);
                        } else {
                            // V: all 128 keys of the block, this CTA's 64 dims, one [128 rows][64 cols] box
                            tma_load_4d_pair(dst, &maps.v, kv_full_leader[slot], 64 * static_cast<int>(cta), key0, w.hkv, w.b);
                        }
                    }
                    if (idx2 >= 0) load_q(wn, 1);
                    idx = idx2; round = round2; w = wn;
                }
            }
        } else if (warp == kMmaWarp) {
            // =========================== MMA issuer (leader CTA only) ===========================
            if (leader && lane == 0) {
                constexpr uint32_t idesc_qk = make_idesc_f16(Elem<T>::kFormat, 0, 0, 2 * kBlockM, kBlockN);
                constexpr uint32_t idesc_pv = make_idesc_f16(Elem<T>::kFormat, 0, 1, 2 * kBlockM, kD);
                const uint32_t q_addr = smem_u32(q_smem), kv_addr = smem_u32(kv_smem);
                auto tmem_s = [&](int t) { return tmem_base + static_cast<uint32_t>(t * 128); };
                auto tmem_o = [&](int t) { return tmem_base + static_cast<uint32_t>(256 + t * 128); };
                auto issue_qk = [&](int t, int qbuf, int slot) {
#pragma unroll
                    for (int kk = 0; kk < kD / 16; ++kk) {
                        // A: [128 rows][64 cols] boxes of the Q tile; B: [64 rows][64 cols] boxes of this CTA's K half
                        const uint64_t a = make_smem_desc_sw128(q_addr + qbuf * kTileBytes + (kk >> 2) * kBoxBytes + (kk & 3) * 32, 16, 1024);
                        const uint64_t bd = make_smem_desc_sw128(kv_addr + slot * kSlotBytes + (kk >> 2) * (kSlotBytes / 2) + (kk & 3) * 32, 16, 1024);
                        umma2_ss(tmem_s(t), a, bd, idesc_qk, kk > 0 ? 1u : 0u);
                    }
                };
                auto issue_pv = [&](int t, int slot, bool accumulate) {
#pragma unroll
                    for (int kk = 0; kk < kBlockN / 16; ++kk) {
                        // V half is MN-major for this product: 16 keys = 2048 bytes per step, 64 dims per CTA
                        const uint64_t bd = make_smem_desc_sw128(kv_addr + slot * kSlotBytes + kk * 2048, kBoxBytes, 1024);
                        umma2_ts(tmem_o(t), tmem_s(t) + kk * 8, bd, idesc_pv, (accumulate || kk > 0) ? 1u : 0u);
                    }
                };
                int kv_item = 0, q_seq = 0;
                int blk[2] = {0, 0};             // running count of score tiles per tile index (barrier phases)
                bool ok = true;
                for (int round = 0; round < n_rounds && ok; ++round) {
                    const int idx = item_of_round(round, n_items, cluster_id, n_clusters);
                    if (idx < 0) continue;
                    const Item w = get_item(p, idx, n_cols, n_rows, 0);
                    int qbuf[2] = {0, 0};
                    const int k0_slot = kv_item % kStages;
                    ok = mbar_wait_cluster(&bar->kv_full[k0_slot], (kv_item / kStages) & 1, abort_flag, 0x200);
#pragma unroll
                    for (int t = 0; t < 2; ++t) {
                        if (!ok) continue;
                        qbuf[t] = q_seq % kQBufs;
                        const int ph = (q_seq / kQBufs) & 1;
                        ++q_seq;
                        // S of this tile is free: every PV of the previous item was issued before this point
                        ok = mbar_wait_cluster(&bar->q_rot[qbuf[t]], ph, abort_flag, 0x210 + t);
                        if (!ok) continue;
                        tc_fence_after();
                        issue_qk(t, qbuf[t], k0_slot);
                        umma2_commit(&bar->s_full[t]);
                        if (w.n == 1) umma2_commit(&bar->q_free[qbuf[t]]);
                    }
                    if (!ok) break;
                    umma2_commit(&bar->kv_empty[k0_slot]);
                    for (int j = 0; j < w.n && ok; ++j) {
                        const int v_item = kv_item + 2 * j + 1, k_item = kv_item + 2 * j + 2;
                        const int v_slot = v_item % kStages, k_slot = k_item % kStages;
                        ok = mbar_wait_cluster(&bar->kv_full[v_slot], (v_item / kStages) & 1, abort_flag, 0x300);
                        bool k_ready = false;
#pragma unroll
                        for (int t = 0; t < 2; ++t) {
                            if (!ok) continue;
                            ok = mbar_wait_cluster(&bar->p_ready[t], blk[t] & 1, abort_flag, 0x400 + t);
                            if (!ok) continue;
                            ++blk[t];
                            tc_fence_after();
                            issue_pv(t, v_slot, j > 0);
                            umma2_commit(&bar->o_done[t]);
                            if (j + 1 < w.n) {
                                if (!k_ready) {
                                    ok = mbar_wait_cluster(&bar->kv_full[k_slot], (k_item / kStages) & 1, abort_flag, 0x500);
                                    if (!ok) continue;
                                    tc_fence_after();
                                    k_ready = true;
                                }
                                issue_qk(t, qbuf[t], k_slot);
                                umma2_commit(&bar->s_full[t]);
                                if (j + 2 == w.n) umma2_commit(&bar->q_free[qbuf[t]]);   // last QK of this tile
                            }
                        }
                        if (!ok) break;
                        umma2_commit(&bar->kv_empty[v_slot]);
                        if (j + 1 < w.n) umma2_commit(&bar->kv_empty[k_slot]);
                    }
                    kv_item += 2 * w.n;
                }
                // everything issued so far has to retire (in both CTAs) before TMEM is released
                umma2_commit(&bar->mma_done);
            }
            __syncwarp();
        } else {
            // =========================== RoPE of this CTA's Q tiles; tells the leader they are ready ===========================
            // 2 warps; warp w owns rows [64w, 64w+64) of each tile.  A step handles two rows: lane l takes 16-byte
            // chunk (l & 15) of row 2*step + (l >> 4).  Without RoPE the warps only forward "tile landed".
            const int rw = warp - kRopeWarp0;
            const int c = lane & 15;
            constexpr int kRopeSeed = 8;                      // steps (of two rows) between exact table reads
            float step_c[4], step_s[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) sincosf(2.0f * p.inv_freq.v[(c * 4 + e) & (kMaxHalfDim - 1)], &step_s[e], &step_c[e]);
            uint32_t q_rot_leader[kQBufs];
#pragma unroll
            for (int b = 0; b < kQBufs; ++b) q_rot_leader[b] = map_to_cta(smem_u32(&bar->q_rot[b]), 0);
            int q_seq = 0;
            bool ok = true;
            for (int round = 0; round < n_rounds && ok; ++round) {
                const int idx = item_of_round(round, n_items, cluster_id, n_clusters);
                if (idx < 0) continue;
                const Item w = get_item(p, idx, n_cols, n_rows, cta);
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    if (!ok) continue;
                    const int b = q_seq % kQBufs, ph = (q_seq / kQBufs) & 1;
                    ++q_seq;
                    ok = mbar_wait_warp(&bar->q_full[b], ph, abort_flag, 0x700 + b);
                    if (!ok) continue;
                    if (rope) {
                        unsigned char* qtile = q_smem + b * kTileBytes + (c >> 3) * kBoxBytes;
                        const int r_first = rw * 64 + (lane >> 4);
                        // rows past T hold zeros: rotating them is harmless; their table row is clamped
                        if constexpr (kExactRope) {
#pragma unroll 2
                            for (int st = 0; st < 32; ++st) {
                                const int r = r_first + 2 * st;
                                const int rowx = min(w.r0[t] + r, p.T - 1);
                                const float4* tabx = reinterpret_cast<const float4*>(p.q_rope_table + static_cast<long long>(rowx) * (kD / 2)) + c * 2;
                                const float4 a0 = __ldg(tabx), a1 = __ldg(tabx + 1);
                                const float csx[4] = {a0.x, a0.z, a1.x, a1.z}, snx[4] = {a0.y, a0.w, a1.y, a1.w};
                                uint4* ptr = reinterpret_cast<uint4*>(qtile + r * 128 + (((c & 7) ^ (r & 7)) << 4));
                                uint4 raw = *ptr;
                                uint32_t* u = &raw.x;
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const float2 x = Elem<T>::unpack2(u[e]);
                                    const float t1 = __fmul_rn(x.x, csx[e]), t2 = __fmul_rn(x.y, snx[e]);
                                    const float t3 = __fmul_rn(x.x, snx[e]), t4 = __fmul_rn(x.y, csx[e]);
                                    u[e] = Elem<T>::pack2(__fsub_rn(t1, t2), __fadd_rn(t3, t4));
                                }
                                *ptr = raw;
                            }
                        } else {
                            float4 seed0, seed1;
                            {
                                const int row = min(w.r0[t] + r_first, p.T - 1);
                                const float4* tab = reinterpret_cast<const float4*>(p.q_rope_table + static_cast<long long>(row) * (kD / 2)) + c * 2;
                                seed0 = __ldg(tab); seed1 = __ldg(tab + 1);
                            }
#pragma unroll 1
                            for (int s0 = 0; s0 < 32; s0 += kRopeSeed) {
                                float cs[4] = {seed0.x, seed0.z, seed1.x, seed1.z};
                                float sn[4] = {seed0.y, seed0.w, seed1.y, seed1.w};
                                if (s0 + kRopeSeed < 32) {             // prefetch the next exact seed
                                    const int row = min(w.r0[t] + r_first + 2 * (s0 + kRopeSeed), p.T - 1);
                                    const float4* tab = reinterpret_cast<const float4*>(p.q_rope_table + static_cast<long long>(row) * (kD / 2)) + c * 2;
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
                                        const float2 x = Elem<T>::unpack2(u[e]);
                                        const float t1 = __fmul_rn(x.x, cs[e]), t2 = __fmul_rn(x.y, sn[e]);
                                        const float t3 = __fmul_rn(x.x, sn[e]), t4 = __fmul_rn(x.y, cs[e]);
                                        u[e] = Elem<T>::pack2(__fsub_rn(t1, t2), __fadd_rn(t3, t4));
                                        // advance this pair's angle by two positions
                                        const float cn = fmaf(cs[e], step_c[e], -sn[e] * step_s[e]);
                                        sn[e] = fmaf(sn[e], step_c[e], cs[e] * step_s[e]);
                                        cs[e] = cn;
                                    }
                                    *ptr = raw;
                                }
                            }
                        }
                    }
                    fence_proxy_async_smem();            // generic-proxy writes -> visible to the tensor core's smem reads
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(q_rot_leader[b]);
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
        const uint32_t p_ready_leader = map_to_cta(smem_u32(&bar->p_ready[t]), 0);
        unsigned char* stage = o_smem + t * kTileBytes;
        int g = 0;                                   // running count of score tiles of this tile index
        bool ok = true;
        bool store_pending = false;                  // thread 0 of the warpgroup: a TMA store may still be reading `stage`
        int epi_phase = 0;                           // items whose epilogue this warpgroup has run

        for (int round = 0; round < n_rounds && ok; ++round) {
            const int idx = item_of_round(round, n_items, cluster_id, n_clusters);
            if (idx < 0) continue;
            const Item w = get_item(p, idx, n_cols, n_rows, cta);
            const int n = w.n;
            const int tile_r0 = w.r0[t];
            const int row = tile_r0 + r;             // query row; >= T for padding rows (computed on zeros, never stored)

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
                float mx8[8];
#pragma unroll
                for (int a = 0; a < 8; ++a) mx8[a] = -INFINITY;
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; i += 2)
                        mx8[(i >> 1) & 7] = fmaxf(mx8[(i >> 1) & 7], fmaxf(__uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1])));
                const float mx = fmaxf(fmax3(mx8[0], mx8[1], mx8[2]), fmaxf(fmax3(mx8[3], mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
                const float m_cand = mx * scale_log2;
                // a block this row sees nothing of (it belongs to a longer tile of the item) has m_cand = -inf: no growth
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
                        for (int c = 0; c < kD / 32; ++c) {
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
                // The staging tile of this warpgroup is written again in this item's epilogue, which every row enters
                // only after the product that this (last) hand-over releases: the thread that issued the previous
                // item's store makes sure, before handing over, that the store has finished reading the tile.
                if (j + 1 == n && r == 0 && store_pending) { bulk_wait_read0(); store_pending = false; }
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(p_ready_leader);
            }
            if (!ok) break;

            // ---- epilogue of this item: O / l -> staging tile in shared memory -> TMA store; LSE ----
            ok = mbar_wait_warp(&bar->o_done[t], (g - 1) & 1, abort_flag, 0xA00 + t);
            if (!ok) break;
            tc_fence_after();
            const float inv_l = 1.0f / l_sum;
            const bool present = tile_r0 < p.T;
#pragma unroll
            for (int c = 0; c < kD / 32; c += 2) {
                uint32_t o[2][32];
                tmem_ld32(o_addr + c * 32, o[0]);
                tmem_ld32(o_addr + (c + 1) * 32, o[1]);
                tmem_ld_wait();
#pragma unroll
                for (int h2 = 0; h2 < 2; ++h2) {
                    // 32 columns = four 16-byte chunks of this row; chunk index inside its 64-column box: ((c + h2) & 1) * 4 + v
                    unsigned char* box = stage + ((c + h2) >> 1) * kBoxBytes + r * 128;
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        uint4 out;
                        out.x = Elem<T>::pack2(__uint_as_float(o[h2][8 * v + 0]) * inv_l, __uint_as_float(o[h2][8 * v + 1]) * inv_l);
                        out.y = Elem<T>::pack2(__uint_as_float(o[h2][8 * v + 2]) * inv_l, __uint_as_float(o[h2][8 * v + 3]) * inv_l);
                        out.z = Elem<T>::pack2(__uint_as_float(o[h2][8 * v + 4]) * inv_l, __uint_as_float(o[h2][8 * v + 5]) * inv_l);
                        out.w = Elem<T>::pack2(__uint_as_float(o[h2][8 * v + 6]) * inv_l, __uint_as_float(o[h2][8 * v + 7]) * inv_l);
                        const int chunk = ((c + h2) & 1) * 4 + v;
                        *reinterpret_cast<uint4*>(box + ((chunk ^ (r & 7)) << 4)) = out;
                    }
                }
            }
            // O has been read out of TMEM: the next item's first PV (issued only after this thread's next P hand-over)
            // may overwrite it
            tc_fence_before();
            fence_proxy_async_smem();                // this row of the staging tile -> visible to the TMA store
            mbar_arrive(&bar->epi_done[t]);
            if (r == 0) {
                // only the issuing thread waits for the other rows (bounded like every wait)
                if (mbar_wait(&bar->epi_done[t], epi_phase & 1, abort_flag, 0xB00 + t) && present) {
                    tma_store_4d(&maps.o, stage, 0, tile_r0, w.hq[t], w.b);
                    tma_store_4d(&maps.o, stage + kBoxBytes, 64, tile_r0, w.hq[t], w.b);
                    bulk_commit();
                    store_pending = true;
                }
            }
            ++epi_phase;
            if (p.lse != nullptr && present && row < p.T)
                p.lse[(static_cast<long long>(w.b) * p.Hq + w.hq[t]) * p.T + row] = (m_ref + fast_log2(l_sum)) * kLn2;
        }
        if (r == 0 && store_pending) bulk_wait0();   // the staging tile must outlive the store's reads
    }

    // ---- teardown: every MMA retired in both CTAs, nobody still signals the peer, then TMEM is released ----
    if (warp == kMmaWarp && lane == 0) mbar_wait(&bar->mma_done, 0, abort_flag, 0x600);
    tc_fence_before();
    __syncthreads();
    cluster_arrive();
    cluster_wait();
    if (warp == kMmaWarp) {
        tc_fence_after();
        tmem_dealloc2(tmem_base, 512);
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

// [B,H,rows,128] view -> 4-D map (D, rows, H, B), box [64 cols][box_rows], 128-byte swizzle.
int make_map(CUtensorMap* m, int dtype, const View4& v, int rows, int H, int B, int box_rows) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return set_detail(VB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(kD), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(B)};
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(v.ss) * 2, static_cast<cuuint64_t>(v.sh) * 2, static_cast<cuuint64_t>(v.sb) * 2};
    for (int i = 0; i < 3; ++i) if (strides[i] == 0) strides[i] = 16;     // a dimension of extent 1 may carry any stride
    cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_rows), 1, 1};
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

// The four maps of the last call of this thread, reused while the views they describe are unchanged (a serving
// loop calls with the same buffers step after step; encoding costs a few microseconds of host time per map).
struct MapKey {
    int dtype, B, Hq, Hkv, T, Skv;
    View4 q, k, v, o;
    bool operator==(const MapKey& x) const {
        auto same = [](const View4& a, const View4& b) { return a.ptr == b.ptr && a.sb == b.sb && a.sh == b.sh && a.ss == b.ss; };
        return dtype == x.dtype && B == x.B && Hq == x.Hq && Hkv == x.Hkv && T == x.T && Skv == x.Skv && same(q, x.q) && same(k, x.k) &&
               same(v, x.v) && same(o, x.o);
    }
};

template <typename T, bool kExactRope>
int launch_t(cudaStream_t s, const PrefillParams& p) {
    static thread_local MapKey cached_key{};
    static thread_local PairMaps cached_maps;
    static thread_local bool cached_valid = false;
    const MapKey key{p.dtype, p.B, p.Hq, p.Hkv, p.T, p.Skv, p.q, p.k, p.v, p.o};
    if (!cached_valid || !(cached_key == key)) {
        cached_valid = false;
        if (int rc = make_map(&cached_maps.q, p.dtype, p.q, p.T, p.Hq, p.B, 128)) return rc;
        if (int rc = make_map(&cached_maps.k, p.dtype, p.k, p.Skv, p.Hkv, p.B, 64)) return rc;
        if (int rc = make_map(&cached_maps.v, p.dtype, p.v, p.Skv, p.Hkv, p.B, 128)) return rc;
        if (int rc = make_map(&cached_maps.o, p.dtype, p.o, p.T, p.Hq, p.B, 128)) return rc;
        cached_key = key;
        cached_valid = true;
    }
    int dev = 0;
    VB200_CUDA_TRY(cudaGetDevice(&dev));
    static thread_local bool configured[64] = {};
    if (dev < 0 || dev >= 64) return set_detail(VB200_ERR_NO_DEVICE, "device ordinal out of range");
    auto kernel = prefill_pair_kernel<T, kExactRope>;
    if (!configured[dev]) {
        VB200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        configured[dev] = true;
    }
    int sms = 0;
    VB200_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int n_items = item_rows(p) * item_cols(p);
    int clusters = sms / 2;
    if (clusters > n_items) clusters = n_items;
    if (clusters < 1) clusters = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(2 * clusters));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    profile_mark_begin(s);
    VB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, cached_maps, p));
    profile_mark_end(s);
    note_launch();
    VB200_CUDA_TRY(cudaPeekAtLastError());
    return VB200_OK;
}

}  // namespace

// head_dim 128, bf16 / fp16.  The caller (launch_prefill_sm100) keeps the single-CTA kernel for head_dim 64.
int launch_prefill_pair_sm100(cudaStream_t s, const PrefillParams& p) {
    // past position 16384 the fp32 angle pos*f of the reference is itself coarse (~6e-8*pos) and only a
    // per-row table read reproduces it
    const bool exact = p.q_rope_table != nullptr && p.start_pos + p.T > 16384;
    if (p.dtype == VB200_BF16) return exact ? launch_t<__nv_bfloat16, true>(s, p) : launch_t<__nv_bfloat16, false>(s, p);
    if (p.dtype == VB200_F16) return exact ? launch_t<__half, true>(s, p) : launch_t<__half, false>(s, p);
    return VB200_ERR_UNSUPPORTED;
}

}  // namespace vb200
