// bf16 / fp16 attention forward for head_dim 128 on sm_100a, two SMs per work item: a cluster of two CTAs runs
// every product as ONE tcgen05.mma.cta_group::2 of M = 256 query rows (one 128-row tile per CTA) against a key /
// value block of which each CTA holds HALF in its shared memory (the K rows 64c .. 64c+63 of the block for
// S = Q K^T, the V columns 64c .. 64c+63 for O += P V).  Halving the B-operand traffic per SM is what lets ONE query
// tile per SM keep the tensor pipe fed (a single CTA needs two tiles per K / V block to stay under the 128 B/clk
// shared-memory limit, prefill_sm100.cu), and one tile per SM leaves TMEM room to take the products off the
// softmax's critical path:
//   TMEM per CTA (512 columns): S[0] [0,128)  S[1] [128,256)  O [256,384)  P[0] [384,448)  P[1] [448,512)
//   block g of the running block count uses S[g & 1] and P[g & 1].  Q K^T of block g+2 is issued as soon as the
//   softmax has READ S of block g into registers, i.e. long before it finishes block g; P has its own columns, so
//   nothing the softmax still needs is overwritten.  The softmax warpgroup therefore goes from block to block
//   (and from one work item to the next) without waiting for a product; the hand-over latencies between the two SMs
//   stay off its path.  A second warpgroup drains O of a finished item (scale by 1/l, stage in shared memory, TMA
//   store, LSE) while the softmax warpgroup is already in the next item.
//
// Math (flash_attention_cpu_dispatch, src/ops/flash_attention.cpp:218-364):
//   s_ij = scale * q_i . k_j ;  key j visible to query i iff j <= start_pos + i
//   O_i = sum_j softmax_j(s_ij) v_j ;  LSE_i = ln sum_j exp(s_ij)
//
// A work item is TWO 128-row query tiles that read the same K / V blocks -- one per CTA: the same rows of two query
// heads of a GQA group, or two adjacent row tiles of one head.  Persistent: cluster x of the grid walks items
// x, x + G, ... in snake order, heaviest (last rows) first.  Roles per CTA (384 threads):
//   warps 0-3    softmax of this CTA's tile: one thread per row = TMEM lane; also the (rare) rescale of O
//   warps 4-7    epilogue of finished items
//   warp  8      TMA producer: this CTA's Q tiles (3 rotating buffers) and its halves of K and V (6-slot ring)
//   warp  9      TMEM owner; in the leader CTA (cluster rank 0) also the ONLY issuer of tcgen05.mma
//   warps 10-11  RoPE of freshly loaded Q tiles, in place in swizzled shared memory
// Hand-overs: the leader's MMA thread waits on barriers in ITS shared memory that both CTAs feed -- the K / V
// "full" barrier receives the transaction bytes of both CTAs' TMA loads (cp.async.bulk.tensor with .cta_group::2
// naming the leader's barrier; no multicast anywhere), "Q rotated", "S read", "P ready" and "O drained" receive
// remote mbarrier arrivals -- and signals back with tcgen05.commit multicast to the same barrier in both CTAs.
//
// Every wait is bounded (mbar_wait); on expiry the CTA drains and returns with the device status word set.
//
// Status: correct (same parity suite as the single-CTA kernel) and selectable with VB200_PREFILL_KERNEL=pair, but
// NOT the default: with one query tile per SM there is one softmax warpgroup per SM, and one warp per SM
// sub-partition cannot overlap its row-maximum and exponential phases (about 1450 cycles per 128x128 block at best,
// against 1100 for two warpgroups that interleave on the MUFU), so the kernel is softmax-bound at a lower rate than
// the single-CTA kernel, whose two tiles per SM keep two softmax warpgroups busy.
#include <cstdio>

#include "kernels.h"

namespace vb200 {

namespace {

constexpr int kBlockM = 128;           // query rows per tile
constexpr int kBlockN = 128;           // keys per block
constexpr int kD = 128;                // head_dim of this kernel
constexpr int kStages = 6;             // ring slots, each HALF a K or V block (16 KB)
constexpr int kQBufs = 3;
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kRopeWarp0 = 10;
constexpr int kThreads = 384;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;
constexpr int kRegSoftmax = 232, kRegEpilogue = 168, kRegOther = 72;     // per thread after setmaxnreg, by warpgroup (168 = the launch value)
static_assert((kRegSoftmax + kRegEpilogue + kRegOther) * 128 <= 168 * 384, "register budget");

constexpr int kBoxBytes = 128 * 128;                 // [128 rows][64 cols] 16-bit box, 128-byte rows, 128B swizzle
constexpr int kTileBytes = 2 * kBoxBytes;            // one [128][128] tile (Q, or the O staging area)
constexpr int kSlotBytes = kBoxBytes;                // half a K block (2 boxes of [64 rows][64 cols]) or half a V block (1 box)
constexpr int kSmemBytes = kQBufs * kTileBytes + kStages * kSlotBytes + kTileBytes + kBlockM * 8 + 1024 + 512;
static_assert(kSmemBytes <= 232448, "227 KB of dynamic shared memory per CTA");

struct __align__(8) Barriers {
    uint64_t q_full[kQBufs];            // local: this CTA's Q tile landed
    uint64_t q_rot[kQBufs];             // leader: both CTAs' Q tiles rotated (or just loaded), 4 warp arrivals
    uint64_t q_free[kQBufs];            // both (multicast commit): last QK^T of the item retired
    uint64_t kv_full[kStages];          // leader: both halves of the slot landed
    uint64_t kv_empty[kStages];         // both (multicast commit)
    uint64_t s_full[2];                 // both (multicast commit): S[b] holds the scores of a block
    uint64_t s_free[2];                 // leader: both softmax warpgroups have S[b] in registers (8 warp arrivals)
    uint64_t p_ready[2];                // leader: P[b] written (8 warp arrivals)
    uint64_t pv_done[2];                // both (multicast commit): the product that read P[b] retired
    uint64_t o_free;                    // leader: both epilogue warpgroups have O in registers (8 warp arrivals)
    uint64_t mma_done;                  // both (multicast commit)
    uint64_t stat_full, stat_free;      // local, softmax <-> epilogue warpgroup: (m, l) of a finished item (128 arrivals)
    uint64_t stage_free;                // local: the previous TMA store has finished reading the staging tile (1 arrival)
    uint64_t epi_done;                  // local: the 128 rows of the staged O tile are written (128 arrivals)
    uint32_t tmem_base;
    int abort_flag;
};

struct PairMaps {
    CUtensorMap q, k, v, o;
};

// How the two tiles of an item are laid over (head, row tile): two heads of a group (an even number of query
// heads per KV head), else two adjacent row tiles of one head.
__host__ __device__ __forceinline__ bool pair_by_heads(const PrefillParams& p) { return (p.Hq / p.Hkv) % 2 == 0; }
__host__ __device__ __forceinline__ int item_cols(const PrefillParams& p) { return pair_by_heads(p) ? p.B * (p.Hq / 2) : p.B * p.Hq; }
__host__ __device__ __forceinline__ int item_rows(const PrefillParams& p) {
    const int span = pair_by_heads(p) ? kBlockM : 2 * kBlockM;
    return (p.T + span - 1) / span;
}

struct Item {
    int b, hkv;
    int hq;          // head of this CTA's tile
    int r0;          // first query row of this CTA's tile (may be >= T: computed on zero rows and not stored)
    int n;           // key blocks BOTH tiles of the item step through (the longer tile's count; the other sees masked blocks)
};

__device__ __forceinline__ Item get_item(const PrefillParams& p, int it, int n_cols, int n_rows, int cta) {
    Item w;
    const int pr = n_rows - 1 - it / n_cols;       // heaviest (last) query rows first
    const int col = it % n_cols;
    int last_r0;
    if (pair_by_heads(p)) {
        w.b = col / (p.Hq / 2);
        w.hq = 2 * (col % (p.Hq / 2)) + cta;
        w.r0 = pr * kBlockM;
        last_r0 = w.r0;
    } else {
        w.b = col / p.Hq;
        w.hq = col % p.Hq;
        w.r0 = (2 * pr + cta) * kBlockM;
        last_r0 = (2 * pr + 1) * kBlockM;
    }
    w.hkv = w.hq / (p.Hq / p.Hkv);
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
// Arrival on a barrier of the peer CTA.  Default semantics (release at CTA scope): what is handed over lives in TMEM
// or was made visible to the async proxy by its writer, and is ordered by the tcgen05 / proxy fences around the
// barrier; a release at cluster scope here was measured at ~1000 cycles per arrival on the arriving warp.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// The same with a cluster-scope release, for generic-proxy data written by this CTA's threads (off the critical path).
__device__ __forceinline__ void mbar_arrive_cluster_release(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

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

// Walks the key blocks of all work items of a cluster in processing order: g counts blocks over the whole kernel
// (it selects the S / P buffer and the barrier phases), j the block inside the current item.
struct BlockCursor {
    int round, n_rounds, n_items, cluster, n_clusters, n_cols, n_rows, cta;
    int item_no;     // items started so far - 1
    int j, g;
    bool valid;
    Item w;
    __device__ void find_item(const PrefillParams& p) {
        int idx = -1;
        while (round < n_rounds && (idx = item_of_round(round, n_items, cluster, n_clusters)) < 0) ++round;
        valid = idx >= 0;
        if (valid) { w = get_item(p, idx, n_cols, n_rows, cta); ++item_no; j = 0; }
    }
    __device__ void init(const PrefillParams& p, int n_rounds_, int n_items_, int cluster_, int n_clusters_, int n_cols_, int n_rows_, int cta_) {
        round = 0; n_rounds = n_rounds_; n_items = n_items_; cluster = cluster_; n_clusters = n_clusters_; n_cols = n_cols_; n_rows = n_rows_; cta = cta_;
        item_no = -1; j = 0; g = 0;
        find_item(p);
    }
    __device__ void next(const PrefillParams& p) {       // to the next block
        ++g;
        if (++j >= w.n) { ++round; find_item(p); }
    }
    __device__ void next_item(const PrefillParams& p) {  // to the first block of the next item
        g += w.n - j;
        ++round;
        find_item(p);
    }
};

template <typename T, bool kExactRope>
__global__ void __launch_bounds__(kThreads, 1)
prefill_pair_kernel(const __grid_constant__ PairMaps maps, PrefillParams p) {
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    unsigned char* q_smem = smem;                                        // kQBufs tiles
    unsigned char* kv_smem = q_smem + kQBufs * kTileBytes;               // kStages half-block slots
    unsigned char* o_smem = kv_smem + kStages * kSlotBytes;              // staging tile of the epilogue
    float2* stats = reinterpret_cast<float2*>(o_smem + kTileBytes);      // [128] (m_ref, l_sum) of the item that just finished
    Barriers* bar = reinterpret_cast<Barriers*>(o_smem + kTileBytes + kBlockM * 8);

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
            for (int s = 0; s < kStages; ++s) { mbar_init(&bar->kv_full[s], 1); mbar_init(&bar->kv_empty[s], 1); }
            for (int b = 0; b < 2; ++b) {
                mbar_init(&bar->s_full[b], 1); mbar_init(&bar->s_free[b], 8); mbar_init(&bar->p_ready[b], 8); mbar_init(&bar->pv_done[b], 1);
            }
            mbar_init(&bar->stat_full, kBlockM); mbar_init(&bar->stat_free, kBlockM);
            mbar_init(&bar->o_free, 8);
            mbar_init(&bar->mma_done, 1);
            mbar_init(&bar->stage_free, 1);
            mbar_init(&bar->epi_done, kBlockM);
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
            // K / V slots are filled in the order the MMA thread consumes them: K(0), K(1), then for every block g of the
            // kernel-wide sequence K(g+2), V(g) -- across item boundaries.
            if (lane == 0) {
                int kv_item = 0;
                bool ok = true;
                const uint32_t kv_full_leader0 = map_to_cta(smem_u32(&bar->kv_full[0]), 0);   // the barriers of one kind are contiguous
                int q_loaded = -1;               // last item number whose Q tile load was issued
                auto load_q = [&](const BlockCursor& c) {
                    if (!ok || !c.valid || c.item_no <= q_loaded) return;
                    const int b = c.item_no % kQBufs, use = c.item_no / kQBufs;
                    if (use > 0) ok = mbar_wait(&bar->q_free[b], (use - 1) & 1, abort_flag, 0x110 + b);
                    if (!ok) return;
                    q_loaded = c.item_no;
                    mbar_arrive_expect_tx(&bar->q_full[b], kTileBytes);
                    // rows at or past T (an absent tile, a ragged last tile) arrive as zeros
                    tma_load_4d(q_smem + b * kTileBytes, &maps.q, &bar->q_full[b], 0, c.w.r0, c.w.hq, c.w.b);
                    tma_load_4d(q_smem + b * kTileBytes + kBoxBytes, &maps.q, &bar->q_full[b], 64, c.w.r0, c.w.hq, c.w.b);
                };
                auto load_half = [&](const BlockCursor& c, bool is_v) {
                    if (!ok) return;
                    const int slot = kv_item % kStages;
                    if (kv_item >= kStages) ok = mbar_wait(&bar->kv_empty[slot], ((kv_item / kStages) - 1) & 1, abort_flag, 0x100);
                    if (!ok) return;
                    ++kv_item;
                    // the leader's barrier collects the bytes of both CTAs' halves
                    if (leader) mbar_arrive_expect_tx(&bar->kv_full[slot], 2 * kSlotBytes);
                    unsigned char* dst = kv_smem + slot * kSlotBytes;
                    const uint32_t full_bar = kv_full_leader0 + 8 * slot;
                    const int key0 = c.j * kBlockN;
                    if (!is_v) {
                        // K: this CTA's 64 keys of the block, all 128 dims, as two [64 rows][64 cols] boxes
                        tma_load_4d_pair(dst, &maps.k, full_bar, 0, key0 + 64 * static_cast<int>(cta), c.w.hkv, c.w.b);
                        tma_load_4d_pair(dst + kSlotBytes / 2, &maps.k, full_bar, 64, key0 + 64 * static_cast<int>(cta), c.w.hkv, c.w.b);
                    } else {
                        // V: all 128 keys of the block, this CTA's 64 dims, one [128 rows][64 cols] box
                        tma_load_4d_pair(dst, &maps.v, full_bar, 64 * static_cast<int>(cta), key0, c.w.hkv, c.w.b);
                    }
                };
                BlockCursor kc, vc;              // K runs two blocks ahead of V
                kc.init(p, n_rounds, n_items, cluster_id, n_clusters, n_cols, n_rows, cta);
                vc = kc;
                for (int pre = 0; pre < 2 && kc.valid && ok; ++pre) { load_q(kc); load_half(kc, false); kc.next(p); }
                while (vc.valid && ok) {
                    if (kc.valid) { load_q(kc); load_half(kc, false); kc.next(p); }
                    load_half(vc, true);
                    vc.next(p);
                }
            }
        } else if (warp == kMmaWarp) {
            // =========================== MMA issuer (leader CTA only) ===========================
            if (leader && lane == 0) {
                constexpr uint32_t idesc_qk = make_idesc_f16(Elem<T>::kFormat, 0, 0, 2 * kBlockM, kBlockN);
                constexpr uint32_t idesc_pv = make_idesc_f16(Elem<T>::kFormat, 0, 1, 2 * kBlockM, kD);
                // Shared-memory matrix descriptors, built once: 128-byte swizzle, 1024 bytes between 8-row groups; per
                // product only the start-address field (low word, in 16-byte units) moves.  The issuing thread's own
                // instruction stream is what bounds the tensor pipe here: every instruction between two MMAs counts.
                const uint64_t desc_q0 = make_smem_desc_sw128(smem_u32(q_smem), 16, 1024);              // Q tile, K-major
                const uint64_t desc_k0 = make_smem_desc_sw128(smem_u32(kv_smem), 16, 1024);             // K half, K-major
                const uint64_t desc_v0 = make_smem_desc_sw128(smem_u32(kv_smem), kBoxBytes, 1024);      // V half, MN-major
                const uint32_t tmem_o = tmem_base + 256;
                int kv_item = 0;
                bool ok = true;
                // S[g & 1] = Q K(block)^T for the block the cursor stands on
                auto issue_qk = [&](const BlockCursor& c) {
                    if (!ok) return;
                    const int qbuf = c.item_no % kQBufs;
                    if (c.j == 0) ok = mbar_wait(&bar->q_rot[qbuf], (c.item_no / kQBufs) & 1, abort_flag, 0x210);
                    // S[g & 1] was last used by block g - 2: both softmax warpgroups must have read it
                    if (ok && c.g >= 2) ok = mbar_wait(&bar->s_free[c.g & 1], ((c.g >> 1) - 1) & 1, abort_flag, 0x220);
                    const int slot = kv_item % kStages;
                    if (ok) ok = mbar_wait(&bar->kv_full[slot], (kv_item / kStages) & 1, abort_flag, 0x200);
                    if (!ok) return;
                    ++kv_item;
                    tc_fence_after();
                    const uint32_t d = tmem_base + static_cast<uint32_t>((c.g & 1) * 128);
                    const uint64_t a0 = desc_q0 + static_cast<uint64_t>(qbuf * (kTileBytes >> 4));
                    const uint64_t b0 = desc_k0 + static_cast<uint64_t>(slot * (kSlotBytes >> 4));
#pragma unroll
                    for (int kk = 0; kk < kD / 16; ++kk) {
                        // A: [128 rows][64 cols] boxes of the Q tile; B: [64 rows][64 cols] boxes of this CTA's K half
                        const uint64_t a = a0 + static_cast<uint64_t>(((kk >> 2) * kBoxBytes + (kk & 3) * 32) >> 4);
                        const uint64_t bd = b0 + static_cast<uint64_t>(((kk >> 2) * (kSlotBytes / 2) + (kk & 3) * 32) >> 4);
                        umma2_ss(d, a, bd, idesc_qk, kk > 0 ? 1u : 0u);
                    }
                    umma2_commit(&bar->s_full[c.g & 1]);
                    umma2_commit(&bar->kv_empty[slot]);
                    if (c.j + 1 == c.w.n) umma2_commit(&bar->q_free[qbuf]);          // last QK of the item
                };
                BlockCursor qk, pv;
                qk.init(p, n_rounds, n_items, cluster_id, n_clusters, n_cols, n_rows, 0);
                pv = qk;
                for (int pre = 0; pre < 2 && qk.valid && ok; ++pre) { issue_qk(qk); qk.next(p); }
                while (pv.valid && ok) {
                    if (qk.valid) { issue_qk(qk); qk.next(p); }
                    if (!ok) break;
                    // O += P[g & 1] V(block)
                    const int b = pv.g & 1;
                    ok = mbar_wait(&bar->p_ready[b], (pv.g >> 1) & 1, abort_flag, 0x400);
                    // the first product of an item overwrites O: the previous item's O must have been drained
                    if (ok && pv.j == 0 && pv.item_no > 0) ok = mbar_wait(&bar->o_free, (pv.item_no - 1) & 1, abort_flag, 0x410);
                    const int slot = kv_item % kStages;
                    if (ok) ok = mbar_wait(&bar->kv_full[slot], (kv_item / kStages) & 1, abort_flag, 0x300);
                    if (!ok) break;
                    ++kv_item;
                    tc_fence_after();
                    const uint32_t a_tmem = tmem_base + static_cast<uint32_t>(384 + b * 64);
                    const uint64_t v0 = desc_v0 + static_cast<uint64_t>(slot * (kSlotBytes >> 4));
                    const uint32_t acc0 = pv.j > 0 ? 1u : 0u;
#pragma unroll
                    for (int kk = 0; kk < kBlockN / 16; ++kk) {
                        // V half is MN-major for this product: 16 keys = 2048 bytes per step, 64 dims per CTA
                        umma2_ts(tmem_o, a_tmem + kk * 8, v0 + static_cast<uint64_t>(kk * (2048 >> 4)), idesc_pv, kk > 0 ? 1u : acc0);
                    }
                    umma2_commit(&bar->pv_done[b]);
                    umma2_commit(&bar->kv_empty[slot]);
                    pv.next(p);
                }
                // everything issued so far has to retire (in both CTAs) before TMEM is released
                umma2_commit(&bar->mma_done);
            }
            __syncwarp();
        } else {
            // =========================== RoPE of this CTA's Q tiles; tells the leader they are ready ===========================
            // 2 warps; warp w owns rows [64w, 64w+64) of the tile.  A step handles two rows: lane l takes 16-byte
            // chunk (l & 15) of row 2*step + (l >> 4).  Without RoPE the warps only forward "tile landed".
            const int rw = warp - kRopeWarp0;
            const int c = lane & 15;
            constexpr int kRopeSeed = 8;                      // steps (of two rows) between exact table reads
            float step_c[4], step_s[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) sincosf(2.0f * p.inv_freq.v[(c * 4 + e) & (kMaxHalfDim - 1)], &step_s[e], &step_c[e]);
            const uint32_t q_rot_leader = map_to_cta(smem_u32(&bar->q_rot[0]), 0);     // the barriers of one kind are contiguous
            bool ok = true;
            BlockCursor it;
            it.init(p, n_rounds, n_items, cluster_id, n_clusters, n_cols, n_rows, cta);
            for (; it.valid && ok; it.next_item(p)) {
                const Item& w = it.w;
                const int b = it.item_no % kQBufs, ph = (it.item_no / kQBufs) & 1;
                ok = mbar_wait_warp(&bar->q_full[b], ph, abort_flag, 0x700 + b);
                if (!ok) break;
                if (rope) {
                    unsigned char* qtile = q_smem + b * kTileBytes + (c >> 3) * kBoxBytes;
                    const int r_first = rw * 64 + (lane >> 4);
                    // rows past T hold zeros: rotating them is harmless; their table row is clamped
                    if constexpr (kExactRope) {
#pragma unroll 2
                        for (int st = 0; st < 32; ++st) {
                            const int r = r_first + 2 * st;
                            const int rowx = min(w.r0 + r, p.T - 1);
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
                            const int row = min(w.r0 + r_first, p.T - 1);
                            const float4* tab = reinterpret_cast<const float4*>(p.q_rope_table + static_cast<long long>(row) * (kD / 2)) + c * 2;
                            seed0 = __ldg(tab); seed1 = __ldg(tab + 1);
                        }
#pragma unroll 1
                        for (int s0 = 0; s0 < 32; s0 += kRopeSeed) {
                            float cs[4] = {seed0.x, seed0.z, seed1.x, seed1.z};
                            float sn[4] = {seed0.y, seed0.w, seed1.y, seed1.w};
                            if (s0 + kRopeSeed < 32) {             // prefetch the next exact seed
                                const int row = min(w.r0 + r_first + 2 * (s0 + kRopeSeed), p.T - 1);
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
                if (lane == 0) mbar_arrive_cluster_release(q_rot_leader + 8 * b);
            }
        }
    } else if (warp < 4) {
        // =========================== softmax (and the rare rescale of O) ===========================
        reg_inc<kRegSoftmax>();
        const int r = tid;                           // row inside the tile = TMEM lane
        const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
        const uint32_t o_addr = tmem_base + lane_base + 256;
        const float scale_log2 = p.scale * kLog2e;
        const uint32_t s_free_leader = map_to_cta(smem_u32(&bar->s_free[0]), 0);
        const uint32_t p_ready_leader = map_to_cta(smem_u32(&bar->p_ready[0]), 0);
        bool ok = true;
        BlockCursor it;
        it.init(p, n_rounds, n_items, cluster_id, n_clusters, n_cols, n_rows, cta);
        while (it.valid && ok) {
            const int n = it.w.n, tile_r0 = it.w.r0, item_no = it.item_no;
            const int row = tile_r0 + r;             // query row; >= T for padding rows (computed on zeros, never stored)
            float m_ref = -INFINITY, l_sum = 0.f;
            for (int j = 0; j < n; ++j) {
                const int g = it.g + j, b = g & 1;
                const uint32_t s_addr = tmem_base + lane_base + static_cast<uint32_t>(b * 128);
                const uint32_t p_addr = tmem_base + lane_base + static_cast<uint32_t>(384 + b * 64);
                ok = mbar_wait_warp(&bar->s_full[b], (g >> 1) & 1, abort_flag, 0x800 + b);
                if (!ok) break;
                tc_fence_after();
                uint32_t s[4][32];
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_ld32(s_addr + c * 32, s[c]);
                tmem_ld_wait();
                // the scores are in registers: the product of block g + 2 may overwrite S[b]
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(s_free_leader + 8 * b);

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
                // a block this row sees nothing of (it belongs to the longer tile of the item) has m_cand = -inf: no growth
                const bool grow = m_cand > m_ref + kRescaleThreshold;      // true on the first block of an item
                if (__any_sync(0xFFFFFFFFu, grow)) {
                    const float m_new = grow ? m_cand : m_ref;
                    const float alpha = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - m_new);
                    if (j > 0) {
                        // every product of this item issued so far (the last one read P of block g - 1) must have landed in O
                        ok = mbar_wait_warp(&bar->pv_done[(g - 1) & 1], ((g - 1) >> 1) & 1, abort_flag, 0x900);
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
                // P[b] was last read by the product of block g - 2
                if (g >= 2) {
                    ok = mbar_wait_warp(&bar->pv_done[b], ((g >> 1) - 1) & 1, abort_flag, 0x910);
                    if (!ok) break;
                    tc_fence_after();
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
                    tmem_st32(p_addr + half * 32, pk);
                }
                l_sum += ((rs[0].x + rs[0].y) + (rs[1].x + rs[1].y)) + ((rs[2].x + rs[2].y) + (rs[3].x + rs[3].y));
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(p_ready_leader + 8 * b);
            }
            if (!ok) break;
            // hand (m, l) of the finished item to the epilogue warpgroup and go straight on to the next item
            // (the epilogue warpgroup read the previous item's pair a whole item ago)
            if (item_no >= 1) ok = mbar_wait_warp(&bar->stat_free, (item_no - 1) & 1, abort_flag, 0x920);
            if (!ok) break;
            stats[r] = make_float2(m_ref, l_sum);
            mbar_arrive(&bar->stat_full);
            it.next_item(p);
        }
    } else {
        // =========================== epilogue of finished items: O / l -> staging tile -> TMA store; LSE ===========================
        const int r = tid - 128;                     // row inside the tile = TMEM lane
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t o_addr = tmem_base + lane_base + 256;
        const uint32_t o_free_leader = map_to_cta(smem_u32(&bar->o_free), 0);
        unsigned char* stage = o_smem;
        bool ok = true;
        bool store_pending = false;                  // thread 0 of the warpgroup: a TMA store may still be reading `stage`
        BlockCursor it;
        it.init(p, n_rounds, n_items, cluster_id, n_clusters, n_cols, n_rows, cta);
        for (; it.valid && ok; it.next_item(p)) {
            const Item& w = it.w;
            const int item_no = it.item_no;
            const int g_last = it.g + w.n - 1;
            const int row = w.r0 + r;
            const bool present = w.r0 < p.T;
            ok = mbar_wait_warp(&bar->stat_full, item_no & 1, abort_flag, 0xA00);
            if (!ok) break;
            const float2 st = stats[r];
            mbar_arrive(&bar->stat_free);
            // the item's last product has landed in O
            ok = mbar_wait_warp(&bar->pv_done[g_last & 1], (g_last >> 1) & 1, abort_flag, 0xA10);
            if (!ok) break;
            tc_fence_after();
            // the previous item's store must have finished reading the staging tile
            if (r == 0) {
                if (store_pending) { bulk_wait_read0(); store_pending = false; }
                mbar_arrive(&bar->stage_free);
            }
            ok = mbar_wait_warp(&bar->stage_free, item_no & 1, abort_flag, 0xA20);
            if (!ok) break;
            const float inv_l = 1.0f / st.y;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                uint32_t o[2][32];
                tmem_ld32(o_addr + (2 * half) * 32, o[0]);
                tmem_ld32(o_addr + (2 * half + 1) * 32, o[1]);
                tmem_ld_wait();
                if (half == 1) {
                    // all of O is in registers (or already staged): the next item's first product may overwrite it
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(o_free_leader);
                }
                // 64 columns = one [128 rows][64 cols] box of the staging tile; 16-byte chunk h2 * 4 + v of this row
                unsigned char* box = stage + half * kBoxBytes + r * 128;
#pragma unroll
                for (int h2 = 0; h2 < 2; ++h2)
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        uint4 out;
                        out.x = Elem<T>::pack2(__uint_as_float(o[h2][8 * v + 0]) * inv_l, __uint_as_float(o[h2][8 * v + 1]) * inv_l);
                        out.y = Elem<T>::pack2(__uint_as_float(o[h2][8 * v + 2]) * inv_l, __uint_as_float(o[h2][8 * v + 3]) * inv_l);
                        out.z = Elem<T>::pack2(__uint_as_float(o[h2][8 * v + 4]) * inv_l, __uint_as_float(o[h2][8 * v + 5]) * inv_l);
                        out.w = Elem<T>::pack2(__uint_as_float(o[h2][8 * v + 6]) * inv_l, __uint_as_float(o[h2][8 * v + 7]) * inv_l);
                        const int chunk = h2 * 4 + v;
                        *reinterpret_cast<uint4*>(box + ((chunk ^ (r & 7)) << 4)) = out;
                    }
            }
            fence_proxy_async_smem();                // this row of the staging tile -> visible to the TMA store
            mbar_arrive(&bar->epi_done);
            if (r == 0) {
                // only the issuing thread waits for the other rows (bounded like every wait)
                if (mbar_wait(&bar->epi_done, item_no & 1, abort_flag, 0xB00) && present) {
                    tma_store_4d(&maps.o, stage, 0, w.r0, w.hq, w.b);
                    tma_store_4d(&maps.o, stage + kBoxBytes, 64, w.r0, w.hq, w.b);
                    bulk_commit();
                    store_pending = true;
                }
            }
            if (p.lse != nullptr && present && row < p.T)
                p.lse[(static_cast<long long>(w.b) * p.Hq + w.hq) * p.T + row] = (st.x + fast_log2(st.y)) * kLn2;
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
    note_prefill_kernel("prefill_pair_kernel");
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
