/*
 * vesper_b200 -- C ABI of the B200 (sm_100a) attention backend.
 *
 * These entry points are what Vesper's CUDA backend seam binds for its
 * attention hot path.  Every function
 *   - borrows all pointers (device memory unless stated), allocates nothing
 *     on the device and frees nothing;
 *   - launches asynchronously on the caller's stream and never synchronises
 *     the device;
 *   - returns VB200_OK or a negative vb200_status (never throws, never aborts).
 * "file:line" citations name the reference interface each entry point stands
 * behind, relative to the reference project root.
 */
#ifndef VESPER_B200_H
#define VESPER_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VB200_ABI_VERSION 1

typedef enum vb200_status {
    VB200_OK = 0,
    VB200_ERR_INVALID_ARG = -1,   /* null pointer, bad shape, Hq % Hkv != 0, ...      */
    VB200_ERR_UNSUPPORTED = -2,   /* dtype / head_dim combination without a kernel    */
    VB200_ERR_ALIGNMENT = -3,     /* pointer or stride not 16-byte aligned            */
    VB200_ERR_WORKSPACE = -4,     /* workspace missing or too small                   */
    VB200_ERR_CUDA = -5,          /* a CUDA runtime/driver call failed                */
    VB200_ERR_NO_DEVICE = -6,     /* no usable sm_100 device                          */
    VB200_ERR_KERNEL_TIMEOUT = -7,/* a bounded in-kernel wait expired (status word)   */
    VB200_ERR_CACHE_OVERFLOW = -8 /* a decode step met a sequence whose new token does
                                     not fit the cache or the planned max_len (status
                                     word; the reference throws from KVCache::update,
                                     src/nn/transformer.cpp:62-66)                     */
} vb200_status;

typedef enum vb200_dtype {
    VB200_F32 = 0,   /* fp32 in/out, fp32 math on CUDA cores                          */
    VB200_BF16 = 1,  /* bf16 in/out, fp32 accumulate                                  */
    VB200_F16 = 2    /* fp16 in/out, fp32 accumulate                                  */
} vb200_dtype;

/* A [B, H, S, D] tensor view: element strides for B, H, S; D is contiguous.
 * Mirrors vesper::Tensor's shape/strides/offset view (include/vesper/core/tensor.h:26-80)
 * with the offset already folded into `ptr`. */
typedef struct vb200_tensor4 {
    void* ptr;
    int64_t stride_b, stride_h, stride_s;
} vb200_tensor4;

/* Rotary embedding in the convention the attention modules use
 * (functional::compute_rope_frequencies + apply_rotary_emb,
 * src/nn/functional.cpp:424-494): adjacent pairs (x[2i], x[2i+1]) rotated by
 * angle float(pos) * inv_freq[i].  inv_freq is a HOST array of D/2 floats, as
 * vb200_rope_inv_freq() fills it (the reference's own fp32 expression). */
typedef struct vb200_rope {
    int32_t enabled;
    const float* inv_freq_host;
} vb200_rope;

/* ---- prefill / flash attention ------------------------------------------
 * One call = for T new tokens at positions start_pos .. start_pos+T-1:
 *   rotate Q and K (if rope.enabled), append rotated K and raw V to the cache
 *   rows [start_pos, start_pos+T) (if k_cache is non-null), then attention of
 *   the T queries over keys [0, start_pos+T), causal = bottom-right aligned
 *   (key j visible to query i iff j <= start_pos + i), GQA by head-group
 *   indexing (kv_head = q_head / (Hq/Hkv)), output O and natural-log LSE.
 * With k_cache == NULL and rope disabled it is exactly the flash op:
 *   replaces flash_attention_cuda_dispatch (src/ops/flash_attention.cpp:28-32,
 *   src/ops/cuda/flash_attention.cu:518-544).
 * With a cache it replaces the chain in GroupedQueryAttention::forward(x,cache,pos)
 *   src/nn/gqa_attention.cpp:124-149 (apply_rotary_emb, KVCache::update,
 *   repeat_kv, scaled_dot_product_attention) and the same chain in
 *   MultiHeadAttention::forward, src/nn/transformer.cpp:184-204.
 */
typedef struct vb200_prefill_args {
    uint32_t struct_size;        /* sizeof(vb200_prefill_args)                       */
    int32_t device;              /* CUDA ordinal, or -1 for the current device       */
    void* stream;                /* cudaStream_t                                     */
    int32_t dtype;               /* vb200_dtype of q,k,v,o and the cache             */
    int32_t B, Hq, Hkv, T, D;    /* T = number of new tokens (query rows)            */
    int32_t start_pos;           /* position of the first new token                  */
    int32_t causal;              /* 0 / 1                                            */
    float scale;                 /* multiplies q.k before max/exp                    */
    vb200_tensor4 q;             /* [B,Hq,T,D]                                       */
    vb200_tensor4 k, v;          /* [B,Hkv,T,D] new keys / values                    */
    vb200_tensor4 o;             /* [B,Hq,T,D] output                                */
    float* lse;                  /* [B,Hq,T] contiguous fp32, nullable               */
    vb200_rope rope;
    vb200_tensor4 k_cache, v_cache; /* [B,Hkv,cap,D]; ptr NULL = no cache            */
    int32_t cache_cap;
    int32_t cache_read_only;     /* 1: the cache already holds the (rotated) keys and
                                    the values of rows [0, start_pos+T); k and v are
                                    ignored (may be NULL) and nothing is written to
                                    the cache -- the T < L shape of
                                    scaled_dot_product_attention,
                                    src/nn/functional.cpp:399-421                     */
    void* workspace;             /* vb200_prefill_workspace_bytes() bytes, 256-aligned */
    size_t workspace_bytes;
} vb200_prefill_args;

size_t vb200_prefill_workspace_bytes(const vb200_prefill_args* a);
int vb200_prefill_fwd(const vb200_prefill_args* a);

/* ---- decode ---------------------------------------------------------------
 * One call = one new token per sequence (T = 1): rotate q and the new k at
 * position seq_lens[b] (if rope.enabled), append k/v at cache row seq_lens[b]
 * (if k_new is non-null), then attention of the one query row over keys
 * [kv_begin, seq_lens[b] + appended) with the Hq/Hkv query heads of a group
 * sharing each K/V fetch, split over `num_splits` CTAs per (b, kv_head) and
 * merged by a log-sum-exp combine.
 * Replaces, for T == 1, the same reference chain as prefill plus the five
 * generic ops of the standard attention path (matmul, div, softmax, matmul,
 * src/nn/functional.cpp:399-421; kernels src/ops/cuda/gemm.cu:257-388,
 * src/ops/cuda/normalization.cu:68-267) and the strided copy behind
 * KVCache::update (src/ops/cuda/copy.cu:17-93).
 *
 * seq_lens is a DEVICE int32[B] holding each sequence's length BEFORE this
 * token; when k_new is given and advance_lens != 0 the kernel stores
 * seq_lens[b] + 1 back after the step (so consecutive calls need no host
 * work).  seq_lens == NULL means every sequence has length `uniform_len`.
 *
 * partial_out != NULL selects the sequence-sharded form (each GPU holds a
 * contiguous shard of the KV sequence): instead of o/lse the kernel writes,
 * per (b, q_head), D+2 floats: O normalised by the shard's own l, then m (max
 * of the scaled scores, natural units), then l (sum of exp(s - m)).  After an
 * all-gather of these records, vb200_lse_combine merges them.  pos_offset is
 * the absolute position of cache row 0 of this shard; q_positions (device
 * int32[B], nullable) gives the query's absolute position for RoPE when it is
 * not pos_offset + seq_lens[b] (i.e. on every shard but the last);
 * append_enabled = 0 makes a shard attend without appending.
 *
 * Capacity: a sequence whose new token would not fit -- seq_lens[b] + 1 greater
 * than cache_cap, or than the max_len the step was planned for -- is not
 * appended, its length is not advanced, it attends to the keys it has, and the
 * device status word records the sequence: vb200_check_kernel_status then
 * returns VB200_ERR_CACHE_OVERFLOW (with seq_lens == NULL the same condition is
 * refused on the host with VB200_ERR_INVALID_ARG).
 */
typedef struct vb200_decode_args {
    uint32_t struct_size;
    int32_t device;
    void* stream;
    int32_t dtype;
    int32_t B, Hq, Hkv, D;
    float scale;
    vb200_tensor4 q;             /* [B,Hq,1,D]                                       */
    vb200_tensor4 k_new, v_new;  /* [B,Hkv,1,D]; ptr NULL = nothing to append        */
    vb200_tensor4 o;             /* [B,Hq,1,D]                                       */
    float* lse;                  /* [B,Hq] fp32, nullable                            */
    vb200_rope rope;
    vb200_tensor4 k_cache, v_cache; /* [B,Hkv,cap,D]                                 */
    int32_t cache_cap;
    int32_t* seq_lens;           /* device int32[B] or NULL                          */
    int32_t uniform_len;         /* used when seq_lens == NULL                       */
    int32_t advance_lens;        /* store len+1 back into seq_lens after appending   */
    int32_t max_len;             /* upper bound of any sequence length after the
                                    step (sizes the split grid); 0 = cache_cap       */
    int32_t num_splits;          /* 0 = choose                                       */
    int64_t pos_offset;          /* absolute position of cache row 0 (sharding)      */
    int32_t append_enabled;      /* 0: ignore k_new/v_new (a shard that does not own
                                    the new token); 1: append and attend to it       */
    const int32_t* q_positions;  /* device int32[B] or NULL                          */
    float* partial_out;          /* NULL, or [B,Hq,D+2] fp32: O/l, then m, then l    */
    void* workspace;
    size_t workspace_bytes;
} vb200_decode_args;

size_t vb200_decode_workspace_bytes(const vb200_decode_args* a);
/* The largest vb200_decode_workspace_bytes of any step these arguments can make
 * as the sequences grow: the maximum over max_len = 1 .. cache_cap, with and
 * without seq_lens (the plan is not monotone in max_len: a shorter step can use
 * more, smaller splits).  Size a buffer once with this and reuse it for every
 * step of a generation (what TransformerLM::forward_with_cache and
 * Generator::generate need, src/models/transformer.cpp:152-188). */
size_t vb200_decode_workspace_bytes_max(const vb200_decode_args* a);
int vb200_decode_fwd(const vb200_decode_args* a);

/* The same decode step for callers that cannot supply a workspace and may not
 * allocate device memory -- e.g. a serving process that has already handed all
 * free HBM to its KV-cache pool, or plugin code inside a framework that owns
 * every device allocation.  No counterpart in the reference (its backends get
 * their buffers from the caller's allocator).  `workspace` and
 * `workspace_bytes` of the argument struct are ignored; the split partials go
 * to an array of VB200_STATIC_SCRATCH_BYTES that is part of the library image
 * on each GPU.  The call allocates and frees nothing.
 *   - A step whose plan needs more than the array holds (compare
 *     vb200_decode_workspace_bytes) returns VB200_ERR_WORKSPACE: lower num_splits
 *     or use vb200_decode_fwd.
 *   - Every call on a GPU shares the array, which keeps the previous call's
 *     contents (none of it needs clearing: a step writes each slot before it
 *     reads it).  Calls that may overlap on one GPU race: keep them on one stream.
 *   - The first call on a device resolves the array's device address; make that
 *     first call before starting any stream capture.  The address is kept for the
 *     life of the process: after a cudaDeviceReset() of that device do not call
 *     this entry point on it again. */
#define VB200_STATIC_SCRATCH_BYTES (16 * 1024 * 1024)
int vb200_decode_fwd_static(const vb200_decode_args* a);

/* Merge R partial results [R, rows, D+2] (layout of partial_out) into
 * out [rows, D] of `dtype` and lse [rows] (nullable):
 *   m* = max m_r,  l* = sum l_r e^{m_r - m*},  O* = sum O_r l_r e^{m_r - m*} / l*
 * -- the online-softmax algebra of src/ops/flash_attention.cpp:309-345 applied
 * across shards. */
int vb200_lse_combine(int device, void* stream, const float* partials, int32_t R,
                      int64_t rows, int32_t D, int32_t dtype, void* out, float* lse);

/* ---- fused exchange + merge for sequence-sharded decode (no reference counterpart) ----------
 * Replaces "all-gather the partial_out records of all ranks, then vb200_lse_combine" by one kernel
 * over NVLink peer memory: every rank stores its records into every rank's exchange buffer as 8-byte words
 * {fp32 value, call number} (plain peer stores; a word is valid as soon as its number matches, so there is no
 * separate flag and no system-wide fence), waits until every rank's words have landed in its own buffer and merges.
 * peer_buffers[r] is rank r's exchange buffer as THIS process addresses it (peer-mapped device
 * memory: CUDA IPC, VMM or a symmetric-memory allocator; entry [rank] is the local buffer); each is
 * vb200_exchange_buffer_bytes(...) long and zero-filled once before the first call.  All ranks
 * must make the same sequence of calls with the same rows / D, and a set of buffers serves ONE entry point
 * (vb200_exchange_combine or vb200_decode_exchange_fwd: they number their calls per exchanging block and cut the
 * rows into blocks differently; mixing them on one buffer ends in the bounded wait's error).  step: 0 = number the calls with
 * a counter kept in the buffer (works under CUDA-graph replay), else a caller-chosen number that
 * grows by one per call.  A rank that never arrives ends the wait after timeout_cycles GPU clock
 * cycles (0 = about one second): the output is left unwritten and vb200_check_kernel_status
 * reports VB200_ERR_KERNEL_TIMEOUT -- the context stays usable. */
#define VB200_EXCHANGE_MAX_WORLD 16
typedef struct vb200_exchange_args {
    size_t struct_size;
    int32_t device;
    void* stream;
    int32_t world, rank;
    void* const* peer_buffers;   /* host array of `world` device pointers */
    const float* partial;        /* local [rows, D+2] records (O/l, m, l) */
    int64_t rows;
    int32_t D;
    int32_t dtype;               /* of out: VB200_BF16 or VB200_F16 */
    void* out;                   /* [rows, D] */
    float* lse;                  /* [rows], nullable */
    uint32_t step;
    int64_t timeout_cycles;
} vb200_exchange_args;
size_t vb200_exchange_buffer_bytes(int32_t world, int64_t rows, int32_t D);
int vb200_exchange_combine(const vb200_exchange_args* a);

/* The whole sequence-sharded decode step of one rank in ONE launch (no reference counterpart): vb200_decode_fwd
 * over this rank's shard of the KV sequence, with the merge of its splits and the exchange above run as the tail of
 * the split kernel -- the CTA that delivers the last split of a (batch, kv_head) merges that group's splits in
 * registers / shared memory, stores the merged records into every rank's exchange buffer, waits (bounded) for the
 * peers' words and writes the final rows.  No combine kernel, no exchange kernel, no partial records in HBM: two
 * launch gaps and two round trips less than vb200_decode_fwd(partial_out) + vb200_exchange_combine, which is what a
 * step of a few microseconds per GPU is made of.
 * `a`: as for vb200_decode_fwd (o, lse, partial_out are ignored; the workspace is needed); `x`: as for
 * vb200_exchange_combine with rows = B * Hq, D and dtype of the decode call (`partial` is ignored; out / lse receive
 * the result).  Needs Hq / Hkv of 4 or 8 and B * Hkv <= 64, without advance_lens; otherwise VB200_ERR_UNSUPPORTED and
 * the two-call form applies.  Every rank must make the same sequence of exchanging calls on its buffer. */
int vb200_decode_exchange_fwd(const vb200_decode_args* a, const vb200_exchange_args* x);

/* ---- attention backward (training; fp32, the reference's training dtype) --------------------
 * dQ, dK, dV of O = softmax(scale Q K^T [causal]) V from the saved O and LSE of the forward, P
 * recomputed tile by tile.  All tensors contiguous [B,H,N,D] fp32 with Hq == Hkv (the reference op
 * takes q, k, v of one shape), lse [B,H,N]; dq, dk, dv are overwritten.  Deterministic (no atomics).
 * workspace: B*H*N floats (vb200_attention_bwd_workspace_bytes).  Replaces
 * flash_attention_backward_cuda_dispatch (src/ops/flash_attention.cpp:34-39,
 * src/ops/cuda/flash_attention.cu:546-576; CPU form src/ops/flash_attention.cpp:366-482); like the
 * reference's CUDA path it has no dropout. */
typedef struct vb200_attention_bwd_args {
    size_t struct_size;
    int32_t device;
    void* stream;
    int32_t dtype;               /* VB200_F32 */
    int32_t B, H, N, D;
    int32_t causal;
    float scale;
    const void *d_out, *q, *k, *v, *out;
    const float* lse;
    void *dq, *dk, *dv;
    void* workspace;
    size_t workspace_bytes;
} vb200_attention_bwd_args;
size_t vb200_attention_bwd_workspace_bytes(const vb200_attention_bwd_args* a);
int vb200_attention_bwd(const vb200_attention_bwd_args* a);

/* ---- cache append without attention ---------------------------------------
 * Rotates K (if rope.enabled) and writes K, V rows [start_pos, start_pos+T)
 * of the cache.  Replaces the copy_strided_cuda_dispatch calls behind
 * KVCache::update (src/nn/transformer.cpp:56-93, src/ops/cuda/copy.cu:75-93). */
int vb200_kv_append(int device, void* stream, int32_t dtype,
                    int32_t B, int32_t Hkv, int32_t T, int32_t D, int32_t start_pos,
                    const vb200_tensor4* k, const vb200_tensor4* v,
                    const vb200_tensor4* k_cache, const vb200_tensor4* v_cache,
                    int32_t cache_cap, const vb200_rope* rope);

/* In-place rotary embedding of x [B,H,S,D] with a caller-built cos/sin table
 * [S, D/2] each.  Replaces apply_rope_cuda (src/nn/rope.cpp:25-28,
 * src/ops/cuda/rope.cu:186-208). */
int vb200_apply_rope(int device, void* stream, float* x, const float* cos_table,
                     const float* sin_table, int32_t batch, int32_t heads,
                     int32_t seq_len, int32_t head_dim);

/* out[b, qh, s, :] = in[b, qh / n_rep, s, :] honouring the input view's strides.
 * Replaces repeat_kv_cuda_dispatch (src/ops/attention_ops.cpp:24-27,
 * src/ops/cuda/attention_ops.cu:69-96).  The attention entry points above do
 * not need it; it exists so the op surface links. */
int vb200_repeat_kv(int device, void* stream, int32_t dtype, const vb200_tensor4* in,
                    void* out, int32_t B, int32_t Hkv, int32_t S, int32_t D, int32_t n_rep);

/* Host helper: inv_freq[i] = powf(theta, -2.0f * i / D), i < D/2 -- the fp32
 * expression of src/nn/functional.cpp:433. */
void vb200_rope_inv_freq(float theta, int32_t D, float* inv_freq_host);

const char* vb200_strerror(int status);
/* Text of the last CUDA error seen by the calling thread (empty if none). */
const char* vb200_last_error_detail(void);
int vb200_abi_version(void);
/* Number of kernels launched by this library from the calling thread since
 * the last reset (used by the benchmark's launch count). */
uint64_t vb200_launch_count(void);
void vb200_reset_launch_count(void);
/* Name of the attention kernel the calling thread's last vb200_prefill_fwd launched ("prefill_sm100_kernel",
 * "prefill_pair_kernel", "prefill_f32_kernel"; "" before the first call): which of the kernels a shape, a dtype or the
 * VB200_PREFILL_KERNEL switch selected, for reports and tests. */
const char* vb200_last_prefill_kernel(void);
/* Optional timing of the dominant kernel of each call (the attention kernel of
 * vb200_prefill_fwd, the split-KV kernel of vb200_decode_fwd), for roofline
 * reports: while enabled, the launch is bracketed by two CUDA events on the
 * caller's stream; vb200_profile_read returns the summed kernel time and the
 * number of brackets since the last enable (it waits for the last one).
 * Per calling thread.  Because a bracket is folded in when the next one starts,
 * enabling this makes consecutive calls wait for each other's kernels: do not
 * leave it on in production. */
int vb200_profile_enable(int enable);
int vb200_profile_read(double* total_ms, uint64_t* launches);
/* Reads and clears the device-side status word that bounded waits and the decode
 * kernels' capacity check set (synchronises the given stream).  Returns VB200_OK,
 * VB200_ERR_KERNEL_TIMEOUT or VB200_ERR_CACHE_OVERFLOW. */
int vb200_check_kernel_status(int device, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* VESPER_B200_H */
