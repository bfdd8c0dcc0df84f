// extern "C" entry points of libvesper_b200: argument validation, workspace
// carving and kernel orchestration.  No device allocation, no synchronisation
// (except vb200_check_kernel_status, which is documented to synchronise).
#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>

#include "kernels.h"

namespace vb200 {

__device__ int g_kernel_status = 0;

int* kernel_status_word() {
    // one symbol instance per device; cache the address per ordinal
    static thread_local int* cache[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!cache[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_kernel_status) != cudaSuccess) return nullptr;
        cache[dev] = static_cast<int*>(p);
    }
    return cache[dev];
}

namespace {
thread_local std::string t_detail;
thread_local uint64_t t_launches = 0;
thread_local const char* t_prefill_kernel = "";
}  // namespace

void note_launch(int n) { t_launches += static_cast<uint64_t>(n); }
void note_prefill_kernel(const char* name) { t_prefill_kernel = name; }

namespace {
struct ProfileState {
    bool enabled = false;
    int dev = -1;
    cudaEvent_t ev[2] = {nullptr, nullptr};
    double total_ms = 0.0;
    uint64_t count = 0;
    bool pending = false;
};
thread_local ProfileState t_prof;

// fold the last bracket into the running total (waits for its end event)
void profile_flush() {
    if (!t_prof.pending) return;
    float ms = 0.f;
    if (cudaEventSynchronize(t_prof.ev[1]) == cudaSuccess && cudaEventElapsedTime(&ms, t_prof.ev[0], t_prof.ev[1]) == cudaSuccess) {
        t_prof.total_ms += ms;
        t_prof.count += 1;
    }
    t_prof.pending = false;
}
}  // namespace

void profile_mark_begin(cudaStream_t s) {
    if (!t_prof.enabled) return;
    profile_flush();
    cudaEventRecord(t_prof.ev[0], s);
}
void profile_mark_end(cudaStream_t s) {
    if (!t_prof.enabled) return;
    cudaEventRecord(t_prof.ev[1], s);
    t_prof.pending = true;
}

int cuda_fail(cudaError_t e, const char* what) {
    t_detail = std::string(what) + ": " + cudaGetErrorString(e);
    return VB200_ERR_CUDA;
}

int set_detail(int status, const char* msg) {
    t_detail = msg;
    return status;
}

namespace {

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
inline int elem_size(int dtype) { return dtype == VB200_F32 ? 4 : 2; }
inline bool dtype_ok(int dtype) { return dtype == VB200_F32 || dtype == VB200_BF16 || dtype == VB200_F16; }

// 16-byte alignment of the base and of every stride, which both the vector
// loads and the TMA descriptors need.
bool view_aligned(const vb200_tensor4& t, int esz) {
    auto ok = [&](long long s) { return (s * esz) % 16 == 0; };
    return (reinterpret_cast<uintptr_t>(t.ptr) % 16 == 0) && ok(t.stride_b) && ok(t.stride_h) && ok(t.stride_s);
}

struct PrefillPlan {
    bool need_table, need_krot;   // krot: rotated K without a cache goes to the workspace
    size_t table_bytes, krot_bytes, total;
};

PrefillPlan plan_prefill(const vb200_prefill_args* a) {
    PrefillPlan pl{};
    pl.need_table = a->rope.enabled != 0;
    pl.need_krot = a->rope.enabled && a->k_cache.ptr == nullptr;
    pl.table_bytes = pl.need_table ? align_up(static_cast<size_t>(a->T) * (a->D / 2) * sizeof(float2), 256) : 0;
    pl.krot_bytes = pl.need_krot ? align_up(static_cast<size_t>(a->B) * a->Hkv * a->T * a->D * elem_size(a->dtype), 256) : 0;
    pl.total = pl.table_bytes + pl.krot_bytes;
    return pl;
}

int validate_prefill(const vb200_prefill_args* a) {
    if (!a || a->struct_size != sizeof(vb200_prefill_args)) return set_detail(VB200_ERR_INVALID_ARG, "vb200_prefill_args: null or struct_size mismatch");
    if (!dtype_ok(a->dtype)) return set_detail(VB200_ERR_UNSUPPORTED, "unknown dtype");
    if (a->B <= 0 || a->Hq <= 0 || a->Hkv <= 0 || a->T <= 0 || a->D <= 0) return set_detail(VB200_ERR_INVALID_ARG, "B, Hq, Hkv, T, D must be positive");
    if (a->Hq % a->Hkv != 0) return set_detail(VB200_ERR_INVALID_ARG, "Hq must be divisible by Hkv");
    if (a->start_pos < 0) return set_detail(VB200_ERR_INVALID_ARG, "start_pos must be >= 0");
    if (!a->q.ptr || !a->o.ptr) return set_detail(VB200_ERR_INVALID_ARG, "q, k, v, o must be non-null");
    const bool ro = a->cache_read_only != 0;
    if (ro && !a->k_cache.ptr) return set_detail(VB200_ERR_INVALID_ARG, "cache_read_only needs k_cache and v_cache");
    if (!ro && (!a->k.ptr || !a->v.ptr)) return set_detail(VB200_ERR_INVALID_ARG, "q, k, v, o must be non-null");
    if (a->D % 8 != 0 || a->D > 128) return set_detail(VB200_ERR_UNSUPPORTED, "head_dim must be a multiple of 8 and <= 128");
    // checked here, ahead of every launch: a call either does all of its work or none of it
    if (a->dtype != VB200_F32 && a->D != 64 && a->D != 128) return set_detail(VB200_ERR_UNSUPPORTED, "bf16/fp16 attention supports head_dim 64 and 128");
    if ((a->k_cache.ptr == nullptr) != (a->v_cache.ptr == nullptr)) return set_detail(VB200_ERR_INVALID_ARG, "k_cache and v_cache must both be given or both be null");
    if (a->k_cache.ptr) {
        if (a->start_pos + a->T > a->cache_cap) return set_detail(VB200_ERR_INVALID_ARG, "start_pos + T exceeds the cache capacity");
    } else if (a->start_pos != 0) {
        return set_detail(VB200_ERR_INVALID_ARG, "start_pos > 0 needs a cache holding the earlier keys");
    }
    if (a->rope.enabled && !a->rope.inv_freq_host) return set_detail(VB200_ERR_INVALID_ARG, "rope enabled without inv_freq_host");
    int esz = elem_size(a->dtype);
    if (!view_aligned(a->q, esz) || !view_aligned(a->o, esz) || (!ro && (!view_aligned(a->k, esz) || !view_aligned(a->v, esz))))
        return set_detail(VB200_ERR_ALIGNMENT, "q/k/v/o base and strides must be 16-byte aligned");
    if (a->k_cache.ptr && (!view_aligned(a->k_cache, esz) || !view_aligned(a->v_cache, esz)))
        return set_detail(VB200_ERR_ALIGNMENT, "cache base and strides must be 16-byte aligned");
    return VB200_OK;
}

void fill_inv_freq(InvFreq& f, const vb200_rope& r, int D) {
    std::memset(&f, 0, sizeof(f));
    if (r.enabled) std::memcpy(f.v, r.inv_freq_host, sizeof(float) * (D / 2));
}

struct DecodePlan {
    int num_splits, chunk, ws_header;
    size_t total;
};

// Streaming multiprocessors of the current device, asked once per ordinal (148 where no device answers,
// e.g. when only workspace sizes are computed on a machine without a GPU).
int sm_count() {
    static int cache[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { (void)cudaGetLastError(); return 148; }
    if (cache[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) { (void)cudaGetLastError(); n = 148; }
        cache[dev] = n;
    }
    return cache[dev];
}

// `waves`: CTAs per SM the split count aims at (4 = two waves of two resident CTAs; the one-launch sharded step asks
// for 1: one CTA per SM, so that the last CTA of a group finds few enough partial records to merge them from shared
// memory in one round).
DecodePlan plan_decode(const vb200_decode_args* a, int waves = 4) {
    DecodePlan pl{};
    const int tile = decode_tile_keys();
    int max_total = (a->max_len > 0 ? a->max_len : a->cache_cap);
    if (max_total < 1) max_total = 1;
    int chunk;
    if (a->num_splits > 0) {
        chunk = (max_total + a->num_splits - 1) / a->num_splits;
    } else {
        // enough CTAs for about two waves of 2 CTAs per SM; with per-sequence lengths never
        // more than 2048 keys per CTA so ragged batches balance (one common length needs no such cap:
        // longer chunks spend less of a CTA's life in its prologue and merge)
        long long units = static_cast<long long>(a->B) * a->Hkv;
        if (!a->seq_lens && waves == 4) {
            // One common length: nothing to balance, so fewer and longer chunks win (measured on 8 groups of 8 heads, split
            // kernel + combine from a graph: 131072 keys 95.4 us with four CTAs per SM, 90.5 with two, 88.8 with one; 16384
            // keys 23.5 / 16.6 / 17.3 us): one CTA per SM once a CTA of the two-per-SM plan would stream 1024 keys or more.
            const long long two = std::max<long long>(1, 2LL * sm_count() / units);
            waves = (max_total / two >= 1024) ? 1 : 2;
        }
        const long long ctas = static_cast<long long>(waves) * sm_count();
        // (one wave: rounded down, so that no SM gets a second CTA -- it would finish last, at twice the time)
        int want = waves == 1 ? static_cast<int>(ctas / units) : static_cast<int>((ctas + units - 1) / units);
        if (want < 1) want = 1;
        chunk = (max_total + want - 1) / want;
        // (measured on 256 groups with 1024-8192 keys each, 256 steps: 5.63 TB/s per step with a cap of 512 keys, 5.82 with
        // 768, 5.94 with 1280, 5.98 with 2048, 5.92 with 4096: a CTA's prologue and merge cost more than the imbalance)
        if (chunk > 2048 && a->seq_lens) chunk = 2048;
        // short contexts: at most 16 splits, so that they can run as one cluster that merges its own partials
        if (max_total <= 16 * 2 * tile && (max_total + chunk - 1) / chunk > 16) chunk = (max_total + 15) / 16;
    }
    chunk = (chunk + tile - 1) / tile * tile;
    if (chunk < tile) chunk = tile;
    pl.chunk = chunk;
    pl.num_splits = (max_total + chunk - 1) / chunk;
    pl.ws_header = (a->B + 63) / 64 * 64;
    int nrep = a->Hq / a->Hkv;
    pl.total = sizeof(float) * (static_cast<size_t>(pl.ws_header) +
                                static_cast<size_t>(a->B) * a->Hkv * pl.num_splits * nrep * (a->D + 2));
    pl.total = align_up(pl.total, 256);
    return pl;
}

int validate_decode(const vb200_decode_args* a) {
    if (!a || a->struct_size != sizeof(vb200_decode_args)) return set_detail(VB200_ERR_INVALID_ARG, "vb200_decode_args: null or struct_size mismatch");
    if (!dtype_ok(a->dtype)) return set_detail(VB200_ERR_UNSUPPORTED, "unknown dtype");
    if (a->B <= 0 || a->Hq <= 0 || a->Hkv <= 0 || a->D <= 0) return set_detail(VB200_ERR_INVALID_ARG, "B, Hq, Hkv, D must be positive");
    if (a->Hq % a->Hkv != 0) return set_detail(VB200_ERR_INVALID_ARG, "Hq must be divisible by Hkv");
    if (!a->q.ptr || !a->k_cache.ptr || !a->v_cache.ptr) return set_detail(VB200_ERR_INVALID_ARG, "q, k_cache, v_cache must be non-null");
    // (vb200_decode_exchange_fwd writes through its exchange arguments and passes neither)
    if ((a->k_new.ptr == nullptr) != (a->v_new.ptr == nullptr)) return set_detail(VB200_ERR_INVALID_ARG, "k_new and v_new must both be given or both be null");
    if (a->cache_cap <= 0) return set_detail(VB200_ERR_INVALID_ARG, "cache_cap must be positive");
    if (!a->seq_lens && (a->uniform_len < 0 || a->uniform_len + (a->k_new.ptr ? 1 : 0) > a->cache_cap))
        return set_detail(VB200_ERR_INVALID_ARG, "uniform_len out of range for the cache");
    if (a->rope.enabled && !a->rope.inv_freq_host) return set_detail(VB200_ERR_INVALID_ARG, "rope enabled without inv_freq_host");
    int esz = elem_size(a->dtype);
    if (!view_aligned(a->q, esz) || !view_aligned(a->k_cache, esz) || !view_aligned(a->v_cache, esz))
        return set_detail(VB200_ERR_ALIGNMENT, "q / cache base and strides must be 16-byte aligned");
    if (a->k_new.ptr && (!view_aligned(a->k_new, esz) || !view_aligned(a->v_new, esz)))
        return set_detail(VB200_ERR_ALIGNMENT, "k_new / v_new base and strides must be 16-byte aligned");
    if (a->o.ptr && !view_aligned(a->o, esz)) return set_detail(VB200_ERR_ALIGNMENT, "o base and strides must be 16-byte aligned");
    return VB200_OK;
}

}  // namespace
}  // namespace vb200

using namespace vb200;

extern "C" {

int vb200_abi_version(void) { return VB200_ABI_VERSION; }

const char* vb200_strerror(int status) {
    switch (status) {
        case VB200_OK: return "ok";
        case VB200_ERR_INVALID_ARG: return "invalid argument";
        case VB200_ERR_UNSUPPORTED: return "unsupported dtype / head_dim / layout";
        case VB200_ERR_ALIGNMENT: return "pointer or stride not 16-byte aligned";
        case VB200_ERR_WORKSPACE: return "workspace missing or too small";
        case VB200_ERR_CUDA: return "CUDA error";
        case VB200_ERR_NO_DEVICE: return "no usable CUDA device";
        case VB200_ERR_KERNEL_TIMEOUT: return "a bounded in-kernel wait expired";
        case VB200_ERR_CACHE_OVERFLOW: return "a sequence's new token does not fit the KV cache / planned max_len";
        default: return "unknown status";
    }
}

const char* vb200_last_error_detail(void) { return t_detail.c_str(); }
uint64_t vb200_launch_count(void) { return t_launches; }
const char* vb200_last_prefill_kernel(void) { return t_prefill_kernel; }
void vb200_reset_launch_count(void) { t_launches = 0; }

void vb200_rope_inv_freq(float theta, int32_t D, float* inv_freq_host) {
    // src/nn/functional.cpp:433: std::pow(theta, -2.0f * i / dim), all fp32
    for (int i = 0; i < D / 2; ++i) inv_freq_host[i] = std::pow(theta, -2.0f * i / D);
}

int vb200_check_kernel_status(int device, void* stream) {
    DeviceGuard g;
    if (int rc = g.init(device)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int host = 0;
    VB200_CUDA_TRY(cudaMemcpyFromSymbolAsync(&host, g_kernel_status, sizeof(int), 0, cudaMemcpyDeviceToHost, s));
    VB200_CUDA_TRY(cudaStreamSynchronize(s));
    if (host == 0) return VB200_OK;
    int zero = 0;
    VB200_CUDA_TRY(cudaMemcpyToSymbolAsync(g_kernel_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, s));
    VB200_CUDA_TRY(cudaStreamSynchronize(s));
    char buf[96];
    if ((host >> 24) == 2) {
        std::snprintf(buf, sizeof(buf), "decode: sequence %d is full (token not appended, length not advanced)", host & 0xFFFFFF);
        return set_detail(VB200_ERR_CACHE_OVERFLOW, buf);
    }
    std::snprintf(buf, sizeof(buf), "kernel wait expired: code %d, site 0x%x", host >> 24, host & 0xFFFFFF);
    return set_detail(VB200_ERR_KERNEL_TIMEOUT, buf);
}

int vb200_profile_enable(int enable) {
    if (enable) {
        int dev = 0;
        VB200_CUDA_TRY(cudaGetDevice(&dev));
        if (t_prof.ev[0] && t_prof.dev != dev) {
            cudaEventDestroy(t_prof.ev[0]); cudaEventDestroy(t_prof.ev[1]);
            t_prof.ev[0] = t_prof.ev[1] = nullptr;
        }
        if (!t_prof.ev[0]) {
            VB200_CUDA_TRY(cudaEventCreate(&t_prof.ev[0]));
            VB200_CUDA_TRY(cudaEventCreate(&t_prof.ev[1]));
            t_prof.dev = dev;
        }
        t_prof.total_ms = 0.0; t_prof.count = 0; t_prof.pending = false;
        t_prof.enabled = true;
    } else {
        profile_flush();
        t_prof.enabled = false;
    }
    return VB200_OK;
}

int vb200_profile_read(double* total_ms, uint64_t* launches) {
    profile_flush();
    if (total_ms) *total_ms = t_prof.total_ms;
    if (launches) *launches = t_prof.count;
    return VB200_OK;
}

size_t vb200_prefill_workspace_bytes(const vb200_prefill_args* a) {
    if (!a || a->struct_size != sizeof(vb200_prefill_args)) return 0;
    return plan_prefill(a).total;
}

int vb200_prefill_fwd(const vb200_prefill_args* a) {
    if (int rc = validate_prefill(a)) return rc;
    PrefillPlan pl = plan_prefill(a);
    if (pl.total > 0) {
        if (!a->workspace || a->workspace_bytes < pl.total) return set_detail(VB200_ERR_WORKSPACE, "prefill workspace too small (see vb200_prefill_workspace_bytes)");
        if (reinterpret_cast<uintptr_t>(a->workspace) % 256 != 0) return set_detail(VB200_ERR_ALIGNMENT, "workspace must be 256-byte aligned");
    }
    DeviceGuard g;
    if (int rc = g.init(a->device)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(a->stream);

    float2* table = nullptr;
    unsigned char* ws = static_cast<unsigned char*>(a->workspace);
    InvFreq f;
    fill_inv_freq(f, a->rope, a->D);
    if (pl.need_table) table = reinterpret_cast<float2*>(ws);
    const bool ro = a->k_cache.ptr && a->cache_read_only;
    // the table alone is needed when nothing is appended or rotated beside Q (read-only cache)
    if (pl.need_table && ro) {
        if (int rc = launch_rope_table(s, table, a->T, a->D, a->start_pos, f)) return rc;
    }

    PrefillParams p{};
    p.dtype = a->dtype;
    p.B = a->B; p.Hq = a->Hq; p.Hkv = a->Hkv; p.T = a->T; p.D = a->D;
    p.Skv = a->start_pos + a->T;
    p.start_pos = a->start_pos;
    p.causal = a->causal;
    p.scale = a->scale;
    p.q = to_view(a->q);
    p.o = to_view(a->o);
    p.lse = a->lse;
    p.q_rope_table = table;
    p.inv_freq = f;
    p.status = kernel_status_word();
    if (!p.status) return set_detail(VB200_ERR_CUDA, "cannot resolve the device status word");

    if (ro) {
        // the cache already holds every key and value this call attends to
        p.k = to_view(a->k_cache);
        p.v = to_view(a->v_cache);
    } else if (a->k_cache.ptr) {
        // RoPE table + RoPE(K) + append in one launch; attention then reads K/V straight from the cache
        if (pl.need_table) {
            if (int rc = launch_rope_append_fused(s, a->dtype, a->B, a->Hkv, a->T, a->D, to_view(a->k), to_view(a->v),
                                                  to_view(a->k_cache), to_view(a->v_cache), a->start_pos, table, f)) return rc;
        } else if (int rc = launch_kv_append(s, a->dtype, a->B, a->Hkv, a->T, a->D, to_view(a->k), to_view(a->v),
                                             to_view(a->k_cache), to_view(a->v_cache), a->start_pos, nullptr)) return rc;
        p.k = to_view(a->k_cache);
        p.v = to_view(a->v_cache);
    } else if (pl.need_krot) {
        View4 krot{ws + pl.table_bytes, static_cast<long long>(a->Hkv) * a->T * a->D, static_cast<long long>(a->T) * a->D, a->D};
        if (int rc = launch_rope_append_fused(s, a->dtype, a->B, a->Hkv, a->T, a->D, to_view(a->k), View4{nullptr, 0, 0, 0},
                                              krot, View4{nullptr, 0, 0, 0}, 0, table, f)) return rc;
        p.k = krot;
        p.v = to_view(a->v);
    } else {
        p.k = to_view(a->k);
        p.v = to_view(a->v);
    }

    if (a->dtype == VB200_F32) return launch_prefill_f32(s, p);
    return launch_prefill_sm100(s, p);
}

size_t vb200_decode_workspace_bytes(const vb200_decode_args* a) {
    if (!a || a->struct_size != sizeof(vb200_decode_args)) return 0;
    if (a->B <= 0 || a->Hkv <= 0 || a->Hq <= 0 || a->D <= 0 || a->Hq % a->Hkv != 0) return 0;
    return plan_decode(a).total;
}

size_t vb200_decode_workspace_bytes_max(const vb200_decode_args* a) {
    if (!a || a->struct_size != sizeof(vb200_decode_args)) return 0;
    if (a->B <= 0 || a->Hkv <= 0 || a->Hq <= 0 || a->D <= 0 || a->Hq % a->Hkv != 0 || a->cache_cap <= 0) return 0;
    vb200_decode_args t = *a;
    int32_t lens_tag = 0;                       // only the pointer's presence enters the plan
    size_t best = 0;
    for (int with_lens = 0; with_lens < 2; ++with_lens) {
        t.seq_lens = with_lens ? &lens_tag : nullptr;
        for (int len = 1; len <= a->cache_cap; ++len) {
            t.max_len = len;
            const size_t n = plan_decode(&t).total;
            if (n > best) best = n;
        }
    }
    return best;
}

namespace {
// Fills the exchange parameters from the C struct (validation shared by both entry points that exchange).
int fill_exchange(ExchangeParams& p, const vb200_exchange_args* a, const char* who) {
    if (!a || a->struct_size != sizeof(vb200_exchange_args)) return set_detail(VB200_ERR_INVALID_ARG, "vb200_exchange_args: null or struct_size mismatch");
    if (a->world <= 0 || a->world > VB200_EXCHANGE_MAX_WORLD || a->rank < 0 || a->rank >= a->world)
        return set_detail(VB200_ERR_INVALID_ARG, "exchange: world must be in [1, 16] and rank in [0, world)");
    if (!a->peer_buffers || !a->out || a->rows <= 0 || a->D <= 0 || a->D % 2 != 0)
        return set_detail(VB200_ERR_INVALID_ARG, "exchange: null pointer, rows <= 0 or odd D");
    if (a->dtype != VB200_BF16 && a->dtype != VB200_F16) return set_detail(VB200_ERR_UNSUPPORTED, "exchange: out must be bf16 or fp16");
    p = ExchangeParams{};
    p.world = a->world; p.rank = a->rank;
    for (int r = 0; r < a->world; ++r) {
        if (!a->peer_buffers[r] || reinterpret_cast<uintptr_t>(a->peer_buffers[r]) % 128 != 0)
            return set_detail(VB200_ERR_ALIGNMENT, "exchange: every exchange buffer must be non-null and 128-byte aligned");
        p.peers[r] = a->peer_buffers[r];
    }
    p.partial = a->partial; p.rows = a->rows; p.D = a->D; p.dtype = a->dtype; p.out = a->out; p.lse = a->lse;
    p.step = a->step; p.timeout_cycles = a->timeout_cycles > 0 ? a->timeout_cycles : kWaitCycles;
    (void)who;
    return VB200_OK;
}

int decode_impl(const vb200_decode_args* a, const vb200_exchange_args* x) {
    if (int rc = validate_decode(a)) return rc;
    if (!x && !a->o.ptr && !a->partial_out) return set_detail(VB200_ERR_INVALID_ARG, "o or partial_out must be given");
    if (a->D % 8 != 0 || a->D > 128) return set_detail(VB200_ERR_UNSUPPORTED, "head_dim must be a multiple of 8 and <= 128");
    DecodePlan pl = plan_decode(a, x ? 1 : 4);
    if (!a->workspace || a->workspace_bytes < pl.total) return set_detail(VB200_ERR_WORKSPACE, "decode workspace too small (see vb200_decode_workspace_bytes)");
    if (reinterpret_cast<uintptr_t>(a->workspace) % 256 != 0) return set_detail(VB200_ERR_ALIGNMENT, "workspace must be 256-byte aligned");
    DeviceGuard g;
    if (int rc = g.init(a->device)) return rc;

    DecodeParams p{};
    p.dtype = a->dtype;
    p.B = a->B; p.Hq = a->Hq; p.Hkv = a->Hkv; p.D = a->D;
    p.scale = a->scale;
    p.q = to_view(a->q);
    p.k_new = to_view(a->k_new);
    p.v_new = to_view(a->v_new);
    p.o = to_view(a->o);
    p.lse = a->lse;
    p.k_cache = to_view(a->k_cache);
    p.v_cache = to_view(a->v_cache);
    p.cache_cap = a->cache_cap;
    p.seq_lens = a->seq_lens;
    p.uniform_len = a->uniform_len;
    p.advance_lens = a->advance_lens;
    p.append = (a->k_new.ptr != nullptr && a->append_enabled) ? 1 : 0;
    p.rope = a->rope.enabled;
    fill_inv_freq(p.inv_freq, a->rope, a->D);
    p.pos_offset = a->pos_offset;
    p.q_positions = a->q_positions;
    p.num_splits = pl.num_splits;
    p.chunk = pl.chunk;
    p.partial_out = a->partial_out;
    p.workspace = static_cast<float*>(a->workspace);
    p.ws_header = pl.ws_header;
    p.status = kernel_status_word();
    if (!p.status) return set_detail(VB200_ERR_CUDA, "cannot resolve the device status word");
    if (x) {
        if (int rc = fill_exchange(p.xchg, x, "vb200_decode_exchange_fwd")) return rc;
        if (x->rows != static_cast<int64_t>(a->B) * a->Hq || x->D != a->D || x->dtype != a->dtype)
            return set_detail(VB200_ERR_INVALID_ARG, "vb200_decode_exchange_fwd: the exchange must carry B * Hq rows of head_dim D in the decode dtype");
        if (pl.num_splits > 1024) return set_detail(VB200_ERR_UNSUPPORTED, "vb200_decode_exchange_fwd: at most 1024 splits");
        if (static_cast<int64_t>(a->B) * a->Hkv > 64)
            return set_detail(VB200_ERR_UNSUPPORTED, "vb200_decode_exchange_fwd: at most 64 (batch, kv_head) groups; use vb200_decode_fwd + vb200_exchange_combine");
        if (p.seq_lens && p.advance_lens && p.append)
            return set_detail(VB200_ERR_UNSUPPORTED, "vb200_decode_exchange_fwd: advance_lens needs the two-call form");
        p.xchg.status = p.status;
        p.fused_exchange = 1;
        p.partial_out = nullptr;
    }
    return launch_decode(static_cast<cudaStream_t>(a->stream), p);
}
}  // namespace

int vb200_decode_fwd(const vb200_decode_args* a) { return decode_impl(a, nullptr); }

int vb200_decode_exchange_fwd(const vb200_decode_args* a, const vb200_exchange_args* x) {
    if (!x) return set_detail(VB200_ERR_INVALID_ARG, "vb200_decode_exchange_fwd: null exchange arguments");
    return decode_impl(a, x);
}

int vb200_lse_combine(int device, void* stream, const float* partials, int32_t R,
                      int64_t rows, int32_t D, int32_t dtype, void* out, float* lse) {
    if (!partials || !out || R <= 0 || rows < 0 || D <= 0) return set_detail(VB200_ERR_INVALID_ARG, "vb200_lse_combine: bad arguments");
    DeviceGuard g;
    if (int rc = g.init(device)) return rc;
    return launch_lse_combine(static_cast<cudaStream_t>(stream), partials, R, rows, D, dtype, out, lse);
}

int vb200_kv_append(int device, void* stream, int32_t dtype,
                    int32_t B, int32_t Hkv, int32_t T, int32_t D, int32_t start_pos,
                    const vb200_tensor4* k, const vb200_tensor4* v,
                    const vb200_tensor4* k_cache, const vb200_tensor4* v_cache,
                    int32_t cache_cap, const vb200_rope* rope) {
    if (!k || !v || !k_cache || !v_cache || !k->ptr || !v->ptr || !k_cache->ptr || !v_cache->ptr)
        return set_detail(VB200_ERR_INVALID_ARG, "vb200_kv_append: null tensor");
    if (!dtype_ok(dtype)) return set_detail(VB200_ERR_UNSUPPORTED, "unknown dtype");
    if (B <= 0 || Hkv <= 0 || T <= 0 || D <= 0 || D % 8 != 0) return set_detail(VB200_ERR_INVALID_ARG, "vb200_kv_append: bad shape");
    if (start_pos < 0 || start_pos + T > cache_cap) return set_detail(VB200_ERR_INVALID_ARG, "vb200_kv_append: rows exceed the cache capacity");
    if (rope && rope->enabled && !rope->inv_freq_host) return set_detail(VB200_ERR_INVALID_ARG, "rope enabled without inv_freq_host");
    int esz = elem_size(dtype);
    if (!view_aligned(*k, esz) || !view_aligned(*v, esz) || !view_aligned(*k_cache, esz) || !view_aligned(*v_cache, esz))
        return set_detail(VB200_ERR_ALIGNMENT, "vb200_kv_append: 16-byte alignment required");
    DeviceGuard g;
    if (int rc = g.init(device)) return rc;
    InvFreq f;
    bool rot = rope && rope->enabled;
    if (rot) fill_inv_freq(f, *rope, D);
    return launch_kv_append(static_cast<cudaStream_t>(stream), dtype, B, Hkv, T, D, to_view(*k), to_view(*v),
                            to_view(*k_cache), to_view(*v_cache), start_pos, nullptr, rot ? &f : nullptr);
}

int vb200_apply_rope(int device, void* stream, float* x, const float* cos_table,
                     const float* sin_table, int32_t batch, int32_t heads,
                     int32_t seq_len, int32_t head_dim) {
    if (!x || !cos_table || !sin_table || batch <= 0 || heads <= 0 || seq_len <= 0 || head_dim <= 0 || head_dim % 2 != 0)
        return set_detail(VB200_ERR_INVALID_ARG, "vb200_apply_rope: bad arguments");
    if (reinterpret_cast<uintptr_t>(x) % 8 != 0) return set_detail(VB200_ERR_ALIGNMENT, "vb200_apply_rope: x must be 8-byte aligned");
    DeviceGuard g;
    if (int rc = g.init(device)) return rc;
    return launch_apply_rope_f32(static_cast<cudaStream_t>(stream), x, cos_table, sin_table, batch, heads, seq_len, head_dim);
}

int vb200_repeat_kv(int device, void* stream, int32_t dtype, const vb200_tensor4* in,
                    void* out, int32_t B, int32_t Hkv, int32_t S, int32_t D, int32_t n_rep) {
    if (!in || !in->ptr || !out || B <= 0 || Hkv <= 0 || S <= 0 || D <= 0 || n_rep <= 0 || D % 8 != 0)
        return set_detail(VB200_ERR_INVALID_ARG, "vb200_repeat_kv: bad arguments");
    if (!dtype_ok(dtype)) return set_detail(VB200_ERR_UNSUPPORTED, "unknown dtype");
    if (!view_aligned(*in, elem_size(dtype)) || reinterpret_cast<uintptr_t>(out) % 16 != 0)
        return set_detail(VB200_ERR_ALIGNMENT, "vb200_repeat_kv: 16-byte alignment required");
    DeviceGuard g;
    if (int rc = g.init(device)) return rc;
    return launch_repeat_kv(static_cast<cudaStream_t>(stream), dtype, to_view(*in), out, B, Hkv, S, D, n_rep);
}

size_t vb200_attention_bwd_workspace_bytes(const vb200_attention_bwd_args* a) {
    if (!a || a->struct_size != sizeof(vb200_attention_bwd_args) || a->B <= 0 || a->H <= 0 || a->N <= 0) return 0;
    return align_up(sizeof(float) * static_cast<size_t>(a->B) * a->H * a->N, 256);
}

int vb200_attention_bwd(const vb200_attention_bwd_args* a) {
    if (!a || a->struct_size != sizeof(vb200_attention_bwd_args)) return set_detail(VB200_ERR_INVALID_ARG, "vb200_attention_bwd_args: null or struct_size mismatch");
    if (a->dtype != VB200_F32) return set_detail(VB200_ERR_UNSUPPORTED, "vb200_attention_bwd: fp32 only (the reference's training dtype)");
    if (a->B <= 0 || a->H <= 0 || a->N <= 0 || a->D <= 0) return set_detail(VB200_ERR_INVALID_ARG, "B, H, N, D must be positive");
    if (a->D > 128) return set_detail(VB200_ERR_UNSUPPORTED, "vb200_attention_bwd: head_dim must be <= 128");
    if (!a->d_out || !a->q || !a->k || !a->v || !a->out || !a->lse || !a->dq || !a->dk || !a->dv)
        return set_detail(VB200_ERR_INVALID_ARG, "vb200_attention_bwd: null tensor");
    if (!a->workspace || a->workspace_bytes < vb200_attention_bwd_workspace_bytes(a))
        return set_detail(VB200_ERR_WORKSPACE, "vb200_attention_bwd: workspace missing or too small");
    DeviceGuard g;
    if (int rc = g.init(a->device)) return rc;
    AttnBwdParams p{};
    p.B = a->B; p.H = a->H; p.N = a->N; p.D = a->D; p.causal = a->causal; p.scale = a->scale;
    p.d_out = static_cast<const float*>(a->d_out); p.q = static_cast<const float*>(a->q); p.k = static_cast<const float*>(a->k);
    p.v = static_cast<const float*>(a->v); p.out = static_cast<const float*>(a->out); p.lse = a->lse;
    p.dq = static_cast<float*>(a->dq); p.dk = static_cast<float*>(a->dk); p.dv = static_cast<float*>(a->dv);
    p.delta = static_cast<float*>(a->workspace);
    return launch_attention_bwd_f32(static_cast<cudaStream_t>(a->stream), p);
}

size_t vb200_exchange_buffer_bytes(int32_t world, int64_t rows, int32_t D) {
    if (world <= 0 || world > VB200_EXCHANGE_MAX_WORLD || rows <= 0 || D <= 0) return 0;
    return exchange_buffer_bytes(world, rows, D);
}

int vb200_exchange_combine(const vb200_exchange_args* a) {
    if (!a || a->struct_size != sizeof(vb200_exchange_args)) return set_detail(VB200_ERR_INVALID_ARG, "vb200_exchange_args: null or struct_size mismatch");
    if (a->world <= 0 || a->world > VB200_EXCHANGE_MAX_WORLD || a->rank < 0 || a->rank >= a->world)
        return set_detail(VB200_ERR_INVALID_ARG, "vb200_exchange_combine: world must be in [1, 16] and rank in [0, world)");
    if (!a->peer_buffers || !a->partial || !a->out || a->rows <= 0 || a->D <= 0 || a->D % 2 != 0)
        return set_detail(VB200_ERR_INVALID_ARG, "vb200_exchange_combine: null pointer, rows <= 0 or odd D");
    if (a->dtype != VB200_BF16 && a->dtype != VB200_F16) return set_detail(VB200_ERR_UNSUPPORTED, "vb200_exchange_combine: out must be bf16 or fp16");
    ExchangeParams p{};
    p.world = a->world; p.rank = a->rank;
    for (int r = 0; r < a->world; ++r) {
        if (!a->peer_buffers[r] || reinterpret_cast<uintptr_t>(a->peer_buffers[r]) % 128 != 0)
            return set_detail(VB200_ERR_ALIGNMENT, "vb200_exchange_combine: every exchange buffer must be non-null and 128-byte aligned");
        p.peers[r] = a->peer_buffers[r];
    }
    if (reinterpret_cast<uintptr_t>(a->partial) % 8 != 0) return set_detail(VB200_ERR_ALIGNMENT, "vb200_exchange_combine: partial must be 8-byte aligned");
    p.partial = a->partial; p.rows = a->rows; p.D = a->D; p.dtype = a->dtype; p.out = a->out; p.lse = a->lse;
    p.step = a->step; p.timeout_cycles = a->timeout_cycles;
    DeviceGuard g;
    if (int rc = g.init(a->device)) return rc;
    p.status = kernel_status_word();
    if (!p.status) return VB200_ERR_CUDA;
    return launch_exchange_combine(static_cast<cudaStream_t>(a->stream), p);
}

// ---- decoder-block operators (vesper_b200_block.h) ---------------------------------------------

static bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

int vb200_linear_bias(int device, void* stream, const void* x, int64_t ldx, const void* w, int64_t ldw,
                      const float* bias, void* out, int64_t ldo, int32_t M, int32_t N, int32_t K,
                      int32_t epilogue, int32_t splits) {
    if (!x || !w || !out || M <= 0 || N <= 0 || K <= 0) return set_detail(VB200_ERR_INVALID_ARG, "vb200_linear: null pointer or non-positive size");
    if (epilogue < VB200_EPI_BF16 || epilogue > VB200_EPI_SWIGLU) return set_detail(VB200_ERR_INVALID_ARG, "vb200_linear: unknown epilogue");
    if (ldx < K || ldw < K) return set_detail(VB200_ERR_INVALID_ARG, "vb200_linear: ldx and ldw must be >= K");
    const int64_t out_cols = epilogue == VB200_EPI_SWIGLU ? N / 2 : N;
    if (ldo < out_cols) return set_detail(VB200_ERR_INVALID_ARG, "vb200_linear: ldo smaller than the output row");
    if (epilogue == VB200_EPI_SWIGLU && N % 2 != 0) return set_detail(VB200_ERR_INVALID_ARG, "vb200_linear: the SwiGLU epilogue needs an even N");
    const int out_elem = (epilogue == VB200_EPI_F32 || epilogue == VB200_EPI_ADD_F32) ? 4 : 2;
    if (K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || (ldo * out_elem) % 16 != 0 || !aligned16(x) || !aligned16(w) || !aligned16(out))
        return set_detail(VB200_ERR_ALIGNMENT, "vb200_linear: K % 8, and 16-byte aligned bases and row strides, are required");
    DeviceGuard g;
    if (int rc = g.init(device)) return rc;
    LinearParams p{};
    p.x = x; p.ldx = ldx; p.w = w; p.ldw = ldw; p.out = out; p.ldo = ldo;
    p.M = M; p.N = N; p.K = K; p.epilogue = epilogue; p.splits = splits;
    p.bias = bias;
    p.status = kernel_status_word();
    if (!p.status) return VB200_ERR_CUDA;
    return launch_linear(static_cast<cudaStream_t>(stream), p);
}

int vb200_linear(int device, void* stream, const void* x, int64_t ldx, const void* w, int64_t ldw,
                 void* out, int64_t ldo, int32_t M, int32_t N, int32_t K, int32_t epilogue, int32_t splits) {
    return vb200_linear_bias(device, stream, x, ldx, w, ldw, nullptr, out, ldo, M, N, K, epilogue, splits);
}

int vb200_linear_f32(int device, void* stream, const float* x, int64_t ldx, const float* w, int64_t ldw, const float* bias,
                     float* out, int64_t ldo, int32_t M, int32_t N, int32_t K) {
    if (!x || !w || !out || M <= 0 || N <= 0 || K <= 0) return set_detail(VB200_ERR_INVALID_ARG, "vb200_linear_f32: null pointer or non-positive size");
    if (ldx < K || ldw < K || ldo < N) return set_detail(VB200_ERR_INVALID_ARG, "vb200_linear_f32: a row stride is smaller than its row");
    DeviceGuard g;
    if (int rc = g.init(device)) return rc;
    return launch_linear_f32(static_cast<cudaStream_t>(stream), x, ldx, w, ldw, bias, out, ldo, M, N, K);
}

int vb200_linear_ex(const vb200_linear_args* a) {
    if (!a || a->struct_size != sizeof(vb200_linear_args)) return set_detail(VB200_ERR_INVALID_ARG, "vb200_linear_args: null or struct_size mismatch");
    if (!a->x || !a->w || !a->out || a->M <= 0 || a->N <= 0 || a->K <= 0) return set_detail(VB200_ERR_INVALID_ARG, "vb200_linear_ex: null pointer or non-positive size");
    if (a->epilogue < VB200_EPI_BF16 || a->epilogue > VB200_EPI_SWIGLU) return set_detail(VB200_ERR_INVALID_ARG, "vb200_linear_ex: unknown epilogue");
    if (a->ldx < a->K || a->ldw < a->K) return set_detail(VB200_ERR_INVALID_ARG, "vb200_linear_ex: ldx and ldw must be >= K");
    const int64_t out_cols = a->epilogue == VB200_EPI_SWIGLU ? a->N / 2 : a->N;
    if (a->ldo < out_cols) return set_detail(VB200_ERR_INVALID_ARG, "vb200_linear_ex: ldo smaller than the output row");
    if (a->epilogue == VB200_EPI_SWIGLU && a->N % 2 != 0) return set_detail(VB200_ERR_INVALID_ARG, "vb200_linear_ex: the SwiGLU epilogue needs an even N");
    const int out_elem = (a->epilogue == VB200_EPI_F32 || a->epilogue == VB200_EPI_ADD_F32) ? 4 : 2;
    if (a->K % 8 != 0 || a->ldx % 8 != 0 || a->ldw % 8 != 0 || (a->ldo * out_elem) % 16 != 0 || !aligned16(a->x) || !aligned16(a->w) || !aligned16(a->out))
        return set_detail(VB200_ERR_ALIGNMENT, "vb200_linear_ex: K % 8, and 16-byte aligned bases and row strides, are required");
    if (a->scaled_copy && (a->epilogue != VB200_EPI_ADD_F32 || !a->copy_scale))
        return set_detail(VB200_ERR_INVALID_ARG, "vb200_linear_ex: scaled_copy needs the += epilogue and copy_scale");
    if (a->rms_rows && (a->rms_dim <= 0 || a->rms_dim % 4 != 0 || a->rms_ld % 4 != 0 || (a->rms_ld != 0 && a->rms_ld < a->rms_dim) || !aligned16(a->rms_rows)))
        return set_detail(VB200_ERR_INVALID_ARG, "vb200_linear_ex: rms_dim must be a positive multiple of 4 and rms_rows 16-byte aligned");
    if (a->rms_rows && a->M > 64 && !a->row_scale)
        return set_detail(VB200_ERR_INVALID_ARG, "vb200_linear_ex: for M > 64 pass row_scale (vb200_row_inv_rms) instead of rms_rows");
    DeviceGuard g;
    if (int rc = g.init(a->device)) return rc;
    LinearParams p{};
    p.x = a->x; p.ldx = a->ldx; p.w = a->w; p.ldw = a->ldw; p.out = a->out; p.ldo = a->ldo;
    p.M = a->M; p.N = a->N; p.K = a->K; p.epilogue = a->epilogue; p.splits = a->splits;
    p.bias = a->bias;
    p.scaled_copy = a->scaled_copy; p.copy_scale = a->copy_scale;
    if (a->row_scale) p.row_scale = a->row_scale;              // a precomputed factor wins over the in-kernel one
    else if (a->rms_rows && a->M <= 64) {
        p.rms_rows = a->rms_rows; p.rms_dim = a->rms_dim; p.rms_eps = a->rms_eps;
        p.rms_ld = a->rms_ld > 0 ? a->rms_ld : a->rms_dim;
    }
    p.status = kernel_status_word();
    if (!p.status) return VB200_ERR_CUDA;
    return launch_linear(static_cast<cudaStream_t>(a->stream), p);
}

int vb200_row_inv_rms(int device, void* stream, const float* h, int64_t ld, float* inv_rms, int32_t M, int32_t dim, float eps) {
    if (!h || !inv_rms || M <= 0 || dim <= 0 || ld < dim) return set_detail(VB200_ERR_INVALID_ARG, "vb200_row_inv_rms: bad arguments");
    if (!aligned16(h)) return set_detail(VB200_ERR_ALIGNMENT, "vb200_row_inv_rms: 16-byte alignment required");
    DeviceGuard g;
    if (int rc = g.init(device)) return rc;
    return launch_row_inv_rms(static_cast<cudaStream_t>(stream), h, ld, inv_rms, M, dim, eps);
}

int vb200_embedding_scaled(int device, void* stream, const void* ids, int32_t ids64, const void* table,
                           float* out, int32_t M, int32_t dim, int32_t vocab, const float* scale, void* scaled_out) {
    if (!ids || !table || !out || !scale || !scaled_out || M <= 0 || dim <= 0 || vocab <= 0)
        return set_detail(VB200_ERR_INVALID_ARG, "vb200_embedding_scaled: bad arguments");
    if (!aligned16(table) || !aligned16(out) || !aligned16(scale) || !aligned16(scaled_out))
        return set_detail(VB200_ERR_ALIGNMENT, "vb200_embedding_scaled: 16-byte alignment required");
    DeviceGuard g;
    if (int rc = g.init(device)) return rc;
    int* status = kernel_status_word();
    if (!status) return VB200_ERR_CUDA;
    return launch_embedding(static_cast<cudaStream_t>(stream), ids, ids64, table, out, M, dim, vocab, status, scale, scaled_out, 0.f, 1);
}

int vb200_linear_add_rmsnorm(int device, void* stream, const void* x, int64_t ldx, const void* w, int64_t ldw,
                             float* h, int32_t M, int32_t N, int32_t K, const float* norm_weight, float eps,
                             void* xn_out, int32_t splits) {
    if (!x || !w || !h || !norm_weight || !xn_out || M <= 0 || N <= 0 || K <= 0)
        return set_detail(VB200_ERR_INVALID_ARG, "vb200_linear_add_rmsnorm: null pointer or non-positive size");
    if (ldx < K || ldw < K) return set_detail(VB200_ERR_INVALID_ARG, "vb200_linear_add_rmsnorm: ldx and ldw must be >= K");
    if (K % 8 != 0 || N % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || !aligned16(x) || !aligned16(w) || !aligned16(h) || !aligned16(norm_weight) || !aligned16(xn_out))
        return set_detail(VB200_ERR_ALIGNMENT, "vb200_linear_add_rmsnorm: K % 8, N % 8 and 16-byte aligned bases and row strides are required");
    DeviceGuard g;
    if (int rc = g.init(device)) return rc;
    LinearParams p{};
    p.x = x; p.ldx = ldx; p.w = w; p.ldw = ldw; p.out = h; p.ldo = N;
    p.M = M; p.N = N; p.K = K; p.epilogue = VB200_EPI_ADD_F32; p.splits = splits;
    p.norm_w = norm_weight; p.norm_out = xn_out; p.norm_ld = N; p.norm_eps = eps;
    p.status = kernel_status_word();
    if (!p.status) return VB200_ERR_CUDA;
    return launch_linear(static_cast<cudaStream_t>(stream), p);
}

int vb200_interleave_rows(int device, void* stream, const void* a, const void* b, void* out, int64_t rows, int64_t cols) {
    if (!a || !b || !out || rows <= 0 || cols <= 0) return set_detail(VB200_ERR_INVALID_ARG, "vb200_interleave_rows: bad arguments");
    if (!aligned16(a) || !aligned16(b) || !aligned16(out)) return set_detail(VB200_ERR_ALIGNMENT, "vb200_interleave_rows: 16-byte alignment required");
    DeviceGuard g;
    if (int rc = g.init(device)) return rc;
    return launch_interleave_rows(static_cast<cudaStream_t>(stream), a, b, out, rows, cols);
}

int vb200_rms_norm(int device, void* stream, const float* x, const float* weight, void* out_bf16,
                   int32_t M, int32_t dim, float eps) {
    if (!x || !weight || !out_bf16 || M <= 0 || dim <= 0) return set_detail(VB200_ERR_INVALID_ARG, "vb200_rms_norm: bad arguments");
    if (!aligned16(x) || !aligned16(weight) || !aligned16(out_bf16)) return set_detail(VB200_ERR_ALIGNMENT, "vb200_rms_norm: 16-byte alignment required");
    DeviceGuard g;
    if (int rc = g.init(device)) return rc;
    return launch_rms_norm(static_cast<cudaStream_t>(stream), x, weight, out_bf16, M, dim, eps);
}

int vb200_silu_mul(int device, void* stream, const void* gate, const void* up, void* out, int64_t n) {
    if (!gate || !up || !out || n <= 0) return set_detail(VB200_ERR_INVALID_ARG, "vb200_silu_mul: bad arguments");
    if (!aligned16(gate) || !aligned16(up) || !aligned16(out)) return set_detail(VB200_ERR_ALIGNMENT, "vb200_silu_mul: 16-byte alignment required");
    DeviceGuard g;
    if (int rc = g.init(device)) return rc;
    return launch_silu_mul(static_cast<cudaStream_t>(stream), gate, up, out, n);
}

int vb200_embedding(int device, void* stream, const void* ids, int32_t ids64, const void* table,
                    float* out, int32_t M, int32_t dim, int32_t vocab) {
    if (!ids || !table || !out || M <= 0 || dim <= 0 || vocab <= 0) return set_detail(VB200_ERR_INVALID_ARG, "vb200_embedding: bad arguments");
    if (!aligned16(table) || !aligned16(out)) return set_detail(VB200_ERR_ALIGNMENT, "vb200_embedding: 16-byte alignment required");
    DeviceGuard g;
    if (int rc = g.init(device)) return rc;
    int* status = kernel_status_word();
    if (!status) return VB200_ERR_CUDA;
    return launch_embedding(static_cast<cudaStream_t>(stream), ids, ids64, table, out, M, dim, vocab, status);
}

int vb200_embedding_rmsnorm(int device, void* stream, const void* ids, int32_t ids64, const void* table,
                            float* out, int32_t M, int32_t dim, int32_t vocab, const float* norm_weight,
                            float eps, void* xn_out) {
    if (!ids || !table || !out || !norm_weight || !xn_out || M <= 0 || dim <= 0 || vocab <= 0)
        return set_detail(VB200_ERR_INVALID_ARG, "vb200_embedding_rmsnorm: bad arguments");
    if (!aligned16(table) || !aligned16(out) || !aligned16(norm_weight) || !aligned16(xn_out))
        return set_detail(VB200_ERR_ALIGNMENT, "vb200_embedding_rmsnorm: 16-byte alignment required");
    DeviceGuard g;
    if (int rc = g.init(device)) return rc;
    int* status = kernel_status_word();
    if (!status) return VB200_ERR_CUDA;
    return launch_embedding(static_cast<cudaStream_t>(stream), ids, ids64, table, out, M, dim, vocab, status, norm_weight, xn_out, eps);
}

int vb200_greedy_step(const vb200_greedy_args* a) {
    if (!a || a->struct_size != sizeof(vb200_greedy_args)) return set_detail(VB200_ERR_INVALID_ARG, "vb200_greedy_args: null or struct_size mismatch");
    if (!a->logits || !a->out_ids || a->B <= 0 || a->vocab <= 0 || a->ld_logits < a->vocab)
        return set_detail(VB200_ERR_INVALID_ARG, "vb200_greedy_step: bad arguments");
    if (a->n_stop > 0 && !a->stop_ids) return set_detail(VB200_ERR_INVALID_ARG, "vb200_greedy_step: n_stop > 0 without stop_ids");
    DeviceGuard g;
    if (int rc = g.init(a->device)) return rc;
    return launch_greedy_step(static_cast<cudaStream_t>(a->stream), *a);
}

}  // extern "C"
