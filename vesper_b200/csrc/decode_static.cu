// vb200_decode_fwd_static: the split-KV decode step for callers that have no
// device memory to hand over as a workspace and may not allocate any.
//
// Typical callers: a serving loop whose process has already given every free
// byte of HBM to its KV-cache pool (a cudaMalloc there fails or forces the pool
// to shrink), and plugin code that runs inside a host framework which owns all
// device allocation and offers no allocator to the plugin.  For them the
// per-split partial results live in a fixed array that is part of the library
// image on every GPU that loads it, instead of in caller memory.
//
// Consequences the caller must know:
//   * The array is VB200_STATIC_SCRATCH_BYTES long; a step whose split plan
//     needs more is rejected with VB200_ERR_WORKSPACE (pass a smaller
//     num_splits, or use vb200_decode_fwd with your own workspace).
//   * All calls on one GPU share the one array and it keeps whatever the
//     previous call left.  Nothing in it has to start at zero: every slot a
//     step reads (the per-sequence length header and the partials of the valid
//     splits) is written earlier in the same step.  Two calls that can run at
//     the same time on one GPU (different streams, different threads) race on
//     it -- order them on one stream.
//   * The first call on each device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current).  That first call
//     should be made before any stream capture begins.
//   * The address is remembered per device ordinal for the life of the process.
//     A host program that calls cudaDeviceReset() destroys the context the
//     address belongs to; do not call this entry point again on that device
//     afterwards (reload the library instead).
//   * The call allocates and frees nothing: no cudaMalloc / cudaFree, no
//     allocating library routine.
#include <cstdio>
#include <mutex>

#include "kernels.h"

namespace vb200 {
namespace {

// Scratch for the split partials: [B,Hkv,splits,n_rep,D+2] fp32 plus the
// length header.  Held by every GPU that loads the library until exit.
static __device__ __align__(256) unsigned char g_decode_scratch[VB200_STATIC_SCRATCH_BYTES];

std::mutex g_scratch_mutex;
void* g_scratch_addr[64] = {nullptr};

// Device address of the array on the CURRENT device.  In host code the name
// g_decode_scratch is only a handle for the runtime, not a device pointer, so
// the address is asked for once per device and cached.
int scratch_address(void** out) {
    int dev = -1;
    VB200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return set_detail(VB200_ERR_NO_DEVICE, "device ordinal out of range");
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_addr[dev]) {
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_decode_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_decode_scratch)");
        if (!ptr) return set_detail(VB200_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
        g_scratch_addr[dev] = ptr;
    }
    *out = g_scratch_addr[dev];
    return VB200_OK;
}

}  // namespace
}  // namespace vb200

using namespace vb200;

extern "C" int vb200_decode_fwd_static(const vb200_decode_args* a) {
    if (!a || a->struct_size != sizeof(vb200_decode_args))
        return set_detail(VB200_ERR_INVALID_ARG, "vb200_decode_args: null or struct_size mismatch");
    const size_t need = vb200_decode_workspace_bytes(a);
    // 0 = a shape no plan exists for (non-positive B, Hq, Hkv or D, Hq not a multiple of Hkv): an argument
    // error, reported as such before the size comparison below can misread it
    if (need == 0) return set_detail(VB200_ERR_INVALID_ARG, "vb200_decode_fwd_static: bad shape (B, Hq, Hkv, D)");
    if (need > static_cast<size_t>(VB200_STATIC_SCRATCH_BYTES)) {
        static thread_local char msg[200];
        snprintf(msg, sizeof(msg),
                 "vb200_decode_fwd_static: this step needs %zu bytes of scratch but the built-in array holds %d; "
                 "lower num_splits or call vb200_decode_fwd with a workspace",
                 need, VB200_STATIC_SCRATCH_BYTES);
        return set_detail(VB200_ERR_WORKSPACE, msg);
    }
    DeviceGuard g;                       // the symbol lookup below needs the target device current
    if (int rc = g.init(a->device)) return rc;
    void* scratch = nullptr;
    if (int rc = scratch_address(&scratch)) return rc;
    vb200_decode_args b = *a;            // same step, scratch swapped in; the caller's struct is untouched
    b.workspace = scratch;
    b.workspace_bytes = VB200_STATIC_SCRATCH_BYTES;
    return vb200_decode_fwd(&b);
}
