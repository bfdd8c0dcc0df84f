// Sequence-sharded decode: exchange of the per-rank partial results (O/l, m, l) and their
// log-sum-exp merge in ONE kernel over NVLink peer memory -- each rank stores its partial rows
// straight into every peer's receive slots (plain 8-byte peer stores {value, call number}, no TMA, no multicast),
// waits (bounded) until every rank's words of this call have landed in its own buffer and merges.
// It stands in for "all-gather, then vb200_lse_combine": one launch, no collective library call, no
// host wait between the two.  The merge algebra is the online-softmax recurrence of
// src/ops/flash_attention.cpp:309-345 applied across shards.
//
// The buffer layout and the protocol itself live in decode_exchange.cuh (the split-KV decode kernel runs the same
// protocol as its tail, see decode_gqa_mma.cu).
#include "decode_exchange.cuh"

namespace vb200 {
namespace {

constexpr int kRowsPerCta = 4;
constexpr int kThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kThreads)
exchange_combine_kernel(ExchangeParams p) {
    const int c = blockIdx.x;
    // Launched with programmatic stream serialization: the blocks may become resident while the kernel that writes the
    // partial records drains; nothing of its output is touched before this wait returns.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const long long r0 = static_cast<long long>(c) * p.rows_per_cta;
    const long long r1 = min(p.rows, r0 + p.rows_per_cta);
    __shared__ uint32_t s_step;
    __shared__ int s_ok;
    extern __shared__ __align__(16) unsigned char stage_raw[];       // all ranks' words of this CTA's rows, when they fit
    exchange_rows<T, kThreads>(p, c, r0, r1, p.partial + r0 * (p.D + 2), threadIdx.x, &s_step, &s_ok, [] { __syncthreads(); },
                               p.stage_floats > 0 ? reinterpret_cast<float*>(stage_raw) : nullptr, p.stage_floats);
}

}  // namespace

size_t exchange_buffer_bytes(int world, long long rows, int D) {
    return kXSlotBase + static_cast<size_t>(2) * world * rows * (D + 2) * 8;      // 8-byte words {value, call number}
}

int launch_exchange_combine(cudaStream_t s, ExchangeParams p) {
    long long ctas = (p.rows + kRowsPerCta - 1) / kRowsPerCta;
    p.rows_per_cta = kRowsPerCta;
    if (ctas > kXMaxCtas) {
        ctas = kXMaxCtas;
        p.rows_per_cta = (p.rows + kXMaxCtas - 1) / kXMaxCtas;
        ctas = (p.rows + p.rows_per_cta - 1) / p.rows_per_cta;
    }
    if (p.timeout_cycles <= 0) p.timeout_cycles = kWaitCycles;
    // room to stage every rank's words of a CTA's rows (8 bytes per value) in shared memory, when that fits
    size_t stage = static_cast<size_t>(p.world) * p.rows_per_cta * (p.D + 2) * 8;
    if (stage > 96 * 1024) stage = 0;
    p.stage_floats = static_cast<int>(stage / 4);
    if (stage > 48 * 1024) {
        static thread_local bool configured[64][2] = {};
        int dev = 0;
        VB200_CUDA_TRY(cudaGetDevice(&dev));
        if (dev < 0 || dev >= 64) return set_detail(VB200_ERR_NO_DEVICE, "device ordinal out of range");
        const int which = p.dtype == VB200_BF16 ? 0 : 1;
        if (!configured[dev][which]) {
            if (which == 0) VB200_CUDA_TRY(cudaFuncSetAttribute(exchange_combine_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
            else VB200_CUDA_TRY(cudaFuncSetAttribute(exchange_combine_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
            configured[dev][which] = true;
        }
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(ctas));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = stage;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    switch (p.dtype) {
        case VB200_BF16: VB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, exchange_combine_kernel<__nv_bfloat16>, p)); break;
        case VB200_F16: VB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, exchange_combine_kernel<__half>, p)); break;
        default: return set_detail(VB200_ERR_UNSUPPORTED, "exchange_combine: dtype must be bf16 or fp16");
    }
    note_launch();
    VB200_CUDA_TRY(cudaPeekAtLastError());
    return VB200_OK;
}

}  // namespace vb200
