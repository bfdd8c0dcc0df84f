// Literal drop-in: the C++ symbols that Vesper's host library leaves undefined when it is compiled with
// -DUSE_CUDA_BACKEND=1 (its src/ops/cuda/*.cu are then NOT compiled), defined on top of libvesper_b200's C ABI.
// Linked with the reference's own, unmodified host objects, this file IS the CUDA backend: ops::flash_attention,
// KVCache::update, repeat_kv, RoPE and scaled_dot_product_attention on Device::CUDA tensors then run on the B200
// kernels.  It is compiled against the reference's headers (vesper::Tensor, include/vesper/core/tensor.h:26-223),
// so it builds only where the reference tree is present; nothing of the reference is copied here.
//
// Three groups of symbols:
//   1. the attention hot path -- adapters of a few lines onto the C ABI:
//        flash_attention_cuda_dispatch            declared src/ops/flash_attention.cpp:28-32, called :102-110
//        flash_attention_backward_cuda_dispatch   declared src/ops/flash_attention.cpp:34-40
//        repeat_kv_cuda_dispatch                  declared src/ops/attention_ops.cpp:24-27
//        apply_rope_cuda                          declared src/nn/rope.cpp:25-28
//   2. what the attention modules and their tests need around it, as small plain kernels written here (fp32, any
//      strides): copy_strided (Tensor::contiguous / copy_from, src/core/tensor.cpp:197-228, 380-405), the pieces of
//      the standard attention path of src/nn/functional.cpp:399-421 (gemm / gemm_batch, div/mul/add scalar,
//      broadcast add/sub/mul/div, softmax), and normal / uniform for vesper::randn on the device (drawn on the host
//      with std::mt19937 and uploaded: test support, not a device generator);
//   3. every other *_cuda_dispatch symbol the host library references: throws "not provided by this backend".
// Errors follow the reference's convention: std::runtime_error with the C ABI's message.
#include <vesper/core/factories.h>
#include <vesper/core/stream.h>
#include <vesper/core/tensor.h>

#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <random>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/vesper_b200.h"

namespace vesper {

namespace {

constexpr int kMaxRank = 8;

[[noreturn]] void not_provided(const char* what) {
    throw std::runtime_error(std::string(what) + ": not provided by this backend (vesper_b200 covers the attention path)");
}

void check(int rc, const char* who) {
    if (rc != VB200_OK)
        throw std::runtime_error(std::string(who) + ": " + vb200_strerror(rc) + ": " + vb200_last_error_detail());
}

void check_launch(const char* who) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) throw std::runtime_error(std::string(who) + ": CUDA launch failed: " + cudaGetErrorString(e));
}

cudaStream_t stream() { return static_cast<cudaStream_t>(Stream::current(Device::CUDA).raw_handle()); }

void require_f32(const Tensor& t, const char* who) {
    if (t.dtype() != DType::Float32) throw std::runtime_error(std::string(who) + ": Float32 only");
}

// [B,H,S,D] view with D contiguous and 16-byte aligned base / strides: what the C ABI takes without a copy
bool abi_ready(const Tensor& t) {
    if (t.ndim() != 4 || t.strides()[3] != 1) return false;
    if (reinterpret_cast<uintptr_t>(t.data_ptr<char>()) % 16 != 0) return false;
    for (int i = 0; i < 3; ++i)
        if ((t.strides()[i] * 4) % 16 != 0) return false;
    return true;
}

vb200_tensor4 view4(const Tensor& t) {
    return {const_cast<char*>(t.data_ptr<char>()), t.strides()[0], t.strides()[1], t.strides()[2]};
}

// The reference's CUDA kernel read q/k/v as if contiguous without checking (src/ops/cuda/flash_attention.cu:540-541);
// here views are honoured: passed by strides when the C ABI can take them, copied otherwise.
Tensor for_abi(const Tensor& t) { return abi_ready(t) ? t : t.contiguous(); }

// An index space of up to kMaxRank dimensions with one stride set per operand.
struct Walk {
    int rank;
    long long shape[kMaxRank];
    long long sa[kMaxRank], sb[kMaxRank], so[kMaxRank];
};

void fill_walk(Walk& w, const std::vector<int64_t>& shape, const std::vector<int64_t>* sa, const std::vector<int64_t>* sb,
               const std::vector<int64_t>& so, const char* who) {
    if (shape.size() > static_cast<size_t>(kMaxRank)) throw std::runtime_error(std::string(who) + ": rank above 8");
    w.rank = static_cast<int>(shape.size());
    for (int d = 0; d < w.rank; ++d) {
        w.shape[d] = shape[d];
        w.sa[d] = sa ? (*sa)[d] : 0;
        w.sb[d] = sb ? (*sb)[d] : 0;
        w.so[d] = so[d];
    }
}

__device__ __forceinline__ void offsets(const Walk& w, long long i, long long& a, long long& b, long long& o) {
    a = b = o = 0;
    for (int d = w.rank - 1; d >= 0; --d) {
        const long long c = i % w.shape[d];
        i /= w.shape[d];
        a += c * w.sa[d]; b += c * w.sb[d]; o += c * w.so[d];
    }
}

enum BinOp { kAdd, kSub, kMul, kDiv };

template <int OP>
__global__ void binary_kernel(const float* a, const float* b, float* out, Walk w, long long n) {
    const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (i >= n) return;
    long long ia, ib, io;
    offsets(w, i, ia, ib, io);
    const float x = a[ia], y = b[ib];
    out[io] = OP == kAdd ? x + y : OP == kSub ? x - y : OP == kMul ? x * y : x / y;
}

template <int OP>
__global__ void scalar_kernel(const float* a, float s, float* out, Walk w, long long n) {
    const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (i >= n) return;
    long long ia, ib, io;
    offsets(w, i, ia, ib, io);
    const float x = a[ia];
    out[io] = OP == kAdd ? x + s : OP == kSub ? x - s : OP == kMul ? x * s : x / s;
}

__global__ void copy_kernel(const float* src, float* dst, Walk w, long long n) {
    const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (i >= n) return;
    long long ia, ib, io;
    offsets(w, i, ia, ib, io);
    dst[io] = src[ia];
}

long long count(const std::vector<int64_t>& shape) {
    long long n = 1;
    for (auto d : shape) n *= d;
    return n;
}

template <int OP>
void binary(const Tensor& a, const std::vector<int64_t>& sa, const Tensor& b, const std::vector<int64_t>& sb, Tensor& out, const char* who) {
    require_f32(a, who); require_f32(b, who);
    Walk w;
    fill_walk(w, out.shape(), &sa, &sb, out.strides(), who);
    const long long n = count(out.shape());
    if (n == 0) return;
    binary_kernel<OP><<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream()>>>(a.data_ptr<float>(), b.data_ptr<float>(), out.data_ptr<float>(), w, n);
    check_launch(who);
}

template <int OP>
void scalar(const Tensor& a, float s, Tensor& out, const char* who) {
    require_f32(a, who);
    Walk w;
    fill_walk(w, out.shape(), &a.strides(), nullptr, out.strides(), who);
    const long long n = count(out.shape());
    if (n == 0) return;
    scalar_kernel<OP><<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream()>>>(a.data_ptr<float>(), s, out.data_ptr<float>(), w, n);
    check_launch(who);
}

// One block per row of the softmax dimension: max, sum of exp, normalise.  `outer` walks every other dimension.
__global__ void softmax_kernel(const float* in, float* out, Walk outer, long long len, long long in_stride, long long out_stride) {
    long long ia, ib, io;
    offsets(outer, blockIdx.x, ia, ib, io);
    const float* x = in + ia;
    float* y = out + io;
    __shared__ float red[32];
    float m = -INFINITY;
    for (long long j = threadIdx.x; j < len; j += blockDim.x) m = fmaxf(m, x[j * in_stride]);
    for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    m = red[0];
    for (int i = 1; i < (blockDim.x >> 5); ++i) m = fmaxf(m, red[i]);
    __syncthreads();
    float s = 0.f;
    for (long long j = threadIdx.x; j < len; j += blockDim.x) s += expf(x[j * in_stride] - m);
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    s = 0.f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) s += red[i];
    for (long long j = threadIdx.x; j < len; j += blockDim.x) y[j * out_stride] = expf(x[j * in_stride] - m) / s;
}

// C[m,n] = sum_k A(m,k) B(k,n) for `batch` matrices; every operand addressed by (batch, row, column) strides, so
// transposed views and the transA / transB flags cost nothing.  16 x 16 tiles through shared memory.
struct GemmArgs {
    const float *a, *b;
    float* c;
    long long M, N, K;
    long long a_batch, a_m, a_k, b_batch, b_k, b_n, c_batch, c_m, c_n;
};

__global__ void gemm_kernel(GemmArgs g) {
    __shared__ float ta[16][17], tb[16][17];
    const long long z = blockIdx.z;
    const float* a = g.a + z * g.a_batch;
    const float* b = g.b + z * g.b_batch;
    float* c = g.c + z * g.c_batch;
    const long long m = blockIdx.y * 16LL + threadIdx.y, n = blockIdx.x * 16LL + threadIdx.x;
    float acc = 0.f;
    for (long long k0 = 0; k0 < g.K; k0 += 16) {
        const long long ka = k0 + threadIdx.x, kb = k0 + threadIdx.y;
        ta[threadIdx.y][threadIdx.x] = (m < g.M && ka < g.K) ? a[m * g.a_m + ka * g.a_k] : 0.f;
        tb[threadIdx.y][threadIdx.x] = (kb < g.K && n < g.N) ? b[kb * g.b_k + n * g.b_n] : 0.f;
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k) acc = fmaf(ta[threadIdx.y][k], tb[k][threadIdx.x], acc);
        __syncthreads();
    }
    if (m < g.M && n < g.N) c[m * g.c_m + n * g.c_n] = acc;
}

void run_gemm(const Tensor& a, const Tensor& b, Tensor& c, long long batch, long long sa, long long sb, long long sc,
              bool transA, bool transB, const char* who) {
    require_f32(a, who); require_f32(b, who);
    const int ra = static_cast<int>(a.ndim()), rb = static_cast<int>(b.ndim()), rc = static_cast<int>(c.ndim());
    GemmArgs g{};
    g.a = a.data_ptr<float>(); g.b = b.data_ptr<float>(); g.c = c.data_ptr<float>();
    g.M = c.shape()[rc - 2]; g.N = c.shape()[rc - 1];
    g.K = transA ? a.shape()[ra - 2] : a.shape()[ra - 1];
    // A(m,k): element [m,k] of the stored matrix, or [k,m] when transA
    g.a_m = transA ? a.strides()[ra - 1] : a.strides()[ra - 2];
    g.a_k = transA ? a.strides()[ra - 2] : a.strides()[ra - 1];
    g.b_k = transB ? b.strides()[rb - 1] : b.strides()[rb - 2];
    g.b_n = transB ? b.strides()[rb - 2] : b.strides()[rb - 1];
    g.c_m = c.strides()[rc - 2]; g.c_n = c.strides()[rc - 1];
    g.a_batch = sa; g.b_batch = sb; g.c_batch = sc;
    if (g.M == 0 || g.N == 0 || batch == 0) return;
    if (batch > 65535) throw std::runtime_error(std::string(who) + ": more than 65535 matrices in a batch");
    dim3 grid(static_cast<unsigned>((g.N + 15) / 16), static_cast<unsigned>((g.M + 15) / 16), static_cast<unsigned>(batch));
    gemm_kernel<<<grid, dim3(16, 16), 0, stream()>>>(g);
    check_launch(who);
}

// vesper::randn / rand on a device tensor: the values come from the host generator and are uploaded.
template <typename Dist>
void fill_from_host(Tensor& t, Dist dist, const char* who) {
    require_f32(t, who);
    if (!t.is_contiguous()) throw std::runtime_error(std::string(who) + ": tensor must be contiguous");
    static std::mt19937 gen(0x5eed);
    std::vector<float> h(t.numel());
    for (auto& x : h) x = dist(gen);
    cudaError_t e = cudaMemcpyAsync(t.data_ptr<float>(), h.data(), h.size() * sizeof(float), cudaMemcpyHostToDevice, stream());
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream());        // `h` goes out of scope
    if (e != cudaSuccess) throw std::runtime_error(std::string(who) + ": " + cudaGetErrorString(e));
}

}  // namespace

namespace ops {

// ---- 1. the attention hot path ---------------------------------------------------------------------------------

// dropout_p / training / dropout_mask_out are accepted and ignored, as the reference's CUDA kernel does
// (src/ops/cuda/flash_attention.cu:518-544; tests/test_flash_attention.cpp:547-576 checks finiteness only).
void flash_attention_cuda_dispatch(const Tensor& q, const Tensor& k, const Tensor& v, Tensor& output, Tensor& lse,
                                   float scale, bool is_causal, float /*dropout_p*/, bool /*training*/, Tensor* /*dropout_mask_out*/) {
    require_f32(q, "flash_attention");
    const Tensor qa = for_abi(q), ka = for_abi(k), va = for_abi(v);
    if (!abi_ready(output) || (lse.defined() && !lse.is_contiguous()))
        throw std::runtime_error("flash_attention: the output tensors the front-end allocates must be contiguous");
    vb200_prefill_args a{};
    a.struct_size = sizeof(a);
    a.device = -1;                                   // the reference has one current device
    a.stream = stream();
    a.dtype = VB200_F32;
    a.B = static_cast<int>(q.shape()[0]); a.Hq = static_cast<int>(q.shape()[1]); a.Hkv = static_cast<int>(k.shape()[1]);
    a.T = static_cast<int>(q.shape()[2]); a.D = static_cast<int>(q.shape()[3]);
    a.causal = is_causal ? 1 : 0;
    a.scale = scale;
    a.q = view4(qa); a.k = view4(ka); a.v = view4(va); a.o = view4(output);
    a.lse = lse.defined() ? lse.data_ptr<float>() : nullptr;
    check(vb200_prefill_fwd(&a), "flash_attention");
}

void flash_attention_backward_cuda_dispatch(const Tensor& grad_output, const Tensor& q, const Tensor& k, const Tensor& v,
                                            const Tensor& output, const Tensor& lse, Tensor& grad_q, Tensor& grad_k, Tensor& grad_v,
                                            float scale, bool is_causal, float dropout_p, const Tensor* /*dropout_mask*/) {
    require_f32(q, "flash_attention_backward");
    if (dropout_p > 0.0f) throw std::runtime_error("flash_attention_backward: dropout is not part of the CUDA path");
    const Tensor dO = grad_output.contiguous(), qc = q.contiguous(), kc = k.contiguous(), vc = v.contiguous(), oc = output.contiguous(),
                 lc = lse.contiguous();
    if (!grad_q.is_contiguous() || !grad_k.is_contiguous() || !grad_v.is_contiguous())
        throw std::runtime_error("flash_attention_backward: gradient tensors must be contiguous");
    vb200_attention_bwd_args a{};
    a.struct_size = sizeof(a);
    a.device = -1;
    a.stream = stream();
    a.dtype = VB200_F32;
    a.B = static_cast<int>(q.shape()[0]); a.H = static_cast<int>(q.shape()[1]); a.N = static_cast<int>(q.shape()[2]); a.D = static_cast<int>(q.shape()[3]);
    a.causal = is_causal ? 1 : 0;
    a.scale = scale;
    a.d_out = dO.data_ptr<char>(); a.q = qc.data_ptr<char>(); a.k = kc.data_ptr<char>(); a.v = vc.data_ptr<char>(); a.out = oc.data_ptr<char>();
    a.lse = lc.data_ptr<float>();
    a.dq = grad_q.data_ptr<char>(); a.dk = grad_k.data_ptr<char>(); a.dv = grad_v.data_ptr<char>();
    const size_t need = vb200_attention_bwd_workspace_bytes(&a);
    Tensor ws = vesper::empty({static_cast<int64_t>((need + 3) / 4)}, DType::Float32, Device::CUDA);   // from the caller's caching allocator
    a.workspace = ws.data_ptr<char>();
    a.workspace_bytes = ws.numel() * 4;
    check(vb200_attention_bwd(&a), "flash_attention_backward");
}

// Honours the strides of a cache view (the reference's dispatcher indexes it as if contiguous, src/ops/cuda/attention_ops.cu:69-96).
void repeat_kv_cuda_dispatch(const Tensor& input, Tensor& output, int64_t n_rep) {
    require_f32(input, "repeat_kv");
    const Tensor in = for_abi(input);
    if (!output.is_contiguous()) throw std::runtime_error("repeat_kv: output must be contiguous");
    vb200_tensor4 iv = view4(in);
    check(vb200_repeat_kv(-1, stream(), VB200_F32, &iv, output.data_ptr<char>(), static_cast<int>(in.shape()[0]), static_cast<int>(in.shape()[1]),
                          static_cast<int>(in.shape()[2]), static_cast<int>(in.shape()[3]), static_cast<int>(n_rep)),
          "repeat_kv");
}

void repeat_kv_backward_cuda_dispatch(const Tensor&, Tensor&, int64_t) { not_provided("repeat_kv_backward"); }

// ---- 2. around the path: plain fp32 kernels -------------------------------------------------------------------

void copy_strided_cuda_dispatch(const Tensor& src, Tensor& dst) {
    require_f32(src, "copy_strided");
    const long long n = count(dst.shape());
    if (n == 0) return;
    Walk w;
    if (src.shape() == dst.shape()) {
        fill_walk(w, dst.shape(), &src.strides(), nullptr, dst.strides(), "copy_strided");
        copy_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream()>>>(src.data_ptr<float>(), dst.data_ptr<float>(), w, n);
        check_launch("copy_strided");
        return;
    }
    // same element count, different shapes (copy_from of a reshaped tensor): element i of one in row-major order
    // goes to element i of the other; at least one side is then walked as a flat array
    if (!src.is_contiguous() && !dst.is_contiguous()) throw std::runtime_error("copy_strided: shapes differ and both tensors are views");
    if (src.is_contiguous()) {
        const std::vector<int64_t> flat(dst.shape().size(), 0);
        std::vector<int64_t> lin(dst.shape().size());
        long long s = 1;
        for (int d = static_cast<int>(dst.shape().size()) - 1; d >= 0; --d) { lin[d] = s; s *= dst.shape()[d]; }
        fill_walk(w, dst.shape(), &lin, nullptr, dst.strides(), "copy_strided");
    } else {
        std::vector<int64_t> lin(src.shape().size());
        long long s = 1;
        for (int d = static_cast<int>(src.shape().size()) - 1; d >= 0; --d) { lin[d] = s; s *= src.shape()[d]; }
        fill_walk(w, src.shape(), &src.strides(), nullptr, lin, "copy_strided");
    }
    copy_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream()>>>(src.data_ptr<float>(), dst.data_ptr<float>(), w, n);
    check_launch("copy_strided");
}

void add_cuda_dispatch(const Tensor& a, const std::vector<int64_t>& sa, const Tensor& b, const std::vector<int64_t>& sb, Tensor& out) { binary<kAdd>(a, sa, b, sb, out, "add"); }
void sub_cuda_dispatch(const Tensor& a, const std::vector<int64_t>& sa, const Tensor& b, const std::vector<int64_t>& sb, Tensor& out) { binary<kSub>(a, sa, b, sb, out, "sub"); }
void mul_cuda_dispatch(const Tensor& a, const std::vector<int64_t>& sa, const Tensor& b, const std::vector<int64_t>& sb, Tensor& out) { binary<kMul>(a, sa, b, sb, out, "mul"); }
void div_cuda_dispatch(const Tensor& a, const std::vector<int64_t>& sa, const Tensor& b, const std::vector<int64_t>& sb, Tensor& out) { binary<kDiv>(a, sa, b, sb, out, "div"); }
void add_scalar_cuda_dispatch(const Tensor& a, float b, Tensor& out) { scalar<kAdd>(a, b, out, "add"); }
void sub_scalar_cuda_dispatch(const Tensor& a, float b, Tensor& out) { scalar<kSub>(a, b, out, "sub"); }
void mul_scalar_cuda_dispatch(const Tensor& a, float b, Tensor& out) { scalar<kMul>(a, b, out, "mul"); }
void div_scalar_cuda_dispatch(const Tensor& a, float b, Tensor& out) { scalar<kDiv>(a, b, out, "div"); }

void softmax_cuda_dispatch(const Tensor& input, int64_t dim, Tensor& output) {
    require_f32(input, "softmax");
    const int rank = static_cast<int>(input.ndim());
    if (dim < 0) dim += rank;
    if (dim < 0 || dim >= rank) throw std::runtime_error("softmax: dim out of range");
    std::vector<int64_t> shape, si, so;
    for (int d = 0; d < rank; ++d)
        if (d != dim) { shape.push_back(input.shape()[d]); si.push_back(input.strides()[d]); so.push_back(output.strides()[d]); }
    Walk w;
    fill_walk(w, shape, &si, nullptr, so, "softmax");
    const long long rows = count(shape), len = input.shape()[dim];
    if (rows == 0 || len == 0) return;
    const int threads = len >= 1024 ? 256 : (len >= 128 ? 128 : 32);
    softmax_kernel<<<static_cast<unsigned>(rows), threads, 0, stream()>>>(input.data_ptr<float>(), output.data_ptr<float>(), w, len,
                                                                         input.strides()[dim], output.strides()[dim]);
    check_launch("softmax");
}

void gemm_cuda_dispatch(const Tensor& a, const Tensor& b, Tensor& c, bool transA, bool transB) {
    run_gemm(a, b, c, 1, 0, 0, 0, transA, transB, "gemm");
}

void gemm_batch_cuda_dispatch(const Tensor& a, const Tensor& b, Tensor& c, int64_t batch_count, int64_t stride_a, int64_t stride_b,
                              int64_t stride_c, bool transA, bool transB) {
    run_gemm(a, b, c, batch_count, stride_a, stride_b, stride_c, transA, transB, "gemm_batch");
}

void normal_cuda_dispatch(Tensor& t, float mean, float std) { fill_from_host(t, std::normal_distribution<float>(mean, std), "normal_"); }
void uniform_cuda_dispatch(Tensor& t, float lo, float hi) { fill_from_host(t, std::uniform_real_distribution<float>(lo, hi), "uniform_"); }

// ---- 3. outside the attention path ----------------------------------------------------------------------------

void adam_update_cuda_dispatch(Tensor&, const Tensor&, const Tensor&, float, float, float, float) { not_provided("adam_update"); }
void addcmul_cuda_dispatch(Tensor&, const Tensor&, const Tensor&, float) { not_provided("addcmul"); }
bool all_true_cuda_dispatch(const Tensor&) { not_provided("all_true"); }
void argmax_cuda_dispatch(const Tensor&, Tensor&) { not_provided("argmax"); }
void cast_cuda_dispatch(const Tensor&, Tensor&) { not_provided("cast"); }
void check_stop_tokens_cuda_dispatch(const Tensor&, Tensor&, const int64_t*, int64_t, int64_t, int64_t) { not_provided("check_stop_tokens"); }
void col2im_cuda_dispatch(const Tensor&, Tensor&, int, int, int, int, int, int) { not_provided("col2im"); }
void cos_cuda_dispatch(const Tensor&, const std::vector<int64_t>&, Tensor&) { not_provided("cos"); }
void embedding_backward_cuda_dispatch(const Tensor&, const Tensor&, int64_t, int64_t, bool, Tensor&) { not_provided("embedding_backward"); }
void embedding_cuda_dispatch(const Tensor&, const Tensor&, int64_t, float, float, Tensor&) { not_provided("embedding"); }
void equal_cuda_dispatch(const Tensor&, const Tensor&, Tensor&) { not_provided("equal"); }
void equal_scalar_cuda_dispatch(const Tensor&, float, Tensor&) { not_provided("equal"); }
void exp_cuda_dispatch(const Tensor&, const std::vector<int64_t>&, Tensor&) { not_provided("exp"); }
void gather_cuda_dispatch(const Tensor&, int64_t, const Tensor&, Tensor&) { not_provided("gather"); }
void gelu_backward_cuda_dispatch(const Tensor&, const Tensor&, Tensor&) { not_provided("gelu_backward"); }
void gelu_cuda_dispatch(const Tensor&, const std::vector<int64_t>&, Tensor&) { not_provided("gelu"); }
void gelu_erf_backward_cuda_dispatch(const Tensor&, const Tensor&, Tensor&) { not_provided("gelu_erf_backward"); }
void gelu_erf_cuda_dispatch(const Tensor&, const std::vector<int64_t>&, Tensor&) { not_provided("gelu_erf"); }
void greater_than_cuda_dispatch(const Tensor&, float, Tensor&) { not_provided("greater_than"); }
void im2col_cuda_dispatch(const Tensor&, Tensor&, int, int, int, int, int, int) { not_provided("im2col"); }
void layer_norm_backward_cuda_dispatch(const Tensor&, const Tensor&, const Tensor&, const std::vector<int64_t>&, float, Tensor&, Tensor&, Tensor&) { not_provided("layer_norm_backward"); }
void layer_norm_cuda_dispatch(const Tensor&, const std::vector<int64_t>&, const Tensor&, const Tensor&, float, Tensor&) { not_provided("layer_norm"); }
void lerp_cuda_dispatch(Tensor&, const Tensor&, float) { not_provided("lerp"); }
void log_cuda_dispatch(const Tensor&, const std::vector<int64_t>&, Tensor&) { not_provided("log"); }
void masked_fill_cuda_dispatch(Tensor&, const Tensor&, float) { not_provided("masked_fill"); }
void max_cols_cuda_dispatch(const Tensor&, Tensor&) { not_provided("max_cols"); }
void max_pool2d_backward_cuda_dispatch(const Tensor&, const Tensor&, Tensor&) { not_provided("max_pool2d_backward"); }
void max_pool2d_cuda_dispatch(const Tensor&, Tensor&, Tensor&, int, int, int, int, int, int) { not_provided("max_pool2d"); }
void multinomial_cuda_dispatch(const Tensor&, Tensor&, int64_t, unsigned long) { not_provided("multinomial"); }
void repetition_penalty_cuda_dispatch(const Tensor&, Tensor&, const Tensor&, float) { not_provided("repetition_penalty"); }
void rms_norm_backward_cuda_dispatch(const Tensor&, const Tensor&, const Tensor&, const std::vector<int64_t>&, float, Tensor&, Tensor&) { not_provided("rms_norm_backward"); }
void rms_norm_cuda_dispatch(const Tensor&, const std::vector<int64_t>&, const Tensor&, float, Tensor&) { not_provided("rms_norm"); }
void scatter_cuda_dispatch(Tensor&, int64_t, const Tensor&, const Tensor&) { not_provided("scatter"); }
void scatter_scalar_cuda_dispatch(Tensor&, int64_t, const Tensor&, float) { not_provided("scatter"); }
void sign_cuda_dispatch(const Tensor&, const std::vector<int64_t>&, Tensor&) { not_provided("sign"); }
void silu_backward_cuda_dispatch(const Tensor&, const Tensor&, Tensor&) { not_provided("silu_backward"); }
void silu_cuda_dispatch(const Tensor&, const std::vector<int64_t>&, Tensor&) { not_provided("silu"); }
void silu_inplace_cuda_dispatch(Tensor&) { not_provided("silu_"); }
void silu_mul_cuda_dispatch(const Tensor&, const Tensor&, Tensor&) { not_provided("silu_mul"); }
void sin_cuda_dispatch(const Tensor&, const std::vector<int64_t>&, Tensor&) { not_provided("sin"); }
void sqrt_cuda_dispatch(const Tensor&, const std::vector<int64_t>&, Tensor&) { not_provided("sqrt"); }
void sum_cols_cuda_dispatch(const Tensor&, Tensor&) { not_provided("sum_cols"); }
void sum_cuda_dispatch(const Tensor&, Tensor&) { not_provided("sum"); }
void top_k_filter_cuda_dispatch(const Tensor&, Tensor&, int64_t) { not_provided("top_k_filter"); }
void top_p_filter_cuda_dispatch(const Tensor&, Tensor&, float) { not_provided("top_p_filter"); }
void topk_cuda_dispatch(const Tensor&, int64_t, Tensor&, Tensor&) { not_provided("topk"); }
void where_cuda_dispatch(const Tensor&, const Tensor&, const Tensor&, Tensor&) { not_provided("where"); }

}  // namespace ops

namespace nn {

// x [batch, heads, seq_len, head_dim] fp32, rotated in place with the caller's [seq_len, head_dim/2] tables
void apply_rope_cuda(float* x, const float* cos, const float* sin, int batch, int heads, int seq_len, int head_dim) {
    check(vb200_apply_rope(-1, stream(), x, cos, sin, batch, heads, seq_len, head_dim), "apply_rope");
}
void apply_rope_inverse_cuda(float*, const float*, const float*, int, int, int, int) { not_provided("apply_rope_inverse"); }

namespace functional {
void relu_cuda_dispatch(const Tensor&, Tensor&) { not_provided("relu"); }
void sigmoid_cuda_dispatch(const Tensor&, Tensor&) { not_provided("sigmoid"); }
}  // namespace functional

}  // namespace nn
}  // namespace vesper
