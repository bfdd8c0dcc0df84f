// ops::repeat_kv (include/vesper/ops/attention_ops.h:21 of the reference).
// The attention entry points index KV heads directly and never need it; it is
// kept for code that still materialises the expansion.  Unlike the reference
// dispatchers (src/ops/attention_ops.cpp:34-52) it honours the input's strides.
#pragma once
#include <vesper/core/tensor.h>

namespace vesper::ops {
Tensor repeat_kv(const Tensor& x, int64_t n_rep);
void repeat_kv_cuda_dispatch(const Tensor& input, Tensor& output, int64_t n_rep);
}  // namespace vesper::ops
