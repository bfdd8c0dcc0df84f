// generation::Generator: greedy generation whose per-token state never leaves the GPU.
#include <vesper/generation/generator.h>

#include <cuda_runtime.h>

#include <algorithm>
#include <stdexcept>
#include <string>

namespace vesper::generation {

namespace {
void cuda_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string("Generator: ") + what + ": " + cudaGetErrorString(e));
}
struct EventPair {
    cudaEvent_t a = nullptr, b = nullptr;
    EventPair() { cuda_check(cudaEventCreate(&a), "cudaEventCreate"); cuda_check(cudaEventCreate(&b), "cudaEventCreate"); }
    ~EventPair() { cudaEventDestroy(a); cudaEventDestroy(b); }
    double ms() const { float t = 0; cudaEventElapsedTime(&t, a, b); return t; }
};
}  // namespace

Tensor Generator::generate(const Tensor& prompt_ids, const SamplingParams& params) {
    if (prompt_ids.ndim() != 2) throw std::runtime_error("prompt_ids must be 2D [Batch, SeqLen]");
    if (params.do_sample) throw std::runtime_error("Generator: only greedy decoding (do_sample = false) is built on this path");
    if (params.repetition_penalty != 1.0f) throw std::runtime_error("Generator: repetition_penalty is not part of this path");
    const int64_t B = prompt_ids.shape()[0], P = prompt_ids.shape()[1], max_new = params.max_new_tokens;
    const auto& cfg = model_->config();
    if (P + max_new > cfg.max_seq_len) throw std::runtime_error("Total sequence length would exceed model's max_seq_len");
    const Device out_device = prompt_ids.device();
    // the loop runs on a stream of its own (the legacy default stream cannot be captured into a graph);
    // work already queued on the caller's stream is waited for first, and the caller's stream is current
    // again on return
    Stream& callers = Stream::current(Device::CUDA);
    callers.synchronize();
    Stream own(Device::CUDA);
    Stream::set_current(own);
    struct Restore { Stream& s; ~Restore() { Stream::set_current(s); } } restore{callers};
    cudaStream_t stream = static_cast<cudaStream_t>(own.raw_handle());
    timings_ = GenerationTimings{};

    model_->init_cache(B, Device::CUDA);

    // device-resident loop state
    models::TransformerLM::DecodeState st;
    st.ids = zeros({B}, DType::Int32, Device::CUDA);
    st.done = zeros({B}, DType::Int32, Device::CUDA);
    st.history = zeros({B, P + max_new}, DType::Int32, Device::CUDA);
    st.lens = empty({B}, DType::Int32, Device::CUDA);
    st.prompt_len = P;
    st.min_new_tokens = params.min_new_tokens;
    st.max_len = P + max_new;
    {
        std::vector<int32_t> lens(static_cast<size_t>(B), static_cast<int32_t>(P));
        st.lens.copy_from_host(lens.data());
        if (!params.stop_token_ids.empty()) {
            std::vector<int32_t> stop(params.stop_token_ids.begin(), params.stop_token_ids.end());
            st.stop_ids = empty({static_cast<int64_t>(stop.size())}, DType::Int32, Device::CUDA);
            st.stop_ids.copy_from_host(stop.data());
        }
    }
    // the prompt as contiguous int32 on the device; history[:, :P] = prompt
    Tensor prompt_dev;
    {
        Tensor host_prompt = prompt_ids.to(Device::CPU).contiguous();
        std::vector<int32_t> p32(static_cast<size_t>(B * P));
        for (int64_t i = 0; i < B * P; ++i)
            p32[static_cast<size_t>(i)] = host_prompt.dtype() == DType::Int64 ? static_cast<int32_t>(host_prompt.data_ptr<int64_t>()[i])
                                                                               : host_prompt.data_ptr<int32_t>()[i];
        prompt_dev = empty({B, P}, DType::Int32, Device::CUDA);
        prompt_dev.copy_from_host(p32.data());
        cuda_check(cudaMemcpy2DAsync(st.history.data_ptr<int32_t>(), sizeof(int32_t) * (P + max_new), prompt_dev.data_ptr<int32_t>(),
                                     sizeof(int32_t) * P, sizeof(int32_t) * P, static_cast<size_t>(B), cudaMemcpyDeviceToDevice, stream),
                   "cudaMemcpy2DAsync");
    }

    // prefill at position 0 and the first pick (src/generation/generator.cpp:62-66, 76-88)
    EventPair pre, dec;
    cuda_check(cudaEventRecord(pre.a, stream), "cudaEventRecord");
    model_->forward_with_cache(prompt_dev, 0, /*last_only=*/true);
    int64_t generated = 0;
    if (max_new > 0) {
        model_->pick_from_last_logits(st);
        generated = 1;
    }
    cuda_check(cudaEventRecord(pre.b, stream), "cudaEventRecord");

    // decode: step i feeds the token picked at step i-1 (position P + i - 1) and picks the next
    const bool graph_ok = use_graph_ && cfg.head_dim() == 128 && max_new > 2;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    std::vector<int32_t> done_host(static_cast<size_t>(B));
    auto all_done = [&]() {
        st.done.copy_to_host(done_host.data());
        for (int32_t d : done_host) if (!d) return false;
        return true;
    };
    cuda_check(cudaEventRecord(dec.a, stream), "cudaEventRecord");
    bool stopped = max_new > 0 && !params.stop_token_ids.empty() && all_done();
    int64_t steps = 0;
    while (!stopped && generated < max_new) {
        if (cfg.head_dim() != 128) {
            // host-positioned fallback for head sizes without the device-position decode kernel
            Tensor tok = st.ids.view({B, 1});
            model_->forward_with_cache(tok, P + generated - 1, true);
            std::vector<int32_t> lens(static_cast<size_t>(B), static_cast<int32_t>(P + generated));
            st.lens.copy_from_host(lens.data());
            model_->pick_from_last_logits(st);
        } else if (graph_ok && steps >= 1) {
            if (!exec) {
                // the first step ran eagerly (buffers exist, kernels are configured); capture the second
                cuda_check(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
                try {
                    model_->decode_step(st);
                } catch (...) {
                    cudaGraph_t g = nullptr;
                    cudaStreamEndCapture(stream, &g);
                    if (g) cudaGraphDestroy(g);
                    throw;
                }
                cuda_check(cudaStreamEndCapture(stream, &graph), "cudaStreamEndCapture");
                cuda_check(cudaGraphInstantiate(&exec, graph, 0), "cudaGraphInstantiate");
                timings_.graph_replay = true;
            }
            cuda_check(cudaGraphLaunch(exec, stream), "cudaGraphLaunch");
        } else {
            model_->decode_step(st);
        }
        ++generated;
        ++steps;
        if (!params.stop_token_ids.empty() && (steps % poll_every_ == 0 || generated == max_new)) stopped = all_done();
    }
    cuda_check(cudaEventRecord(dec.b, stream), "cudaEventRecord");
    cuda_check(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
    if (exec) cudaGraphExecDestroy(exec);
    if (graph) cudaGraphDestroy(graph);
    timings_.prefill_ms = pre.ms();
    timings_.decode_ms = dec.ms();
    timings_.decode_steps = steps;

    model_->clear_cache();
    if (!params.stop_token_ids.empty() && generated > 0) {
        // The done mask is polled only every few steps, so the loop may have run past the step at which
        // the last sequence stopped; the reference ends right there (src/generation/generator.cpp:109-119).
        std::vector<int32_t> hist(static_cast<size_t>(B * (P + max_new)));
        st.history.copy_to_host(hist.data());
        int64_t cut = 0;
        bool every_sequence_stopped = true;
        for (int64_t b = 0; b < B && every_sequence_stopped; ++b) {
            int64_t first = -1;
            for (int64_t i = 0; i < generated && first < 0; ++i) {
                if (i + 1 < params.min_new_tokens) continue;
                const int32_t tok = hist[static_cast<size_t>(b * (P + max_new) + P + i)];
                for (int64_t sid : params.stop_token_ids) if (tok == static_cast<int32_t>(sid)) { first = i; break; }
            }
            if (first < 0) every_sequence_stopped = false;
            else cut = std::max(cut, first + 1);
        }
        if (every_sequence_stopped) generated = std::min(generated, cut);
    }
    Tensor result = empty({B, P + generated}, DType::Int32, Device::CUDA);
    cuda_check(cudaMemcpy2DAsync(result.data_ptr<int32_t>(), sizeof(int32_t) * (P + generated), st.history.data_ptr<int32_t>(),
                                 sizeof(int32_t) * (P + max_new), sizeof(int32_t) * (P + generated), static_cast<size_t>(B),
                                 cudaMemcpyDeviceToDevice, stream),
               "cudaMemcpy2DAsync");
    cuda_check(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
    return out_device == Device::CUDA ? result : result.to(out_device);
}

}  // namespace vesper::generation
