// generation::Generator -- greedy generation with the reference's loop structure
// (include/vesper/generation/generator.h:30-76, src/generation/generator.cpp:36-142): prefill the
// prompt at position 0, then one token per iteration; a sequence is done once it emits a stop token
// after min_new_tokens; the loop ends at max_new_tokens or when every sequence is done.
//
// B200 form: the sampled ids, the per-sequence lengths, the done mask and the token history stay
// on the device; one decode step is captured in a CUDA graph and replayed, and the host reads the
// done mask only every `poll_every` steps instead of the reference's copy per token (:100-107).
#pragma once
#include <vesper/core/tensor.h>
#include <vesper/models/transformer.h>

#include <cstdint>
#include <vector>

namespace vesper::generation {

struct SamplingParams {
    float temperature = 1.0f;
    int64_t top_k = 0;
    float top_p = 1.0f;
    float repetition_penalty = 1.0f;
    int64_t min_new_tokens = 0;
    int64_t max_new_tokens = 256;
    std::vector<int64_t> stop_token_ids;
    bool do_sample = true;       // only do_sample == false (greedy) is built on this path
    int64_t seed = -1;
};

struct GenerationTimings {
    double prefill_ms = 0.0;     // device time of the prompt pass (CUDA events)
    double decode_ms = 0.0;      // device time of all decode steps
    int64_t decode_steps = 0;
    bool graph_replay = false;
};

class Generator {
public:
    explicit Generator(models::TransformerLM* model) : model_(model) {}

    // prompt_ids [Batch, PromptLen] Int32 / Int64; returns [Batch, PromptLen + generated] Int32 on
    // the prompt's device.
    Tensor generate(const Tensor& prompt_ids, const SamplingParams& params);

    void set_use_graph(bool on) { use_graph_ = on; }
    void set_poll_every(int n) { poll_every_ = n > 0 ? n : 1; }
    const GenerationTimings& last_timings() const { return timings_; }
    models::TransformerLM* model() { return model_; }

private:
    models::TransformerLM* model_;
    bool use_graph_ = true;
    int poll_every_ = 16;
    GenerationTimings timings_;
};

}  // namespace vesper::generation
