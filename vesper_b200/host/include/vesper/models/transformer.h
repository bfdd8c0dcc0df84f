// models::TransformerLM -- the inference surface of the reference's language model
// (include/vesper/models/transformer.h:39-152, src/models/transformer.cpp:43-206) for the
// Llama-style family: token embedding, N pre-norm blocks (RMSNorm -> fused QKV -> RoPE + cache
// append + grouped-query attention -> output projection -> residual; RMSNorm -> SwiGLU MLP ->
// residual, src/models/transformer_block.cpp:183-205), final RMSNorm, untied LM head.
//
// B200 layout: weights bf16 (the gate / up projections interleaved row by row so the SwiGLU product
// is the GEMM epilogue), residual stream fp32, activations bf16, one bf16 KV cache per layer
// [B, kv_heads, max_seq_len, head_dim], per-sequence lengths on the device.  The attention kernels
// read q/k/v straight out of the fused QKV buffer through strides ([B,T,H,D] memory seen as
// [B,H,T,D]) and write the head-merged layout the output projection wants: none of the reference's
// transposes / .contiguous() copies (src/nn/gqa_attention.cpp:117-122,151) exist here.
#pragma once
#include <vesper/core/tensor.h>
#include <vesper/models/config.h>
#include <vesper/nn/transformer.h>

#include <map>
#include <memory>
#include <string>
#include <vector>

namespace vesper::models {

class TransformerLM {
public:
    explicit TransformerLM(const TransformerConfig& config);
    ~TransformerLM();

    // Parameter names and shapes as the reference's named_parameters() reports them:
    // tok_embeddings.weight, layers.N.attention_norm.weight, layers.N.attention.wqkv.weight,
    // layers.N.attention.wo.weight, layers.N.ffn_norm.weight, layers.N.feed_forward.{gate,up,down}_proj.weight,
    // norm.weight, output.weight.
    std::map<std::string, std::vector<int64_t>> parameter_shapes() const;
    // Loads one parameter from host fp32 values (rounded to bf16 for matrices; norm weights stay fp32).
    void load_parameter(const std::string& name, const float* host_values, int64_t numel);

    // tokens [Batch, NewTokens] Int32 or Int64 (CPU or CUDA); returns fp32 logits
    // [Batch, NewTokens, Vocab], or [Batch, 1, Vocab] for the last position when last_only.
    Tensor forward_with_cache(const Tensor& tokens, int64_t start_pos, bool last_only = false);

    void init_cache(int64_t batch_size, Device device);
    void clear_cache();
    bool has_cache() const { return !kv_caches_.empty(); }
    const TransformerConfig& config() const { return config_; }
    int64_t num_parameters() const;

    // ---- device-resident decode step, used by generation::Generator ----
    // One greedy decode step for the whole batch with no host round trip: embeds ids_dev
    // [Batch] int32, runs every block at the per-sequence positions in the device length array
    // (advanced by one inside), writes logits and the arg-max ids back into ids_dev; appends the new
    // id to history_dev [Batch, history_ld] at column = the new length and updates done_dev.
    // All launches go to the current stream and are CUDA-graph capturable after one eager call.
    struct DecodeState {
        Tensor ids;        // [B] int32: in = token to process, out = next token
        Tensor lens;       // [B] int32: cached length per sequence
        Tensor history;    // [B, history_ld] int32
        Tensor done;       // [B] int32
        Tensor stop_ids;   // [n_stop] int32 (may be undefined)
        int64_t prompt_len = 0;
        int64_t min_new_tokens = 0;
        int64_t max_len = 0;          // upper bound of any sequence length during the loop (plans the split-KV launch)
    };
    void decode_step(DecodeState& st);
    // Greedy pick on the logits of the last forward_with_cache(..., last_only=true) call: writes
    // st.ids, st.history[:, lens], st.done.
    void pick_from_last_logits(DecodeState& st);

private:
    struct Layer;
    struct Buffers;
    void ensure_buffers(int64_t rows, int64_t batch);
    void run_blocks(int64_t B, int64_t T, int64_t start_pos, bool device_positions, int* lens_dev, int64_t max_len);

    TransformerConfig config_;
    Tensor tok_emb_;                       // [vocab, dim] bf16
    Tensor final_norm_;                    // [dim] fp32
    Tensor lm_head_;                       // [vocab, dim] bf16
    std::vector<std::unique_ptr<Layer>> layers_;
    std::vector<std::unique_ptr<nn::KVCache>> kv_caches_;
    std::unique_ptr<Buffers> buf_;
    float inv_freq_[64];
};

}  // namespace vesper::models
