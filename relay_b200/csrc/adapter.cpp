// The reference-side binding: relay::Backend implemented over the C boundary
// (include/relay_b200.h). It defines the two symbols engine/include/relay/backend.h:84-98
// declares under RELAY_CUDA and only engine/src/cuda_backend.cu defines — make_cuda_backend
// and CudaOptions::from_env — so relay's engine, transfer engine, worker, C API, tools and
// tests link against this file instead of cuda_backend.cu and run on the B200 backend
// unchanged. Compiled against the reference's headers (never copied into this tree):
//   g++ -std=c++20 -DRELAY_CUDA=1 -I<relay>/engine/include -Iinclude -c adapter.cpp
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "relay/backend.h"
#include "relay_b200.h"

namespace relay {

namespace {

// -1 from the C boundary back into the exception the reference's backend throws.
[[noreturn]] void rethrow() {
  const std::string what = rb200_last_error();
  switch (rb200_last_error_kind()) {
    case RB200_ERR_INVALID_ARGUMENT: throw std::invalid_argument(what);
    case RB200_ERR_OUT_OF_RANGE: throw std::out_of_range(what);
    case RB200_ERR_LOGIC: throw std::logic_error(what);
    default: throw std::runtime_error(what);
  }
}

void check(int rc) {
  if (rc < 0) rethrow();
}

class B200Backend final : public Backend {
 public:
  B200Backend(const HostWeights& w, int num_blocks, int block_size, int device, int max_batch_tokens, int max_context,
              CudaOptions options)
      : c_(w.config) {
    layout_ = {c_.layers, c_.kv_heads, c_.head_dim, block_size, num_blocks};
    rb200_model_config cc{};
    cc.hidden = c_.hidden;
    cc.intermediate = c_.intermediate;
    cc.layers = c_.layers;
    cc.heads = c_.heads;
    cc.kv_heads = c_.kv_heads;
    cc.head_dim = c_.head_dim;
    cc.vocab = c_.vocab;
    cc.max_position = c_.max_position;
    cc.rms_eps = c_.rms_eps;
    cc.rope_theta = c_.rope_theta;
    cc.rope_scaling_type = c_.rope_scaling.type == "llama3" ? 1 : 0;
    cc.rope_factor = c_.rope_scaling.factor;
    cc.rope_low_freq_factor = c_.rope_scaling.low_freq_factor;
    cc.rope_high_freq_factor = c_.rope_scaling.high_freq_factor;
    cc.rope_original_max_position = c_.rope_scaling.original_max_position;
    cc.tie_embeddings = w.lm_head.empty();
    cc.qkv_bias = !w.layers.empty() && !w.layers[0].bqkv.empty();
    std::vector<rb200_layer_weights> layers(w.layers.size());
    for (std::size_t l = 0; l < w.layers.size(); ++l) {
      const LayerWeights& L = w.layers[l];
      layers[l] = {L.attn_norm.data(), L.wqkv.data(), L.bqkv.empty() ? nullptr : L.bqkv.data(), L.wo.data(),
                   L.mlp_norm.data(), L.w_gate_up.data(), L.w_down.data()};
    }
    rb200_weights hw{w.embed.data(), w.final_norm.data(), w.lm_head.empty() ? nullptr : w.lm_head.data(), layers.data()};
    const uint32_t flags = (options.int8_weights ? RB200_INT8_WEIGHTS : 0) |
                           (options.reference_attention ? RB200_REFERENCE_ATTENTION : 0);
    h_ = rb200_create(&cc, &hw, num_blocks, block_size, device, max_batch_tokens, max_context, flags);
    if (!h_) rethrow();
  }
  ~B200Backend() override { rb200_destroy(h_); }

  const ModelConfig& config() const override { return c_; }
  const KVLayout& kv_layout() const override { return layout_; }
  std::string name() const override { return "cuda"; }  // what relay's tools print and tests expect of this slot

  std::vector<float> forward(const ForwardBatch& batch, LayerObserver* observer) override {
    std::vector<int32_t> tok, len, pos, tlen, tabs;
    std::vector<uint8_t> want;
    std::size_t rows = 0;
    for (const SeqChunk& ch : batch.seqs) {
      tok.insert(tok.end(), ch.tokens.begin(), ch.tokens.end());
      len.push_back(static_cast<int32_t>(ch.tokens.size()));
      pos.push_back(ch.start_pos);
      tlen.push_back(static_cast<int32_t>(ch.block_table.size()));
      tabs.insert(tabs.end(), ch.block_table.begin(), ch.block_table.end());
      want.push_back(ch.want_logits ? 1 : 0);
      rows += batch.all_logits ? ch.tokens.size() : (ch.want_logits && !ch.tokens.empty() ? 1 : 0);
    }
    std::vector<float> out(rows * static_cast<std::size_t>(c_.vocab));
    auto trampoline = [](void* ctx, int layer) { static_cast<LayerObserver*>(ctx)->kv_written(layer); };
    const int r = rb200_forward(h_, static_cast<int>(batch.seqs.size()), tok.data(), len.data(), pos.data(), tlen.data(),
                                tabs.data(), want.data(), batch.all_logits ? 1 : 0,
                                observer ? static_cast<rb200_layer_cb>(trampoline) : nullptr, observer, out.data(),
                                out.size());
    if (r < 0) rethrow();
    out.resize(static_cast<std::size_t>(r) * c_.vocab);
    return out;
  }

  std::size_t kv_block_bytes() const override { return rb200_kv_block_bytes(h_); }

  void read_kv_block(int layer, int block, void* k_out, void* v_out) override {
    const int32_t b = block;
    check(rb200_read_kv_layer(h_, layer, &b, 1, k_out, v_out));
  }
  void write_kv_block(int layer, int block, const void* k_in, const void* v_in) override {
    const int32_t b = block;
    check(rb200_write_kv_layer(h_, layer, &b, 1, k_in, v_in));
  }
  void read_kv_layer(int layer, const std::vector<int>& blocks, void* out) override {
    auto* k = static_cast<unsigned char*>(out);
    check(rb200_read_kv_layer(h_, layer, blocks.data(), static_cast<int>(blocks.size()), k,
                              k + blocks.size() * kv_block_bytes()));
  }
  void write_kv_layer(int layer, const std::vector<int>& blocks, const void* in) override {
    const auto* k = static_cast<const unsigned char*>(in);
    check(rb200_write_kv_layer(h_, layer, blocks.data(), static_cast<int>(blocks.size()), k,
                               k + blocks.size() * kv_block_bytes()));
  }
  void wait_kv_written(int layer) override { check(rb200_wait_kv_written(h_, layer)); }
  void update_weight(const std::string& name, const float* src, std::size_t n) override {
    check(rb200_update_weight(h_, name.c_str(), src, n));
  }

 private:
  ModelConfig c_;
  KVLayout layout_;
  rb200_backend* h_ = nullptr;
};

}  // namespace

CudaOptions CudaOptions::from_env() {
  const uint32_t f = rb200_flags_from_env();
  CudaOptions o;
  o.reference_attention = (f & RB200_REFERENCE_ATTENTION) != 0;
  o.int8_weights = (f & RB200_INT8_WEIGHTS) != 0;
  return o;
}

std::unique_ptr<Backend> make_cuda_backend(const HostWeights& weights, int num_blocks, int block_size, int device,
                                           int max_batch_tokens, int max_context, CudaOptions options) {
  return std::make_unique<B200Backend>(weights, num_blocks, block_size, device, max_batch_tokens, max_context, options);
}

}  // namespace relay
