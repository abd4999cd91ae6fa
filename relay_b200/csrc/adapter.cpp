// The reference-side binding: relay::Backend implemented over the C boundary
// (include/relay_b200.h). It defines the two symbols engine/include/relay/backend.h:84-98
// declares under RELAY_CUDA and only engine/src/cuda_backend.cu defines — make_cuda_backend
// and CudaOptions::from_env — so relay's engine, transfer engine, worker, C API, tools and
// tests link against this file instead of cuda_backend.cu and run on the B200 backend
// unchanged. Compiled against the reference's headers (never copied into this tree):
//   g++ -std=c++20 -DRELAY_CUDA=1 -I<relay>/engine/include -Iinclude -c adapter.cpp
#include <atomic>
#include <cstring>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "relay/backend.h"
#include "relay/kv_transfer.h"
#include "relay_b200.h"
#include "relay_b200_transfer.h"

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
    const int link = send_link_.load();
    if (link >= 0) {
      // A wrapped KVSender connection is attached: the pages leave over the link, ordered behind the
      // layer's K/V append on the device; `out` stays as it is and the wrapper drops it from the frame.
      check(rb200_kv_link_send_layer(h_, link, layer, blocks.data(), static_cast<int>(blocks.size())));
      // relay frees the blocks once the frame is written: they must have been read by then
      check(rb200_kv_link_wait_gathered(h_, link, 30000));
      posted_.fetch_add(1);
      return;
    }
    auto* k = static_cast<unsigned char*>(out);
    check(rb200_read_kv_layer(h_, layer, blocks.data(), static_cast<int>(blocks.size()), k,
                              k + blocks.size() * kv_block_bytes()));
  }
  void write_kv_layer(int layer, const std::vector<int>& blocks, const void* in) override {
    if (recv_link_.load() >= 0) {
      // A wrapped KVReceiver connection is attached: `in` holds nothing (the wrapper read no payload);
      // the pages come from the link and are in the cache when this returns.
      std::lock_guard<std::mutex> lock(recv_mu_);
      if (!pending_ || pending_layer_ != layer || pending_blocks_ != static_cast<int>(blocks.size()))
        throw std::logic_error("kv link: write_kv_layer does not match the Layer frame that was just read");
      pending_ = false;
      check(rb200_kv_link_recv_layer(h_, recv_link_.load(), layer, blocks.data(), static_cast<int>(blocks.size())));
      check(rb200_kv_link_wait(h_, recv_link_.load(), recv_timeout_ms_));
      return;
    }
    const auto* k = static_cast<const unsigned char*>(in);
    check(rb200_write_kv_layer(h_, layer, blocks.data(), static_cast<int>(blocks.size()), k,
                               k + blocks.size() * kv_block_bytes()));
  }
  void wait_kv_written(int layer) override { check(rb200_wait_kv_written(h_, layer)); }
  void update_weight(const std::string& name, const float* src, std::size_t n) override {
    check(rb200_update_weight(h_, name.c_str(), src, n));
  }

  // ---- the transfer engine over a K/V link (relay_b200_transfer.h) ----
  rb200_backend* handle() const { return h_; }
  void attach_sender(int link) {
    int none = -1;
    if (!send_link_.compare_exchange_strong(none, link)) throw std::logic_error("kv link: the backend already feeds a wrapped sender connection");
    posted_.store(0);
  }
  void detach_sender() { send_link_.store(-1); }
  // One Layer frame's payload has been sent over the link since the last call? (the wrapper asks per frame)
  bool take_posted() {
    int n = posted_.load();
    while (n > 0 && !posted_.compare_exchange_weak(n, n - 1)) {
    }
    return n > 0;
  }
  void attach_receiver(int link, int timeout_ms) {
    int none = -1;
    if (!recv_link_.compare_exchange_strong(none, link)) throw std::logic_error("kv link: the backend already lands a wrapped receiver connection");
    recv_timeout_ms_ = timeout_ms;
    pending_ = false;
  }
  void detach_receiver() {
    drop_pending();
    recv_link_.store(-1);
  }
  // The wrapper has read a Layer frame's header: its payload (n blocks of `layer`) waits on the link.
  void set_pending(int layer, int n) {
    std::lock_guard<std::mutex> lock(recv_mu_);
    pending_ = true;
    pending_layer_ = layer;
    pending_blocks_ = n;
  }
  // The frame was not written (the receiver had no room and dropped it): drop it from the link too.
  void drop_pending() {
    std::lock_guard<std::mutex> lock(recv_mu_);
    if (!pending_) return;
    pending_ = false;
    rb200_kv_link_skip_layer(h_, recv_link_.load(), pending_blocks_);
  }

 private:
  ModelConfig c_;
  KVLayout layout_;
  rb200_backend* h_ = nullptr;
  std::atomic<int> send_link_{-1}, recv_link_{-1}, posted_{0};
  std::mutex recv_mu_;
  bool pending_ = false;
  int pending_layer_ = 0, pending_blocks_ = 0, recv_timeout_ms_ = 30000;
};

B200Backend& as_b200(Backend& b) {
  auto* p = dynamic_cast<B200Backend*>(&b);
  if (!p) throw std::invalid_argument("kv link: not a backend of relay_b200 (relay::make_cuda_backend)");
  return *p;
}

bool layer_frame(const void* data, std::size_t len, FrameHeader* out) {
  if (len != sizeof(FrameHeader)) return false;
  std::memcpy(out, data, sizeof(FrameHeader));
  return out->magic == kFrameMagic;
}

// What a KVSender writes to: every frame goes to `inner` as it is, except that a Layer frame
// leaves only its header there (its payload went over the link inside read_kv_layer).
class LinkSenderConnection final : public Connection {
 public:
  LinkSenderConnection(Connection& inner, B200Backend& be, int link) : inner_(inner), be_(be) { be_.attach_sender(link); }
  ~LinkSenderConnection() override { be_.detach_sender(); }
  void send(const Slice* slices, int n) override {
    FrameHeader h;
    if (n >= 2 && layer_frame(slices[0].data, slices[0].len, &h) && h.type == static_cast<std::uint16_t>(FrameType::Layer) &&
        h.payload > 0) {
      if (!be_.take_posted()) throw std::logic_error("kv link: a Layer frame whose pages were not sent over the link");
      inner_.send(slices, 1);
      return;
    }
    inner_.send(slices, n);
  }
  void recv(void* dst, std::size_t len) override { inner_.recv(dst, len); }
  void close() override { inner_.close(); }
  std::string describe() const override { return "kv-link(" + inner_.describe() + ")"; }

 private:
  Connection& inner_;
  B200Backend& be_;
};

// What a KVReceiver reads from. It follows the frame stream (a 32-byte header, then `payload`
// bytes in one or more reads): the payload of a Layer frame is not on `inner`, so that read
// returns at once and the frame is remembered for write_kv_layer; if the next header is read
// while it is still remembered, the receiver has dropped the frame, and so does the link.
class LinkReceiverConnection final : public Connection {
 public:
  LinkReceiverConnection(Connection& inner, B200Backend& be, int link, int timeout_ms) : inner_(inner), be_(be) {
    be_.attach_receiver(link, timeout_ms);
    block_bytes_ = be.kv_block_bytes();
  }
  ~LinkReceiverConnection() override {
    try {
      be_.detach_receiver();
    } catch (...) {
    }
  }
  void send(const Slice* slices, int n) override { inner_.send(slices, n); }
  void recv(void* dst, std::size_t len) override {
    if (skip_ > 0) {  // the payload of the Layer frame whose header was just read
      if (len != skip_) throw std::logic_error("kv link: a Layer payload read in pieces");
      skip_ = 0;
      be_.set_pending(layer_, blocks_);
      return;
    }
    if (remaining_ > 0) {  // the payload of another kind of frame
      inner_.recv(dst, len);
      remaining_ -= len < remaining_ ? len : remaining_;
      return;
    }
    be_.drop_pending();
    inner_.recv(dst, len);
    FrameHeader h;
    if (!layer_frame(dst, len, &h)) return;
    if (h.type == static_cast<std::uint16_t>(FrameType::Layer) && h.payload > 0) {
      if (h.payload % (2 * block_bytes_) != 0) return;  // the receiver rejects it itself (engine/src/kv_transfer.cpp:277)
      skip_ = h.payload;
      layer_ = static_cast<int>(h.a);
      blocks_ = static_cast<int>(h.payload / (2 * block_bytes_));
    } else {
      remaining_ = h.payload;
    }
  }
  void close() override { inner_.close(); }
  std::string describe() const override { return "kv-link(" + inner_.describe() + ")"; }

 private:
  Connection& inner_;
  B200Backend& be_;
  std::size_t block_bytes_ = 0, skip_ = 0, remaining_ = 0;
  int layer_ = 0, blocks_ = 0;
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

namespace b200 {

KvLinkEnd kv_link_create(Backend& backend, int n_slots, std::size_t slot_bytes) {
  KvLinkEnd e;
  e.link = rb200_kv_link_create(as_b200(backend).handle(), n_slots, slot_bytes, e.handle);
  if (e.link < 0) rethrow();
  return e;
}

void kv_link_connect(Backend& backend, int link, const void* peer_handle) {
  check(rb200_kv_link_connect(as_b200(backend).handle(), link, peer_handle));
}

void kv_link_connect_local(Backend& a, int link_a, Backend& b, int link_b) {
  check(rb200_kv_link_connect_local(as_b200(a).handle(), link_a, as_b200(b).handle(), link_b));
}

void kv_link_close(Backend& backend, int link) { check(rb200_kv_link_close(as_b200(backend).handle(), link)); }

std::unique_ptr<Connection> kv_link_sender_connection(Connection& inner, Backend& backend, int link) {
  return std::make_unique<LinkSenderConnection>(inner, as_b200(backend), link);
}

std::unique_ptr<Connection> kv_link_receiver_connection(Connection& inner, Backend& backend, int link, int timeout_ms) {
  return std::make_unique<LinkReceiverConnection>(inner, as_b200(backend), link, timeout_ms);
}

}  // namespace b200

}  // namespace relay
