// The backend: owns device weights, KV pools and activations, flattens a batch, routes its
// tokens to the decode / prefill attention kernels and sequences one forward pass on its
// stream. Behaviour, argument checks and error texts follow the reference's CudaBackend
// (engine/src/cuda_backend.cu:311-759) so that relay's engine, transfer engine and tests can
// drive it unchanged through the adapter; the kernels are this repository's own.
#include "backend.h"

#include <chrono>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <thread>

namespace rb200 {

// ---- error slot, device helpers ---------------------------------------------------------

namespace {
thread_local std::string g_error;
thread_local int g_error_kind = RB200_OK;
}  // namespace

void set_last_error(int kind, const std::string& what) {
  g_error = what;
  g_error_kind = kind;
}

std::atomic<uint64_t>& launch_counter() {
  static std::atomic<uint64_t> n{0};
  return n;
}

int sm_count() {
  static std::atomic<int> cached[64];  // zero-initialised; racing first calls store the same value
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return 148;  // B200; only used for planning when no device is present
  }
  if (cached[dev].load(std::memory_order_relaxed) == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = 148;
    }
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return cached[dev].load(std::memory_order_relaxed);
}

DeviceBuf::DeviceBuf(size_t n, bool zero) : bytes(n) {
  if (n == 0) return;
  RB_CUDA(cudaMalloc(&p, n));
  if (zero) RB_CUDA(cudaMemset(p, 0, n));
}
std::atomic<bool> g_device_wedged{false};

DeviceBuf::~DeviceBuf() {
  if (p && !g_device_wedged.load()) cudaFree(p);  // cudaFree waits for the whole device
}
DeviceBuf& DeviceBuf::operator=(DeviceBuf&& o) noexcept {
  if (this != &o) {
    if (p && !g_device_wedged.load()) cudaFree(p);
    p = o.p;
    bytes = o.bytes;
    o.p = nullptr;
    o.bytes = 0;
  }
  return *this;
}
void DeviceBuf::ensure(size_t n) {
  if (n <= bytes) return;
  *this = DeviceBuf(n);
}

PinnedBuf::~PinnedBuf() {
  if (p && !g_device_wedged.load()) cudaFreeHost(p);
}
void PinnedBuf::ensure(size_t n) {
  if (n <= bytes) return;
  if (p) RB_CUDA(cudaFreeHost(p));
  p = nullptr;
  bytes = 0;
  RB_CUDA(cudaMallocHost(&p, n));
  bytes = n;
}

WeightView Matrix::view() const {
  WeightView v;
  if (int8) {
    v.i8 = data.as<int8_t>();
    v.scale = scale.as<float>();
  } else {
    v.f16 = data.as<__half>();
  }
  v.N = N;
  v.K = ld;  // the padded width: columns K..ld-1 are zero on both sides of the product
  v.ld = ld;
  return v;
}

// ---- construction -----------------------------------------------------------------------

namespace {
constexpr int kPad = 64;                                 // k granularity of the GEMM / GEMV kernels
constexpr size_t kStageFloats = size_t(16) << 20;        // 64 MB staging for weight uploads

void rope_inv_freq(const rb200_model_config& c, std::vector<float>& inv) {
  // ModelConfig::rope_inv_freq (engine/src/config.cpp:79-109)
  const int half = c.head_dim / 2;
  inv.resize(half);
  for (int i = 0; i < half; ++i) {
    const float exponent = static_cast<float>(2 * i) / static_cast<float>(c.head_dim);
    inv[i] = 1.0f / std::pow(static_cast<float>(c.rope_theta), exponent);
  }
  if (c.rope_scaling_type == 1) {
    const double pi = 3.14159265358979323846;
    const double low_wavelen = c.rope_original_max_position / c.rope_low_freq_factor;
    const double high_wavelen = c.rope_original_max_position / c.rope_high_freq_factor;
    for (int i = 0; i < half; ++i) {
      const float f = inv[i];
      const float wavelen = 2.0f * static_cast<float>(pi) / f;
      float scaled = wavelen > low_wavelen ? f / static_cast<float>(c.rope_factor) : f;
      if (!(wavelen < high_wavelen) && !(wavelen > low_wavelen)) {
        const float smooth = static_cast<float>((c.rope_original_max_position / wavelen - c.rope_low_freq_factor) /
                                                (c.rope_high_freq_factor - c.rope_low_freq_factor));
        scaled = (1 - smooth) * f / static_cast<float>(c.rope_factor) + smooth * f;
      }
      inv[i] = scaled;
    }
  }
}
}  // namespace

void Backend::set_device() const {
  // Every entry point passes here: once a stream has been abandoned behind a wait nobody will
  // satisfy, further work in this process could block for ever in a device-wide synchronisation.
  if (g_device_wedged.load())
    fail(RB200_ERR_RUNTIME, "a K/V link stream of this process is stuck behind an unreleased wait; the process must be restarted");
  RB_CUDA(cudaSetDevice(device_));
}

Matrix Backend::make_matrix(int N, int K, bool int8) {
  Matrix m;
  m.N = N;
  m.K = K;
  m.ld = round_up(K, kPad);
  m.int8 = int8;
  m.data = DeviceBuf(static_cast<size_t>(N) * m.ld * (int8 ? 1 : 2), true);
  if (int8) {
    m.scale = DeviceBuf(static_cast<size_t>(N) * 4);
    std::vector<float> ones(N, 1.0f);  // the scale of an all-zero row (engine/src/cuda_backend.cu:295)
    RB_CUDA(cudaMemcpy(m.scale.p, ones.data(), ones.size() * 4, cudaMemcpyHostToDevice));
  }
  return m;
}

template <class F>
void Backend::for_row_chunks(const float* src, int rows, int cols, F&& apply) {
  cudaPointerAttributes a{};
  bool local = false;
  if (cudaPointerGetAttributes(&a, src) == cudaSuccess) {
    local = (a.type == cudaMemoryTypeDevice && a.device == device_) || a.type == cudaMemoryTypeManaged;
  } else {
    cudaGetLastError();  // plain host memory on older drivers
  }
  if (local) {
    apply(src, 0, rows);
    return;
  }
  const size_t per = std::max<size_t>(1, kStageFloats / static_cast<size_t>(cols));
  stage_.ensure(std::min<size_t>(per, rows) * cols * 4);
  for (size_t r0 = 0; r0 < static_cast<size_t>(rows); r0 += per) {
    const size_t nr = std::min(per, rows - r0);
    // cudaMemcpyDefault: host memory or another GPU's memory (peer copy), decided by the address
    RB_CUDA(cudaMemcpyAsync(stage_.p, src + r0 * cols, nr * cols * 4, cudaMemcpyDefault, stream_));
    apply(stage_.as<float>(), static_cast<int>(r0), static_cast<int>(nr));
  }
}

void Backend::upload_matrix(Matrix& m, const float* src, int N, int K) {
  for_row_chunks(src, N, K, [&](const float* dev, int r0, int nr) {
    if (m.int8)
      launch_quantize_rows_int8(dev, m.data.as<int8_t>() + static_cast<size_t>(r0) * m.ld, m.scale.as<float>() + r0, nr, K,
                                m.ld, stream_);
    else
      launch_convert_rows_f16(dev, m.data.as<__half>() + static_cast<size_t>(r0) * m.ld, nr, K, m.ld, stream_);
  });
  RB_CUDA(cudaGetLastError());
  RB_CUDA(cudaStreamSynchronize(stream_));
}

void Backend::upload_vector(DeviceBuf& dst, const float* src, size_t n) {
  RB_CUDA(cudaMemcpyAsync(dst.p, src, n * 4, cudaMemcpyDefault, stream_));
  RB_CUDA(cudaStreamSynchronize(stream_));
}

Backend::Backend(const rb200_model_config& cfg, const rb200_weights* w, int num_blocks, int block_size, int device,
                 int max_batch_tokens, int max_context, uint32_t flags)
    : c_(cfg), flags_(flags), device_(device), num_blocks_(num_blocks), block_size_(block_size),
      max_tokens_(max_batch_tokens), max_context_(max_context) {
  RB_REQUIRE(c_.hidden > 0 && c_.intermediate > 0 && c_.layers > 0 && c_.heads > 0 && c_.kv_heads > 0 &&
                 c_.head_dim > 0 && c_.vocab > 0,
             "model config: sizes must be positive");
  RB_REQUIRE(c_.heads % c_.kv_heads == 0, "num_attention_heads must be a multiple of num_key_value_heads");
  RB_REQUIRE(c_.head_dim % 2 == 0, "head_dim must be even");
  RB_REQUIRE(num_blocks > 0 && block_size > 0 && max_batch_tokens > 0 && max_context > 0, "backend: sizes must be positive");
  RB_REQUIRE(kv_block_bytes() % 16 == 0, "a KV block must be a multiple of 16 bytes");
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
    cudaGetLastError();
    fail(RB200_ERR_RUNTIME, "no CUDA device: the B200 backend has no CPU fallback");
  }
  RB_REQUIRE(device >= 0 && device < ndev, "backend: no such CUDA device");
  set_device();
  RB_CUDA(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
  RB_CUDA(cudaStreamCreateWithFlags(&copy_stream_, cudaStreamNonBlocking));
  layer_done_.resize(c_.layers);
  for (auto& e : layer_done_) RB_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));

  const int H = c_.hidden, D = c_.head_dim, Q = c_.heads * D, KV = c_.kv_heads * D, QKV = Q + 2 * KV, I = c_.intermediate;
  Hp_ = round_up(H, kPad);
  Qp_ = round_up(Q, kPad);
  Ip_ = round_up(I, kPad);
  const AttnShape shape{c_.heads, c_.kv_heads, D, block_size_, QKV, Qp_, pool_rows()};
  fast_attention_ = !(flags_ & RB200_REFERENCE_ATTENTION) && fast_attention_supported(shape);

  const bool q8 = flags_ & RB200_INT8_WEIGHTS;
  embed_ = make_matrix(c_.vocab, H, false);
  if (!c_.tie_embeddings) lm_head_ = make_matrix(c_.vocab, H, false);
  final_norm_ = DeviceBuf(static_cast<size_t>(H) * 4, true);
  {
    std::vector<float> inv;
    rope_inv_freq(c_, inv);
    inv_freq_ = DeviceBuf(inv.size() * 4);
    RB_CUDA(cudaMemcpy(inv_freq_.p, inv.data(), inv.size() * 4, cudaMemcpyHostToDevice));
  }
  layers_.resize(c_.layers);
  // The largest counters-and-partials region of any matrix, plus the largest digit buffer (64 tokens).
  size_t gemv_head = std::max(gemv_scratch_bytes(c_.vocab, Hp_, 0), size_t(256)), gemv_digits = i8_digits_bytes(64, Hp_);
  for (Layer& L : layers_) {
    L.attn_norm = DeviceBuf(static_cast<size_t>(H) * 4, true);
    L.mlp_norm = DeviceBuf(static_cast<size_t>(H) * 4, true);
    if (c_.qkv_bias) L.bqkv = DeviceBuf(static_cast<size_t>(QKV) * 4, true);
    L.wqkv = make_matrix(QKV, H, q8);
    L.wo = make_matrix(H, Q, q8);
    L.w_gate_up = make_matrix(2 * I, H, q8);
    L.w_down = make_matrix(H, I, q8);
  }
  for (const Matrix* m : {&layers_[0].wqkv, &layers_[0].wo, &layers_[0].w_gate_up, &layers_[0].w_down})
  {
    gemv_head = std::max(gemv_head, gemv_scratch_bytes(m->N, m->ld, 0));
    gemv_digits = std::max(gemv_digits, i8_digits_bytes(64, m->ld));
  }
  gemv_scratch_ = DeviceBuf(gemv_head + gemv_digits + 256, true);

  if (w) {
    RB_REQUIRE(w->embed && w->final_norm && w->layers, "weights: embed, final_norm and layers are required");
    RB_REQUIRE(c_.tie_embeddings || w->lm_head, "weights: lm_head is required unless embeddings are tied");
    upload_matrix(embed_, w->embed, c_.vocab, H);
    if (!c_.tie_embeddings) upload_matrix(lm_head_, w->lm_head, c_.vocab, H);
    upload_vector(final_norm_, w->final_norm, H);
    for (int l = 0; l < c_.layers; ++l) {
      const rb200_layer_weights& s = w->layers[l];
      Layer& L = layers_[l];
      RB_REQUIRE(s.attn_norm && s.wqkv && s.wo && s.mlp_norm && s.w_gate_up && s.w_down, "weights: a layer tensor is missing");
      RB_REQUIRE(!c_.qkv_bias || s.bqkv, "weights: bqkv is required when qkv_bias is set");
      upload_vector(L.attn_norm, s.attn_norm, H);
      upload_vector(L.mlp_norm, s.mlp_norm, H);
      if (c_.qkv_bias) upload_vector(L.bqkv, s.bqkv, QKV);
      upload_matrix(L.wqkv, s.wqkv, QKV, H);
      upload_matrix(L.wo, s.wo, H, Q);
      upload_matrix(L.w_gate_up, s.w_gate_up, 2 * I, H);
      upload_matrix(L.w_down, s.w_down, H, I);
    }
  }

  // K and V pools: [layers][num_blocks][kv_heads][block_size][head_dim] fp16, zeroed
  // (engine/src/cuda_backend.cu:368-371).
  const size_t pool = static_cast<size_t>(layer_elems()) * c_.layers * 2;
  kc_ = DeviceBuf(pool, true);
  vc_ = DeviceBuf(pool, true);

  const size_t T = max_tokens_;
  x_ = DeviceBuf(T * H * 4);
  xn_ = DeviceBuf(T * Hp_ * 2, true);
  qkv_ = DeviceBuf(T * QKV * 4);
  attn_ = DeviceBuf(T * Qp_ * 2, true);  // columns q_dim..Qp_-1 stay zero forever
  gu_ = DeviceBuf(T * 2 * I * 4);
  act_ = DeviceBuf(T * Ip_ * 2, true);
  if (fast_attention_) {
    const size_t want = decode_scratch_bytes(shape, max_tokens_, max_context_);
    if (want <= (size_t(1) << 30)) decode_scratch_ = DeviceBuf(want);
  }
  RB_CUDA(cudaDeviceSynchronize());
}

Backend::~Backend() {
  cudaSetDevice(device_);
  nccl_finalize_noexcept();
  try {  // a link wait the peer never satisfied must not block the destructor: before any device-wide sync
    bool idle = links_idle();
    for (int i = 0; i < 50 && !idle; ++i) {  // work in flight gets half a second to drain
      std::this_thread::sleep_for(std::chrono::milliseconds(10));
      idle = links_idle();
    }
    if (!idle) links_release();
  } catch (...) {
  }
  if (!g_device_wedged.load()) cudaDeviceSynchronize();
  session_.reset();
  links_.clear();
  if (pass_done_) cudaEventDestroy(pass_done_);
  for (auto e : layer_done_) cudaEventDestroy(e);
  for (IdSlot& s : id_slots_)
    if (s.uploaded) cudaEventDestroy(s.uploaded);
  if (stream_) cudaStreamDestroy(stream_);
  if (copy_stream_) cudaStreamDestroy(copy_stream_);
}

// ---- forward ------------------------------------------------------------------------------

Backend::PickSpec Backend::pick_of(const Outputs& out, int R) const {
  PickSpec pick;
  if (!out.tokens) return pick;
  pick.kind = out.sampling ? Pick::Sample : Pick::Greedy;
  pick.logprobs = out.logprobs != nullptr;
  if (out.sampling)
    for (int r = 0; r < R; ++r) {
      const rb200_sampling_params& sp = out.sampling[r];
      if (sp.temperature > 0.0f && !(sp.top_p > 0.0f)) fail(RB200_ERR_INVALID_ARGUMENT, "sampling: top_p must be positive");
      pick.truncated = pick.truncated || sampling_truncated(sp, c_.vocab);
    }
  // greedy with log-probabilities runs the sampling kernel with temperature 0 rows
  if (pick.kind == Pick::Greedy && pick.logprobs) pick.kind = Pick::Sample;
  return pick;
}

// Copies of the pass's results to the host, enqueued behind its kernels.
void Backend::fetch_outputs(const Outputs& out, int R, PickSpec pick) {
  if (R == 0) return;
  const size_t rows = static_cast<size_t>(R);
  if (pick.kind != Pick::None) {
    RB_CUDA(cudaMemcpyAsync(out.tokens, argmax_tok_.p, rows * 4, cudaMemcpyDeviceToHost, stream_));
    if (pick.kind == Pick::Greedy && out.greedy_logit)
      RB_CUDA(cudaMemcpyAsync(out.greedy_logit, argmax_val_.p, rows * 4, cudaMemcpyDeviceToHost, stream_));
    if (pick.logprobs) RB_CUDA(cudaMemcpyAsync(out.logprobs, logprob_.p, rows * 8, cudaMemcpyDeviceToHost, stream_));
  }
  if (out.logits) RB_CUDA(cudaMemcpyAsync(out.logits, logits_.p, rows * c_.vocab * 4, cudaMemcpyDeviceToHost, stream_));
}

int Backend::forward(int n_seqs, const int32_t* tokens, const int32_t* chunk_len, const int32_t* start_pos,
                     const int32_t* table_len, const int32_t* tables, const uint8_t* want_logits, bool all_logits,
                     rb200_layer_cb cb, void* cb_ctx, const Outputs& out) {
  set_device();  // the caller's current device may be another GPU (engine/src/cuda_backend.cu:505)
  RB_REQUIRE(n_seqs >= 0, "forward: negative sequence count");
  const int H = c_.hidden, D = c_.head_dim, Q = c_.heads * D, KV = c_.kv_heads * D, QKV = Q + 2 * KV, I = c_.intermediate;
  const int V = c_.vocab, bs = block_size_;

  // Pass 1: validate in the reference's order and size the metadata.
  long long T_ll = 0, table_ints = 0;
  {
    long long t = 0, tb = 0;
    for (int s = 0; s < n_seqs; ++s) {
      RB_REQUIRE(chunk_len[s] >= 0 && start_pos[s] >= 0 && table_len[s] >= 0, "forward: negative chunk field");
      const long long end = static_cast<long long>(start_pos[s]) + chunk_len[s];
      const long long need = (end + bs - 1) / bs;
      if (table_len[s] < need) fail(RB200_ERR_INVALID_ARGUMENT, "block table too short");
      if (end > max_context_) fail(RB200_ERR_INVALID_ARGUMENT, "sequence longer than max_context");
      for (int i = 0; i < chunk_len[s]; ++i)
        if (tokens[t + i] < 0 || tokens[t + i] >= V) fail(RB200_ERR_OUT_OF_RANGE, "token id out of range");
      for (long long i = 0; i < need; ++i)
        if (tables[tb + i] < 0 || tables[tb + i] >= num_blocks_) fail(RB200_ERR_INVALID_ARGUMENT, "block id out of range");
      t += chunk_len[s];
      tb += table_len[s];
      table_ints += (need + 3) / 4 * 4;  // each table starts 16-byte aligned on the device
    }
    T_ll = t;
  }
  if (T_ll == 0) return 0;
  if (T_ll > max_tokens_) fail(RB200_ERR_INVALID_ARGUMENT, "batch has more tokens than max_batch_tokens");
  const int T = static_cast<int>(T_ll);

  // Pass 2: flatten into one pinned buffer -> one host-to-device copy.
  // Layout (ints): tokens[T4] pos[T4] seq[T4] rows[T4] decode[T4] tiles[2 T4] table_off[S4] tables[...]
  // and, when the device samples, the rows' sampling parameters (8 ints each) behind the tables.
  const size_t S4 = static_cast<size_t>(round_up(n_seqs, 4));
  const size_t T4 = static_cast<size_t>(round_up(T, 4));
  const size_t sampling_off = T4 * 7 + S4 + static_cast<size_t>(table_ints);  // a multiple of 4 ints: 16-byte aligned
  static_assert(sizeof(rb200_sampling_params) == 32, "sampling parameters are 8 ints");
  const size_t total_ints = sampling_off + (out.tokens ? static_cast<size_t>(T) * 8 : 0);
  meta_host_.ensure(total_ints * 4);
  meta_dev_.ensure(total_ints * 4);
  int* hm = meta_host_.as<int>();
  int *h_tok = hm, *h_pos = hm + T4, *h_seq = hm + 2 * T4, *h_rows = hm + 3 * T4, *h_dec = hm + 4 * T4;
  int* h_tiles = hm + 5 * T4;
  int* h_toff = hm + 7 * T4;
  int* h_tables = h_toff + S4;
  int R = 0, n_decode = 0, n_tiles = 0, max_ctx = 0;
  {
    int t = 0;
    long long tb_in = 0, tb_out = 0;
    for (int s = 0; s < n_seqs; ++s) {
      const int n = chunk_len[s];
      const int end = start_pos[s] + n;
      const int need = (end + bs - 1) / bs;
      h_toff[s] = static_cast<int>(tb_out);
      std::memcpy(h_tables + tb_out, tables + tb_in, static_cast<size_t>(need) * 4);
      for (int i = need; i < (need + 3) / 4 * 4; ++i) h_tables[tb_out + i] = 0;
      tb_in += table_len[s];
      tb_out += (need + 3) / 4 * 4;
      for (int i = 0; i < n; ++i) {
        if (all_logits) h_rows[R++] = t + i;
        h_tok[t + i] = tokens[t + i];
        h_pos[t + i] = start_pos[s] + i;
        h_seq[t + i] = s;
      }
      if (!all_logits && n > 0 && (want_logits ? want_logits[s] != 0 : true)) h_rows[R++] = t + n - 1;
      // Single tokens go to the split-context decode kernel, longer chunks to the flash
      // prefill kernel in tiles of up to 64 rows (engine/src/cuda_backend.cu:528-545).
      if (n == 1) {
        h_dec[n_decode++] = t;
        max_ctx = std::max(max_ctx, end);
      } else {
        for (int r = 0; r < n; r += kPrefillRows) {
          h_tiles[2 * n_tiles] = t + r;
          h_tiles[2 * n_tiles + 1] = std::min(kPrefillRows, n - r);
          ++n_tiles;
        }
      }
      t += n;
    }
  }
  if (out.logits && static_cast<size_t>(R) * V > out.cap_floats) fail(RB200_ERR_INVALID_ARGUMENT, "logits buffer too small");
  if (out.tokens && static_cast<size_t>(R) > out.cap_rows) fail(RB200_ERR_INVALID_ARGUMENT, "token buffer too small");
  const PickSpec pick = pick_of(out, R);
  if (pick.kind == Pick::Sample) {
    auto* sp = reinterpret_cast<rb200_sampling_params*>(hm + sampling_off);
    for (int r = 0; r < R; ++r) sp[r] = out.sampling ? out.sampling[r] : rb200_sampling_params{0.0f, 1.0f, 0, 0, 0, 0};
  }

  RB_CUDA(cudaMemcpyAsync(meta_dev_.p, hm, total_ints * 4, cudaMemcpyHostToDevice, stream_));
  plan_ = Plan{T, R, n_decode, n_tiles, max_ctx, T4, S4, pick.kind == Pick::Sample ? sampling_off : 0};
  const AttnShape shape{c_.heads, c_.kv_heads, D, bs, QKV, Qp_, pool_rows()};
  if (fast_attention_ && n_decode > 0) decode_scratch_.ensure(decode_scratch_bytes(shape, n_decode, max_ctx));
  ensure_row_buffers(R, pick);
  (void)H; (void)I; (void)KV;

  Prof prof = begin_profile();
  enqueue(meta_dev_.as<int>(), plan_, cb, cb_ctx, pick, &prof);
  layer_events_stale_ = false;
  fetch_outputs(out, R, pick);
  // Steps of every size run tcgen05 kernels (the few-token linear layers too), so the word their
  // bounded pipeline waits leave a code in comes back with every pass, behind the results.
  result_host_.ensure(sizeof(int));
  RB_CUDA(cudaMemcpyAsync(result_host_.p, umma_status_word(), sizeof(int), cudaMemcpyDeviceToHost, stream_));
  RB_CUDA(cudaGetLastError());
  RB_CUDA(cudaStreamSynchronize(stream_));
  end_profile(prof);
  check_pipeline_status();
  return R;
}

// Reads the status word copied to result_host_ by the pass that just completed. A pass in which
// a wait gave up produced no valid output: it fails, and the word is cleared so that the next
// pass is judged on its own.
void Backend::check_pipeline_status() {
  const int code = *result_host_.as<int>();
  if (code == 0) return;
  umma_status_clear(stream_);
  RB_CUDA(cudaStreamSynchronize(stream_));
  fail(RB200_ERR_RUNTIME, "a tcgen05 pipeline wait timed out (code " + std::to_string(code) + ")");
}

// One forward pass's kernels, from metadata that is already on the device.
void Backend::ensure_row_buffers(int R, PickSpec pick) {
  if (R <= 0) return;
  logits_.ensure(static_cast<size_t>(R) * c_.vocab * 4);
  if (pick.kind != Pick::None) {
    argmax_tok_.ensure(static_cast<size_t>(R) * 4);
    argmax_val_.ensure(static_cast<size_t>(R) * 4);
  }
  if (pick.logprobs) logprob_.ensure(static_cast<size_t>(R) * 8);
}

void Backend::enqueue(const int* dm, const Plan& p, rb200_layer_cb cb, void* cb_ctx, PickSpec pick, Prof* prof,
                      bool layer_events) {
  const int H = c_.hidden, D = c_.head_dim, Q = c_.heads * D, KV = c_.kv_heads * D, QKV = Q + 2 * KV, I = c_.intermediate;
  const int V = c_.vocab, bs = block_size_, T = p.T, R = p.R;
  const size_t T4 = p.T4;
  const int *d_tok = dm, *d_pos = dm + T4, *d_seq = dm + 2 * T4, *d_rows = dm + 3 * T4, *d_dec = dm + 4 * T4;
  const int2* d_tiles = reinterpret_cast<const int2*>(dm + 5 * T4);
  const int* d_toff = dm + 7 * T4;
  const int* d_tables = d_toff + p.S4;
  const TokenMeta meta{d_pos, d_seq, d_toff, d_tables};
  const AttnShape shape{c_.heads, c_.kv_heads, D, bs, QKV, Qp_, pool_rows()};
  const float eps = static_cast<float>(c_.rms_eps);
  float* x = x_.as<float>();
  __half* xn = xn_.as<__half>();
  float* qkv = qkv_.as<float>();
  __half* attn = attn_.as<__half>();
  float* gu = gu_.as<float>();
  __half* act = act_.as<__half>();
  void* gs = gemv_scratch_.p;
  const size_t gsb = gemv_scratch_.bytes;
  (void)V;

  if (prof) mark(*prof, kMarkStart);
  launch_embed(d_tok, embed_.data.as<__half>(), x, T, H, embed_.ld, stream_);
  for (int l = 0; l < c_.layers; ++l) {
    Layer& L = layers_[l];
    __half* kc = kc_.as<__half>() + static_cast<size_t>(l) * layer_elems();
    __half* vc = vc_.as<__half>() + static_cast<size_t>(l) * layer_elems();
    // Where the projection behind a norm reads its input as int8 digits, the norm writes them.
    const I8Digits dq = H % 4 == 0 ? linear_digits_dest(L.wqkv.view(), xn, Hp_, T, gs, gsb) : I8Digits{};
    launch_rmsnorm(x, nullptr, L.attn_norm.as<float>(), xn, T, H, Hp_, eps, stream_, dq);
    launch_linear(L.wqkv.view(), xn, Hp_, qkv, T, 0.0f, gs, gsb, stream_, dq.digits != nullptr);
    launch_qkv_post(qkv, c_.qkv_bias ? L.bqkv.as<float>() : nullptr, inv_freq_.as<float>(), meta, T, kc, vc, c_.heads,
                    c_.kv_heads, D, bs, stream_);
    // This layer's K and V are enqueued; a transfer thread may wait on the event and read
    // them while later layers run (engine/src/cuda_backend.cu:580-581).
    if (layer_events) RB_CUDA(cudaEventRecord(layer_done_[l], stream_));
    if (cb) cb(cb_ctx, l);
    if (fast_attention_) {
      if (p.n_tiles > 0) {
        if (prof) mark(*prof, kMarkPrefillBegin);
        launch_prefill_attention(shape, qkv, meta, d_tiles, p.n_tiles, kc, vc, attn, stream_);
        if (prof) mark(*prof, kMarkPrefillEnd);
      }
      if (p.n_decode > 0) {
        if (prof) mark(*prof, kMarkDecodeBegin);
        launch_decode_attention(shape, qkv, meta, d_dec, p.n_decode, p.max_ctx, kc, vc, decode_scratch_.as<float>(), attn,
                                stream_);
        if (prof) mark(*prof, kMarkDecodeEnd);
      }
    } else {
      launch_reference_attention(shape, qkv, meta, T, kc, vc, attn, stream_);
    }
    launch_linear(L.wo.view(), attn, Qp_, x, T, 1.0f, gs, gsb, stream_);  // x += attn wo^T
    const I8Digits dm = H % 4 == 0 ? linear_digits_dest(L.w_gate_up.view(), xn, Hp_, T, gs, gsb) : I8Digits{};
    launch_rmsnorm(x, nullptr, L.mlp_norm.as<float>(), xn, T, H, Hp_, eps, stream_, dm);
    launch_linear(L.w_gate_up.view(), xn, Hp_, gu, T, 0.0f, gs, gsb, stream_, dm.digits != nullptr);
    // SwiGLU writes the digits the down projection reads, where it reads digits
    const I8Digits dd = (I % 4 == 0 && Ip_ % 32 == 0) ? linear_digits_dest(L.w_down.view(), act, Ip_, T, gs, gsb) : I8Digits{};
    launch_silu_mul(gu, act, T, I, Ip_, stream_, dd);
    launch_linear(L.w_down.view(), act, Ip_, x, T, 1.0f, gs, gsb, stream_, dd.digits != nullptr);  // x += act w_down^T
  }
  if (R > 0) {
    launch_rmsnorm(x, d_rows, final_norm_.as<float>(), xn, R, H, Hp_, eps, stream_);
    const Matrix& head = c_.tie_embeddings ? embed_ : lm_head_;
    launch_linear(head.view(), xn, Hp_, logits_.as<float>(), R, 0.0f, gs, gsb, stream_);
    if (pick.kind == Pick::Greedy)
      launch_argmax_rows(logits_.as<float>(), R, c_.vocab, argmax_tok_.as<int>(), argmax_val_.as<float>(), stream_);
    else if (pick.kind == Pick::Sample)
      launch_sample_rows(logits_.as<float>(), R, c_.vocab, reinterpret_cast<const rb200_sampling_params*>(dm + p.sampling_off),
                         argmax_tok_.as<int>(), pick.logprobs ? logprob_.as<double>() : nullptr, stream_, pick.truncated);
  }
  if (prof) mark(*prof, kMarkEnd);
  RB_CUDA(cudaGetLastError());
}

// ---- measurement support --------------------------------------------------------------------

Backend::Prof Backend::begin_profile() {
  Prof p;
  p.on = profiling_;
  p.first = 0;
  p.n = 0;
  return p;
}

void Backend::mark(Prof& p, int kind) {
  if (!p.on) return;
  if (static_cast<size_t>(p.n) >= prof_events_.size()) {
    const size_t old = prof_events_.size();
    prof_events_.resize(old + 256);
    for (size_t i = old; i < prof_events_.size(); ++i) RB_CUDA(cudaEventCreate(&prof_events_[i]));
    prof_kinds_.resize(prof_events_.size());
  }
  RB_CUDA(cudaEventRecord(prof_events_[p.n], stream_));
  prof_kinds_[p.n] = kind;
  ++p.n;
}

void Backend::end_profile(Prof& p) {
  if (!p.on || p.n < 2) return;
  float ms = 0.f;
  for (int i = 0; i + 1 < p.n; ++i) {
    const int a = prof_kinds_[i], b = prof_kinds_[i + 1];
    if (a == kMarkDecodeBegin && b == kMarkDecodeEnd) {
      RB_CUDA(cudaEventElapsedTime(&ms, prof_events_[i], prof_events_[i + 1]));
      profile_.decode_attn_ms += ms;
      profile_.decode_attn_calls += 1;
    } else if (a == kMarkPrefillBegin && b == kMarkPrefillEnd) {
      RB_CUDA(cudaEventElapsedTime(&ms, prof_events_[i], prof_events_[i + 1]));
      profile_.prefill_attn_ms += ms;
      profile_.prefill_attn_calls += 1;
    }
  }
  RB_CUDA(cudaEventElapsedTime(&ms, prof_events_[0], prof_events_[p.n - 1]));
  profile_.total_ms += ms;
  profile_.forwards += 1;
}

void Backend::set_profiling(bool on) { profiling_ = on; }

rb200_profile Backend::take_profile() {
  rb200_profile out = profile_;
  profile_ = rb200_profile{};
  return out;
}

float Backend::replay(int iters) {
  set_device();
  RB_REQUIRE(plan_.T > 0, "forward_replay: no forward pass to replay");
  RB_REQUIRE(iters > 0, "forward_replay: iters must be positive");
  cudaEvent_t a, b;
  RB_CUDA(cudaEventCreate(&a));
  RB_CUDA(cudaEventCreate(&b));
  float total = 0.f;
  try {
    RB_CUDA(cudaEventRecord(a, stream_));
    for (int i = 0; i < iters; ++i) {
      Prof prof = begin_profile();
      PickSpec pick;
      if ((flags_ & RB200_GPU_ARGMAX) != 0 && argmax_tok_.bytes >= static_cast<size_t>(plan_.R) * 4) pick.kind = Pick::Greedy;
      enqueue(meta_dev_.as<int>(), plan_, nullptr, nullptr, pick, &prof);
      if (prof.on) {  // per-pass marks are read back before the next pass reuses the events
        RB_CUDA(cudaStreamSynchronize(stream_));
        end_profile(prof);
      }
    }
    RB_CUDA(cudaEventRecord(b, stream_));
    result_host_.ensure(sizeof(int));
    RB_CUDA(cudaMemcpyAsync(result_host_.p, umma_status_word(), sizeof(int), cudaMemcpyDeviceToHost, stream_));
    RB_CUDA(cudaStreamSynchronize(stream_));
    check_pipeline_status();
    RB_CUDA(cudaEventElapsedTime(&total, a, b));
  } catch (...) {
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    throw;
  }
  cudaEventDestroy(a);
  cudaEventDestroy(b);
  return total;
}

namespace {
// Counter-based N(0,1): two rounds of a 64-bit mix per pair, Box-Muller.
__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  return z ^ (z >> 31);
}
__global__ void fill_normal_f16_kernel(__half2* out, size_t n_pairs, unsigned long long seed) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n_pairs;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const unsigned long long r = mix64(seed + 0x9E3779B97F4A7C15ULL * (i + 1));
    const float u1 = (static_cast<float>(r >> 40) + 1.0f) * (1.0f / 16777216.0f);          // (0, 1]
    const float u2 = static_cast<float>((r >> 8) & 0xFFFFFF) * (1.0f / 16777216.0f);      // [0, 1)
    const float rad = sqrtf(-2.0f * __logf(u1));
    float sn, cs;
    __sincosf(6.283185307179586f * u2, &sn, &cs);
    out[i] = __floats2half2_rn(rad * cs, rad * sn);
  }
}
}  // namespace

void Backend::debug_fill_kv(unsigned long long seed) {
  set_device();
  const size_t pairs = static_cast<size_t>(layer_elems()) * c_.layers / 2;
  count_launch();
  fill_normal_f16_kernel<<<sm_count() * 8, 256, 0, stream_>>>(kc_.as<__half2>(), pairs, seed);
  count_launch();
  fill_normal_f16_kernel<<<sm_count() * 8, 256, 0, stream_>>>(vc_.as<__half2>(), pairs, seed ^ 0x5555555555555555ULL);
  RB_CUDA(cudaGetLastError());
  RB_CUDA(cudaStreamSynchronize(stream_));
}

// ---- KV block I/O (engine/src/cuda_backend.cu:611-664) --------------------------------------

void Backend::check_layer(int layer) const {
  RB_REQUIRE(layer >= 0 && layer < c_.layers, "no such layer");
}

void Backend::check_blocks(const int32_t* blocks, int n) const {
  RB_REQUIRE(n >= 0, "negative block count");
  for (int i = 0; i < n; ++i) RB_REQUIRE(blocks[i] >= 0 && blocks[i] < num_blocks_, "block id out of range");
}

void Backend::ensure_kv_staging(size_t n_blocks) {
  const size_t bytes = 2 * n_blocks * kv_block_bytes();
  kv_staging_.ensure(bytes);  // a regrow frees the old buffer, which waits for work still using it
  kv_pinned_.ensure(bytes);
  kv_ids_.ensure(n_blocks * sizeof(int));
}

void* Backend::staging_ids(const int32_t* blocks, int n) {
  if (id_slots_.empty()) {
    id_slots_.resize(16);
    for (IdSlot& s : id_slots_) RB_CUDA(cudaEventCreateWithFlags(&s.uploaded, cudaEventDisableTiming));
  }
  IdSlot& slot = id_slots_[id_next_];
  id_next_ = (id_next_ + 1) % static_cast<int>(id_slots_.size());
  if (slot.used) RB_CUDA(cudaEventSynchronize(slot.uploaded));
  slot.buf.ensure(static_cast<size_t>(n) * sizeof(int));
  std::memcpy(slot.buf.p, blocks, static_cast<size_t>(n) * sizeof(int));
  RB_CUDA(cudaMemcpyAsync(kv_ids_.p, slot.buf.p, static_cast<size_t>(n) * sizeof(int), cudaMemcpyHostToDevice, copy_stream_));
  RB_CUDA(cudaEventRecord(slot.uploaded, copy_stream_));
  slot.used = true;
  return kv_ids_.p;
}

void Backend::read_kv_layer(int layer, const int32_t* blocks, int n, void* k_out, void* v_out) {
  set_device();
  check_layer(layer);
  check_blocks(blocks, n);
  if (n == 0) return;
  std::lock_guard<std::mutex> lock(copy_mu_);
  const size_t bb = kv_block_bytes();
  ensure_kv_staging(n);
  const int* ids = static_cast<const int*>(staging_ids(blocks, n));
  const size_t off = static_cast<size_t>(layer) * layer_elems();
  launch_kv_gather(kc_.as<__half>() + off, vc_.as<__half>() + off, ids, n, bb, kv_staging_.p, copy_stream_);
  RB_CUDA(cudaGetLastError());
  RB_CUDA(cudaMemcpyAsync(kv_pinned_.p, kv_staging_.p, 2 * n * bb, cudaMemcpyDeviceToHost, copy_stream_));
  RB_CUDA(cudaStreamSynchronize(copy_stream_));
  std::memcpy(k_out, kv_pinned_.p, n * bb);
  std::memcpy(v_out, kv_pinned_.as<char>() + n * bb, n * bb);
}

void Backend::write_kv_layer(int layer, const int32_t* blocks, int n, const void* k_in, const void* v_in) {
  set_device();
  check_layer(layer);
  check_blocks(blocks, n);
  if (n == 0) return;
  std::lock_guard<std::mutex> lock(copy_mu_);
  const size_t bb = kv_block_bytes();
  ensure_kv_staging(n);
  std::memcpy(kv_pinned_.p, k_in, n * bb);
  std::memcpy(kv_pinned_.as<char>() + n * bb, v_in, n * bb);
  const int* ids = static_cast<const int*>(staging_ids(blocks, n));
  RB_CUDA(cudaMemcpyAsync(kv_staging_.p, kv_pinned_.p, 2 * n * bb, cudaMemcpyHostToDevice, copy_stream_));
  const size_t off = static_cast<size_t>(layer) * layer_elems();
  launch_kv_scatter(kc_.as<__half>() + off, vc_.as<__half>() + off, ids, n, bb, kv_staging_.p, copy_stream_);
  RB_CUDA(cudaGetLastError());
  RB_CUDA(cudaStreamSynchronize(copy_stream_));
}

void Backend::wait_kv_written(int layer) {
  check_layer(layer);
  // A pass replayed as a CUDA graph records no per-layer events: wait for the whole pass.
  if (layer_events_stale_ && pass_done_) RB_CUDA(cudaEventSynchronize(pass_done_));
  else RB_CUDA(cudaEventSynchronize(layer_done_[layer]));
}

// ---- weight update (engine/src/cuda_backend.cu:429-477) -------------------------------------

void Backend::update_weight(const std::string& name, const float* src, size_t n) {
  set_device();
  RB_REQUIRE(src != nullptr, "update_weight: null source");
  auto check = [&](size_t want) {
    if (n != want) fail(RB200_ERR_INVALID_ARGUMENT, "update_weight " + name + ": wrong size");
  };
  auto matrix = [&](Matrix& m) {
    check(static_cast<size_t>(m.N) * m.K);
    upload_matrix(m, src, m.N, m.K);
  };
  auto vector = [&](DeviceBuf& d) {
    check(d.bytes / 4);
    upload_vector(d, src, n);
  };
  if (name == "embed") {
    matrix(embed_);
  } else if (name == "lm_head") {
    if (c_.tie_embeddings) fail(RB200_ERR_INVALID_ARGUMENT, "update_weight: tied embeddings have no lm_head");
    matrix(lm_head_);
  } else if (name == "final_norm") {
    vector(final_norm_);
  } else if (name.rfind("layers.", 0) == 0) {
    const size_t dot = name.find('.', 7);
    int i = -1;
    if (dot != std::string::npos && dot > 7) {
      char* end = nullptr;
      const std::string num = name.substr(7, dot - 7);
      const long v = std::strtol(num.c_str(), &end, 10);
      if (end && *end == '\0') i = static_cast<int>(v);
    }
    if (i < 0 || i >= static_cast<int>(layers_.size())) fail(RB200_ERR_INVALID_ARGUMENT, "update_weight: no " + name);
    Layer& L = layers_[i];
    const std::string f = name.substr(dot + 1);
    if (f == "attn_norm") vector(L.attn_norm);
    else if (f == "mlp_norm") vector(L.mlp_norm);
    else if (f == "bqkv" && L.bqkv.bytes) vector(L.bqkv);
    else if (f == "wqkv") matrix(L.wqkv);
    else if (f == "wo") matrix(L.wo);
    else if (f == "w_gate_up") matrix(L.w_gate_up);
    else if (f == "w_down") matrix(L.w_down);
    else fail(RB200_ERR_INVALID_ARGUMENT, "update_weight: no " + name);
  } else {
    fail(RB200_ERR_INVALID_ARGUMENT, "update_weight: no " + name);
  }
}

}  // namespace rb200

// ---- C boundary -------------------------------------------------------------------------------

using namespace rb200;

struct rb200_backend {
  std::unique_ptr<Backend> impl;
};

extern "C" {

const char* rb200_last_error(void) { return g_error.c_str(); }
int rb200_last_error_kind(void) { return g_error_kind; }

int rb200_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

uint32_t rb200_flags_from_env(void) {
  uint32_t f = 0;
  if (const char* a = std::getenv("RELAY_CUDA_ATTENTION")) f |= std::string(a) == "m0" ? RB200_REFERENCE_ATTENTION : 0;
  if (const char* q = std::getenv("RELAY_CUDA_INT8")) f |= std::string(q) == "1" ? RB200_INT8_WEIGHTS : 0;
  return f;
}

int rb200_rope_inv_freq(const rb200_model_config* cfg, float* out) {
  return guarded([&] {
    RB_REQUIRE(cfg && out && cfg->head_dim > 0 && cfg->head_dim % 2 == 0, "rope_inv_freq: bad config");
    std::vector<float> inv;
    rope_inv_freq(*cfg, inv);
    std::memcpy(out, inv.data(), inv.size() * 4);
    return static_cast<int>(inv.size());
  });
}

int rb200_quantize_rows_int8(const float* w, int N, int K, int8_t* q_out, float* scale_out) {
  return guarded([&] {
    RB_REQUIRE(w && q_out && scale_out && N >= 0 && K > 0, "quantize_rows_int8: bad arguments");
    for (int n = 0; n < N; ++n) {
      const float* row = w + static_cast<size_t>(n) * K;
      float mx = 0.0f;
      for (int k = 0; k < K; ++k) mx = std::max(mx, std::fabs(row[k]));
      const float sc = mx > 0.0f ? mx / 127.0f : 1.0f;
      scale_out[n] = sc;
      for (int k = 0; k < K; ++k) q_out[static_cast<size_t>(n) * K + k] = static_cast<int8_t>(std::lrintf(row[k] / sc));
    }
    return 0;
  });
}

rb200_backend* rb200_create(const rb200_model_config* cfg, const rb200_weights* weights, int num_blocks, int block_size,
                            int device, int max_batch_tokens, int max_context, uint32_t flags) {
  rb200_backend* h = nullptr;
  const int rc = guarded([&] {
    RB_REQUIRE(cfg != nullptr, "create: null config");
    auto b = std::make_unique<rb200_backend>();
    b->impl = std::make_unique<Backend>(*cfg, weights, num_blocks, block_size, device, max_batch_tokens, max_context, flags);
    h = b.release();
    return 0;
  });
  return rc == 0 ? h : nullptr;
}

void rb200_destroy(rb200_backend* b) { delete b; }

const char* rb200_name(const rb200_backend*) { return "b200"; }

int rb200_get_config(const rb200_backend* b, rb200_model_config* out) {
  return guarded([&] {
    RB_REQUIRE(b && out, "get_config: null argument");
    *out = b->impl->config();
    return 0;
  });
}

int rb200_get_kv_layout(const rb200_backend* b, int32_t out[5]) {
  return guarded([&] {
    RB_REQUIRE(b && out, "get_kv_layout: null argument");
    const rb200_model_config& c = b->impl->config();
    out[0] = c.layers;
    out[1] = c.kv_heads;
    out[2] = c.head_dim;
    out[3] = b->impl->block_size();
    out[4] = b->impl->num_blocks();
    return 0;
  });
}

int rb200_forward(rb200_backend* b, int n_seqs, const int32_t* tokens, const int32_t* chunk_len, const int32_t* start_pos,
                  const int32_t* table_len, const int32_t* tables, const uint8_t* want_logits, int all_logits,
                  rb200_layer_cb cb, void* cb_ctx, float* logits_out, size_t cap_floats) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr, "forward: null backend");
    Backend::Outputs out;
    out.logits = logits_out;
    out.cap_floats = cap_floats;
    return b->impl->forward(n_seqs, tokens, chunk_len, start_pos, table_len, tables, want_logits, all_logits != 0, cb,
                            cb_ctx, out);
  });
}

int rb200_forward_greedy(rb200_backend* b, int n_seqs, const int32_t* tokens, const int32_t* chunk_len,
                         const int32_t* start_pos, const int32_t* table_len, const int32_t* tables,
                         const uint8_t* want_logits, int all_logits, rb200_layer_cb cb, void* cb_ctx, int32_t* token_out,
                         float* logit_out, size_t cap_rows) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr && token_out != nullptr, "forward_greedy: null argument");
    Backend::Outputs out;
    out.tokens = token_out;
    out.greedy_logit = logit_out;
    out.cap_rows = cap_rows;
    return b->impl->forward(n_seqs, tokens, chunk_len, start_pos, table_len, tables, want_logits, all_logits != 0, cb,
                            cb_ctx, out);
  });
}

int rb200_forward_sample(rb200_backend* b, int n_seqs, const int32_t* tokens, const int32_t* chunk_len,
                         const int32_t* start_pos, const int32_t* table_len, const int32_t* tables,
                         const uint8_t* want_logits, int all_logits, rb200_layer_cb cb, void* cb_ctx,
                         const rb200_sampling_params* sampling, int32_t* token_out, double* logprob_out, size_t cap_rows) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr && token_out != nullptr && sampling != nullptr, "forward_sample: null argument");
    Backend::Outputs out;
    out.tokens = token_out;
    out.sampling = sampling;
    out.logprobs = logprob_out;
    out.cap_rows = cap_rows;
    return b->impl->forward(n_seqs, tokens, chunk_len, start_pos, table_len, tables, want_logits, all_logits != 0, cb,
                            cb_ctx, out);
  });
}

int rb200_decode_open(rb200_backend* b, int n_seqs, const int32_t* context_len, const int32_t* table_len,
                      const int32_t* tables) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr, "decode_open: null backend");
    b->impl->decode_open(n_seqs, context_len, table_len, tables);
    return 0;
  });
}

int rb200_decode_set_slot(rb200_backend* b, int slot, int context_len, int table_len, const int32_t* table) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr, "decode_set_slot: null backend");
    b->impl->decode_set_slot(slot, context_len, table_len, table);
    return 0;
  });
}

int rb200_decode_step(rb200_backend* b, const int32_t* tokens, int n_new_blocks, const int32_t* new_block_seq,
                      const int32_t* new_block_id, const rb200_sampling_params* sampling, int32_t* token_out,
                      double* logprob_out, float* logits_out, size_t cap_floats) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr, "decode_step: null backend");
    Backend::Outputs out;
    out.tokens = token_out;
    out.sampling = sampling;
    out.logprobs = logprob_out;
    out.logits = logits_out;
    out.cap_floats = cap_floats;
    return b->impl->decode_step(tokens, n_new_blocks, new_block_seq, new_block_id, out);
  });
}

int rb200_decode_close(rb200_backend* b) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr, "decode_close: null backend");
    b->impl->decode_close();
    return 0;
  });
}

size_t rb200_kv_block_bytes(const rb200_backend* b) { return b ? b->impl->kv_block_bytes() : 0; }

int rb200_read_kv_layer(rb200_backend* b, int layer, const int32_t* blocks, int n, void* k_out, void* v_out) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr, "read_kv_layer: null backend");
    b->impl->read_kv_layer(layer, blocks, n, k_out, v_out);
    return 0;
  });
}

int rb200_write_kv_layer(rb200_backend* b, int layer, const int32_t* blocks, int n, const void* k_in, const void* v_in) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr, "write_kv_layer: null backend");
    b->impl->write_kv_layer(layer, blocks, n, k_in, v_in);
    return 0;
  });
}

int rb200_wait_kv_written(rb200_backend* b, int layer) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr, "wait_kv_written: null backend");
    b->impl->wait_kv_written(layer);
    return 0;
  });
}

int rb200_update_weight(rb200_backend* b, const char* name, const float* src, size_t n) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr && name != nullptr, "update_weight: null argument");
    b->impl->update_weight(name, src, n);
    return 0;
  });
}

int rb200_set_profiling(rb200_backend* b, int on) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr, "set_profiling: null backend");
    b->impl->set_profiling(on != 0);
    return 0;
  });
}

int rb200_get_profile(rb200_backend* b, rb200_profile* out) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr && out != nullptr, "get_profile: null argument");
    *out = b->impl->take_profile();
    return 0;
  });
}

int rb200_forward_replay(rb200_backend* b, int iters, float* ms_out) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr && ms_out != nullptr, "forward_replay: null argument");
    *ms_out = b->impl->replay(iters);
    return 0;
  });
}

int rb200_debug_fill_kv(rb200_backend* b, uint64_t seed) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr, "debug_fill_kv: null backend");
    b->impl->debug_fill_kv(seed);
    return 0;
  });
}

uint64_t rb200_kernel_launches(void) { return rb200::launch_counter().load(); }

int rb200_nccl_init(rb200_backend* b, const void* id, int nranks, int rank) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr && id != nullptr, "nccl_init: null argument");
    b->impl->nccl_init(id, nranks, rank);
    return 0;
  });
}

int rb200_nccl_finalize(rb200_backend* b) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr, "nccl_finalize: null backend");
    b->impl->nccl_finalize();
    return 0;
  });
}

int rb200_send_kv_layer(rb200_backend* b, int peer, int layer, const int32_t* blocks, int n) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr, "send_kv_layer: null backend");
    b->impl->send_kv_layer(peer, layer, blocks, n);
    return 0;
  });
}

int rb200_recv_kv_layer(rb200_backend* b, int peer, int layer, const int32_t* blocks, int n) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr, "recv_kv_layer: null backend");
    b->impl->recv_kv_layer(peer, layer, blocks, n);
    return 0;
  });
}

int rb200_kv_link_create(rb200_backend* b, int n_slots, size_t slot_bytes, void* handle_out) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr, "kv_link_create: null backend");
    return b->impl->kv_link_create(n_slots, slot_bytes, handle_out);
  });
}

int rb200_kv_link_connect(rb200_backend* b, int link, const void* peer_handle) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr, "kv_link_connect: null backend");
    b->impl->kv_link_connect(link, peer_handle);
    return 0;
  });
}

int rb200_kv_link_send_layer(rb200_backend* b, int link, int layer, const int32_t* blocks, int n) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr, "kv_link_send_layer: null backend");
    b->impl->kv_link_send_layer(link, layer, blocks, n);
    return 0;
  });
}

int rb200_kv_link_recv_layer(rb200_backend* b, int link, int layer, const int32_t* blocks, int n) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr, "kv_link_recv_layer: null backend");
    b->impl->kv_link_recv_layer(link, layer, blocks, n);
    return 0;
  });
}

int rb200_kv_link_send_layers(rb200_backend* b, int link, int first_layer, int n_layers, const int32_t* blocks, int n) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr, "kv_link_send_layers: null backend");
    b->impl->kv_link_send_layers(link, first_layer, n_layers, blocks, n);
    return 0;
  });
}

int rb200_kv_link_recv_layers(rb200_backend* b, int link, int first_layer, int n_layers, const int32_t* blocks, int n) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr, "kv_link_recv_layers: null backend");
    b->impl->kv_link_recv_layers(link, first_layer, n_layers, blocks, n);
    return 0;
  });
}

int rb200_kv_link_skip_layers(rb200_backend* b, int link, int n_layers, int n) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr, "kv_link_skip_layers: null backend");
    b->impl->kv_link_skip_layers(link, n_layers, n);
    return 0;
  });
}

int rb200_kv_link_connect_local(rb200_backend* a, int link_a, rb200_backend* b, int link_b) {
  return guarded([&] {
    RB_REQUIRE(a != nullptr && b != nullptr, "kv_link_connect_local: null backend");
    a->impl->kv_link_connect_local(link_a, *b->impl, link_b);
    return 0;
  });
}

int rb200_kv_link_skip_layer(rb200_backend* b, int link, int n) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr, "kv_link_skip_layer: null backend");
    b->impl->kv_link_skip_layer(link, n);
    return 0;
  });
}

int rb200_kv_link_wait(rb200_backend* b, int link, int timeout_ms) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr, "kv_link_wait: null backend");
    b->impl->kv_link_wait(link, timeout_ms);
    return 0;
  });
}

int rb200_kv_link_wait_gathered(rb200_backend* b, int link, int timeout_ms) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr, "kv_link_wait_gathered: null backend");
    b->impl->kv_link_wait_gathered(link, timeout_ms);
    return 0;
  });
}

int rb200_kv_link_close(rb200_backend* b, int link) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr, "kv_link_close: null backend");
    b->impl->kv_link_close(link);
    return 0;
  });
}

int rb200_kv_hop_sync(rb200_backend* b, int timeout_ms) {
  return guarded([&] {
    RB_REQUIRE(b != nullptr, "kv_hop_sync: null backend");
    b->impl->kv_hop_sync(timeout_ms);
    return 0;
  });
}

}  // extern "C"
