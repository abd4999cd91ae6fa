// The backend object behind the rb200_* handle: device weights, the paged KV pools, the
// activation buffers and the two streams, with the same responsibilities and threading
// rules as the reference's CudaBackend (engine/src/cuda_backend.cu:311-759): forward() is
// called by one thread at a time; KV layer reads/writes may come from other threads at any
// time and run on their own stream under copy_mu_.
#pragma once

#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "kernels.h"

namespace rb200 {

// Device memory with RAII; zero-filled on allocation when asked.
// Set when a stream of this process is left behind a wait nobody will satisfy (a K/V link whose
// release did not get through): from then on nothing that synchronises the whole device may be
// called, so buffers are abandoned instead of freed and destructors skip their device-wide sync.
extern std::atomic<bool> g_device_wedged;

struct DeviceBuf {
  void* p = nullptr;
  size_t bytes = 0;
  DeviceBuf() = default;
  explicit DeviceBuf(size_t n, bool zero = false);
  ~DeviceBuf();
  DeviceBuf(DeviceBuf&& o) noexcept : p(o.p), bytes(o.bytes) { o.p = nullptr; o.bytes = 0; }
  DeviceBuf& operator=(DeviceBuf&& o) noexcept;
  DeviceBuf(const DeviceBuf&) = delete;
  DeviceBuf& operator=(const DeviceBuf&) = delete;
  template <class T>
  T* as() const { return static_cast<T*>(p); }
  void ensure(size_t n);  // regrow (contents lost) when smaller than n
};

struct PinnedBuf {
  void* p = nullptr;
  size_t bytes = 0;
  ~PinnedBuf();
  void ensure(size_t n);
  template <class T>
  T* as() const { return static_cast<T*>(p); }
};

// A weight matrix [N][ld]: fp16, or int8 + per-row scale. Columns K..ld-1 are zero.
struct Matrix {
  int N = 0, K = 0, ld = 0;
  bool int8 = false;
  DeviceBuf data, scale;
  WeightView view() const;
};

struct Layer {
  DeviceBuf attn_norm, mlp_norm, bqkv;
  Matrix wqkv, wo, w_gate_up, w_down;
};

// The NCCL communicator of the KV hop (an ncclComm_t, kept opaque here).
struct NcclState {
  void* comm = nullptr;
  int nranks = 0, rank = -1;
};

// One end of a K/V link (kv_link.cu): this end's region (a ring of landing slots with two
// counters each), the peer's region mapped through CUDA IPC, and the streams the link's work runs on.
struct KvLink {
  int n_slots = 0;
  size_t slot_bytes = 0;
  DeviceBuf region;
  void* peer = nullptr;
  bool peer_is_ipc = false;  // mapped with cudaIpcOpenMemHandle (another process) rather than taken by address
  static constexpr int kStreams = 2;       // consecutive messages alternate between them (four measured no faster)
  cudaStream_t streams[kStreams] = {};
  cudaEvent_t gathered[kStreams] = {};     // behind the latest gather on each stream
  // cudaErrorNotReady while any stream (or, gathers_only, any gather) still has work; errors pass through
  cudaError_t busy(bool gathers_only = false) const;
  cudaStream_t release_stream = nullptr;          // carries nothing but the host's release of this end's counters
  PinnedBuf release_words;                        // what that release writes (filled when the link is created)
  uint32_t sent = 0, received = 0;  // messages enqueued so far in each direction
  bool broken = false;
  bool wedged = false;  // still busy after a release: its region is abandoned, not freed
  ~KvLink();
};

struct DecodeSession {
  int S = 0;    // slots
  int cap = 0;  // block-table entries per slot (a multiple of 4: tables stay 16-byte aligned)
  size_t T4 = 0, S4 = 0;
  std::vector<int> ctx, tlen;  // host mirror: keys in the cache and table entries in use, per slot
  // forward()'s metadata layout with tables `cap` apart, then the per-step delta:
  //   header[4] = {new blocks, 1 if the device feeds its own tokens, 0, 0}
  //   tokens[S4], (slot, table index, block id)[S] padded to 4 ints, sampling parameters[S]
  DeviceBuf meta;
  PinnedBuf delta_host;
  size_t delta_off = 0, tokens_off = 0, blocks_off = 0, sampling_off = 0, delta_ints = 0;  // in ints from meta
  bool have_picked = false;  // the previous step left one picked token per slot on the device
  // captured steps by launch geometry; `seen` holds geometries that have run once uncaptured
  std::map<uint64_t, cudaGraphExec_t> graphs;
  std::map<uint64_t, int> seen;
  uintptr_t buffers_sig = 0;
  ~DecodeSession() {
    for (auto& g : graphs) cudaGraphExecDestroy(g.second);
  }
};

class Backend {
 public:
  Backend(const rb200_model_config& cfg, const rb200_weights* w, int num_blocks, int block_size, int device,
          int max_batch_tokens, int max_context, uint32_t flags);
  ~Backend();

  const rb200_model_config& config() const { return c_; }
  int num_blocks() const { return num_blocks_; }
  int block_size() const { return block_size_; }
  size_t kv_block_bytes() const { return static_cast<size_t>(c_.kv_heads) * block_size_ * c_.head_dim * 2; }
  long long pool_rows() const { return static_cast<long long>(num_blocks_) * c_.kv_heads * block_size_; }
  long long layer_elems() const { return static_cast<long long>(c_.kv_heads) * block_size_ * c_.head_dim * num_blocks_; }

  // What a pass hands back to the host, per logits row: the float32 logits, or the token the
  // device picked (greedy with its logit, or sampled per `sampling` with its log-probability).
  struct Outputs {
    float* logits = nullptr;
    size_t cap_floats = 0;
    int32_t* tokens = nullptr;
    float* greedy_logit = nullptr;
    const rb200_sampling_params* sampling = nullptr;  // host, one per logits row; null: greedy
    double* logprobs = nullptr;
    size_t cap_rows = 0;
  };
  // Returns the number of logit rows.
  int forward(int n_seqs, const int32_t* tokens, const int32_t* chunk_len, const int32_t* start_pos,
              const int32_t* table_len, const int32_t* tables, const uint8_t* want_logits, bool all_logits,
              rb200_layer_cb cb, void* cb_ctx, const Outputs& out);

  // Decode session: a batch of single-token sequences whose positions and block tables stay on
  // the device between steps (session.cu).
  void decode_open(int n_seqs, const int32_t* context_len, const int32_t* table_len, const int32_t* tables);
  void decode_set_slot(int slot, int context_len, int table_len, const int32_t* table);
  int decode_step(const int32_t* tokens, int n_new_blocks, const int32_t* new_block_seq, const int32_t* new_block_id,
                  const Outputs& out);
  void decode_close();

  void read_kv_layer(int layer, const int32_t* blocks, int n, void* k_out, void* v_out);
  void write_kv_layer(int layer, const int32_t* blocks, int n, const void* k_in, const void* v_in);
  void wait_kv_written(int layer);
  void update_weight(const std::string& name, const float* src, size_t n);

  // measurement support
  void set_profiling(bool on);
  rb200_profile take_profile();
  float replay(int iters);  // re-enqueues the last forward pass's kernels; returns device milliseconds
  void debug_fill_kv(unsigned long long seed);

  // kv_hop.cu
  void nccl_init(const void* id, int nranks, int rank);
  void nccl_finalize();
  void send_kv_layer(int peer, int layer, const int32_t* blocks, int n);
  void recv_kv_layer(int peer, int layer, const int32_t* blocks, int n);
  void kv_hop_sync(int timeout_ms);
  void nccl_finalize_noexcept() noexcept;

  // kv_link.cu
  int kv_link_create(int n_slots, size_t slot_bytes, void* handle_out);
  void kv_link_connect(int link, const void* peer_handle);
  void kv_link_send_layers(int link, int layer0, int n_layers, const int32_t* blocks, int n);
  void kv_link_recv_layers(int link, int layer0, int n_layers, const int32_t* blocks, int n);
  void kv_link_send_layer(int link, int layer, const int32_t* blocks, int n) { kv_link_send_layers(link, layer, 1, blocks, n); }
  void kv_link_recv_layer(int link, int layer, const int32_t* blocks, int n) { kv_link_recv_layers(link, layer, 1, blocks, n); }
  void kv_link_connect_local(int link, Backend& other, int other_link);
  void kv_link_skip_layers(int link, int n_layers, int n);
  void kv_link_skip_layer(int link, int n) { kv_link_skip_layers(link, 1, n); }
  void kv_link_wait(int link, int timeout_ms);
  void kv_link_wait_gathered(int link, int timeout_ms);
  void kv_link_close(int link);

 private:
  void set_device() const;
  void check_layer(int layer) const;
  void check_blocks(const int32_t* blocks, int n) const;
  void upload_matrix(Matrix& m, const float* src_any, int N, int K);
  void upload_vector(DeviceBuf& dst, const float* src_any, size_t n);
  Matrix make_matrix(int N, int K, bool int8);
  // Feeds src (host, or device memory of any GPU) to apply(dev_ptr, first_row, rows) as
  // float32 rows resident on this device, staging through stage_ when it is not local.
  template <class F>
  void for_row_chunks(const float* src, int rows, int cols, F&& apply);
  void* staging_ids(const int32_t* blocks, int n);  // under copy_mu_: block ids on the device
  void ensure_kv_staging(size_t n_blocks);

  // What the last forward pass flattened: enough to enqueue its kernels again.
  struct Plan {
    int T = 0, R = 0, n_decode = 0, n_tiles = 0, max_ctx = 0;
    size_t T4 = 0, S4 = 0;
    size_t sampling_off = 0;  // ints from the start of the metadata to the rows' sampling parameters (0: none)
  };
  // How the logits rows are reduced on the device at the end of a pass.
  enum class Pick { None, Greedy, Sample };
  struct PickSpec {
    Pick kind = Pick::None;
    bool logprobs = false;
    bool truncated = false;  // some row asks for top-k / nucleus truncation
  };
  // Event marks of one pass while profiling is on.
  struct Prof {
    bool on = false;
    int first = 0, n = 0;
  };
  enum { kMarkStart, kMarkEnd, kMarkDecodeBegin, kMarkDecodeEnd, kMarkPrefillBegin, kMarkPrefillEnd };
  // `meta`: the packed metadata on the device (the layout forward() documents); `layer_events`:
  // record layer_done_[l] behind each layer's K/V append (not while the stream is being captured).
  void enqueue(const int* meta, const Plan& p, rb200_layer_cb cb, void* cb_ctx, PickSpec pick, Prof* prof,
               bool layer_events = true);
  void check_pipeline_status();
  void ensure_row_buffers(int R, PickSpec pick);
  // Validates the sampling parameters of R rows and says how the device will pick.
  PickSpec pick_of(const Outputs& out, int R) const;
  void fetch_outputs(const Outputs& out, int R, PickSpec pick);
  Prof begin_profile();
  void mark(Prof& p, int kind);
  void end_profile(Prof& p);

  Plan plan_;
  bool profiling_ = false;
  rb200_profile profile_{};
  std::vector<cudaEvent_t> prof_events_;
  std::vector<int> prof_kinds_;

  rb200_model_config c_;
  uint32_t flags_;
  int device_, num_blocks_, block_size_, max_tokens_, max_context_;
  int Hp_, Qp_, Ip_;  // hidden, q_dim and intermediate rounded up to the GEMM's k granularity
  bool fast_attention_ = false;
  cudaStream_t stream_ = nullptr, copy_stream_ = nullptr;
  std::vector<cudaEvent_t> layer_done_;

  Matrix embed_, lm_head_;
  DeviceBuf final_norm_, inv_freq_;
  std::vector<Layer> layers_;
  DeviceBuf kc_, vc_;

  DeviceBuf x_, xn_, qkv_, attn_, gu_, act_, logits_, argmax_tok_, argmax_val_, logprob_;
  DeviceBuf meta_dev_, decode_scratch_, gemv_scratch_, stage_;
  PinnedBuf meta_host_, result_host_;

  std::mutex copy_mu_;
  DeviceBuf kv_staging_, kv_ids_;
  PinnedBuf kv_pinned_;
  // Block ids travel host -> device through a small ring of pinned slots, so that calls
  // which only enqueue (the NCCL hop) can run ahead of the copy stream without a later
  // call overwriting ids an earlier upload has not read yet.
  struct IdSlot {
    PinnedBuf buf;
    cudaEvent_t uploaded = nullptr;
    bool used = false;
  };
  std::vector<IdSlot> id_slots_;
  int id_next_ = 0;

  std::unique_ptr<NcclState> nccl_;
  std::vector<std::unique_ptr<KvLink>> links_;  // under copy_mu_
  KvLink& link_of(int link);
  bool links_idle();
  void links_release();

  std::unique_ptr<DecodeSession> session_;
  cudaEvent_t pass_done_ = nullptr;  // recorded behind a pass that ran as a graph (no per-layer events)
  bool layer_events_stale_ = false;
};

}  // namespace rb200
