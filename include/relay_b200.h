/* relay_b200 — the C boundary of the B200 (sm_100a) implementation of relay's per-token
 * compute path.
 *
 * Two groups of entry points:
 *
 *  1. The backend: everything relay's `relay::Backend` virtual interface offers
 *     (engine/include/relay/backend.h:43-81) on an opaque handle, with plain pointers and
 *     sizes, so that a thin C++ subclass (or a cgo / ctypes / Swift binding) turns each
 *     virtual into one call. `make_cuda_backend` (backend.h:95-97) maps to rb200_create.
 *
 *  2. The operators: each hand-written kernel of the path on caller-owned DEVICE buffers,
 *     for parity tests and measurements at the shapes the model-level path does not reach.
 *
 * Conventions (the reference C API's, engine/include/relay/c_api.h:5-6 and
 * engine/src/c_api.cpp:31-46): functions that can fail return 0 or a valid pointer on
 * success and -1 or NULL on failure; rb200_last_error() then says why, per thread.
 * rb200_last_error_kind() classifies it the way the reference's exceptions do
 * (engine/src/cuda_backend.cu:512-518, 546, 448).
 *
 * There is no CPU fallback behind any of these calls: without a CUDA device they fail.
 */
#ifndef RELAY_B200_H
#define RELAY_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- errors ------------------------------------------------------------------------ */

enum {
  RB200_OK = 0,
  RB200_ERR_INVALID_ARGUMENT = 1, /* std::invalid_argument in the reference */
  RB200_ERR_OUT_OF_RANGE = 2,     /* std::out_of_range (token id) */
  RB200_ERR_RUNTIME = 3,          /* std::runtime_error (CUDA / NCCL) */
  RB200_ERR_LOGIC = 4             /* std::logic_error (e.g. update of an int8 matrix refused) */
};

const char* rb200_last_error(void);
int rb200_last_error_kind(void);
/* Number of CUDA devices the library can see (0 without a driver); never fails. */
int rb200_device_count(void);

/* ---- model description ------------------------------------------------------------- */

/* relay::ModelConfig (engine/include/relay/config.h:20-47), the fields the path reads. */
typedef struct rb200_model_config {
  int32_t hidden, intermediate, layers, heads, kv_heads, head_dim, vocab, max_position;
  double rms_eps, rope_theta;
  int32_t rope_scaling_type; /* 0: none, 1: "llama3" (config.h:12-18) */
  double rope_factor, rope_low_freq_factor, rope_high_freq_factor, rope_original_max_position;
  int32_t tie_embeddings, qkv_bias;
} rb200_model_config;

/* relay::LayerWeights / relay::HostWeights (engine/include/relay/weights.h:13-34):
 * float32, row-major [out, in], q/k/v fused into wqkv and gate/up into w_gate_up. */
typedef struct rb200_layer_weights {
  const float* attn_norm; /* [hidden] */
  const float* wqkv;      /* [q_dim + 2 kv_dim, hidden] */
  const float* bqkv;      /* [q_dim + 2 kv_dim] or NULL */
  const float* wo;        /* [hidden, q_dim] */
  const float* mlp_norm;  /* [hidden] */
  const float* w_gate_up; /* [2 intermediate, hidden]: gate rows, then up rows */
  const float* w_down;    /* [hidden, intermediate] */
} rb200_layer_weights;

typedef struct rb200_weights {
  const float* embed;      /* [vocab, hidden] */
  const float* final_norm; /* [hidden] */
  const float* lm_head;    /* [vocab, hidden], NULL when tied to embed */
  const rb200_layer_weights* layers;
} rb200_weights;

/* relay::CudaOptions (backend.h:85-94). */
enum {
  RB200_INT8_WEIGHTS = 1,        /* CudaOptions::int8_weights: per-output-row int8 for the layer matrices */
  RB200_REFERENCE_ATTENTION = 2, /* CudaOptions::reference_attention: the simple one-CTA-per-(token, head) kernel */
  RB200_GPU_ARGMAX = 4           /* forward also leaves each logit row's greedy token on the device (rb200_forward_greedy) */
};
/* CudaOptions::from_env (engine/src/cuda_backend.cu:37-42): RELAY_CUDA_ATTENTION=m0, RELAY_CUDA_INT8=1. */
uint32_t rb200_flags_from_env(void);

/* The head_dim/2 inverse rotary frequencies with Llama-3 scaling applied
 * (ModelConfig::rope_inv_freq, engine/src/config.cpp:79-109). Host only. */
int rb200_rope_inv_freq(const rb200_model_config* cfg, float* out);

/* Per-row symmetric int8 quantisation exactly as the reference's to_device_matrix
 * (engine/src/cuda_backend.cu:282-304): scale = max|w| / 127 (1 for a zero row),
 * q = lrintf(w / scale). Host only; w is [N, K] float32. */
int rb200_quantize_rows_int8(const float* w, int N, int K, int8_t* q_out, float* scale_out);

/* ---- the backend (relay::Backend) ---------------------------------------------------- */

typedef struct rb200_backend rb200_backend;

/* make_cuda_backend (backend.h:95-97; ctor engine/src/cuda_backend.cu:313-391).
 * `weights` may be NULL: every tensor then starts as zeros and is filled through
 * rb200_update_weight (which also takes device pointers), so a model too large for a
 * float32 host copy can be built tensor by tensor. */
rb200_backend* rb200_create(const rb200_model_config* cfg, const rb200_weights* weights, int num_blocks,
                            int block_size, int device, int max_batch_tokens, int max_context, uint32_t flags);
void rb200_destroy(rb200_backend* b);

/* Backend::name(): "b200". */
const char* rb200_name(const rb200_backend* b);
int rb200_get_config(const rb200_backend* b, rb200_model_config* out);
/* KVLayout (engine/include/relay/kv_cache.h:22-36): layers, kv_heads, head_dim, block_size, num_blocks. */
int rb200_get_kv_layout(const rb200_backend* b, int32_t out[5]);

/* LayerObserver::kv_written (backend.h:37-41): called on the calling thread right after
 * layer `layer`'s K/V append is enqueued; pair with rb200_wait_kv_written. */
typedef void (*rb200_layer_cb)(void* ctx, int layer);

/* Backend::forward (backend.h:50-52; engine/src/cuda_backend.cu:504-603). The batch is
 * relay::ForwardBatch flattened: chunk s has chunk_len[s] tokens (consecutive in `tokens`)
 * starting at position start_pos[s], and table_len[s] block ids (consecutive in `tables`).
 * want_logits may be NULL (all chunks want them). Writes [rows, vocab] float32 to
 * logits_out (host memory; cap_floats is its capacity) and returns rows, or -1.
 * Errors mirror the reference: "block table too short", "sequence longer than
 * max_context", "batch has more tokens than max_batch_tokens" (invalid argument),
 * "token id out of range" (out of range). An empty batch returns 0. */
int rb200_forward(rb200_backend* b, int n_seqs, const int32_t* tokens, const int32_t* chunk_len,
                  const int32_t* start_pos, const int32_t* table_len, const int32_t* tables,
                  const uint8_t* want_logits, int all_logits, rb200_layer_cb cb, void* cb_ctx, float* logits_out,
                  size_t cap_floats);

/* The same forward pass, but instead of the logits it returns each logit row's greedy
 * token (lowest id wins a tie: engine/src/sampler.cpp:17-22) and its logit, computed on
 * the device, so that only 8 bytes per row cross to the host. Needs RB200_GPU_ARGMAX. */
int rb200_forward_greedy(rb200_backend* b, int n_seqs, const int32_t* tokens, const int32_t* chunk_len,
                         const int32_t* start_pos, const int32_t* table_len, const int32_t* tables,
                         const uint8_t* want_logits, int all_logits, rb200_layer_cb cb, void* cb_ctx,
                         int32_t* token_out, float* logit_out, size_t cap_rows);

/* relay::SamplingParams (engine/include/relay/sampler.h:17-24), the fields the sampler reads,
 * plus `index`: the request's n-th generated token, which with `seed` fixes the random number
 * (engine/src/sampler.cpp:9-15), so a row samples the same token alone, in a batch or after
 * a recompute. */
typedef struct rb200_sampling_params {
  float temperature; /* <= 0: greedy */
  float top_p;       /* 1: no nucleus truncation */
  int32_t top_k;     /* 0: no limit */
  int32_t reserved;  /* 0 */
  uint64_t seed;
  uint64_t index;
} rb200_sampling_params;

/* The same forward pass with the sampler run on the device: per logits row, the token relay's
 * sample() / sample_with_log_prob() pick from that row (engine/src/sampler.cpp:33-72, called
 * per row by engine/src/engine.cpp:270-282) and, when logprob_out is not NULL, the
 * log-probability Engine reports with it (float64; relay narrows it to float). `sampling` is a
 * host array, one entry per logits row. All of relay's sampler runs on the device: greedy rows
 * (lowest id on ties), temperature sampling without truncation (inverse CDF in id order), and
 * top-k / nucleus truncation (candidates by decreasing logit, ties by id; sampler.cpp:77-104). */
int rb200_forward_sample(rb200_backend* b, int n_seqs, const int32_t* tokens, const int32_t* chunk_len,
                         const int32_t* start_pos, const int32_t* table_len, const int32_t* tables,
                         const uint8_t* want_logits, int all_logits, rb200_layer_cb cb, void* cb_ctx,
                         const rb200_sampling_params* sampling, int32_t* token_out, double* logprob_out,
                         size_t cap_rows);

/* ---- decode sessions ------------------------------------------------------------------
 * The step-with-deltas form of rb200_forward for steady-state decoding. The reference flattens
 * and uploads every sequence's token, position and whole block table on every step
 * (engine/src/cuda_backend.cu:508-566, driven by engine/src/engine.cpp:184-202); a session
 * keeps them on the device and a step brings only what changed. Results are bit-identical to
 * rb200_forward on the same batch. One session per backend; rb200_forward may be called in
 * between (for example to prefill a sequence that then takes a slot). */

/* Opens a session of n_seqs slots. Slot s has context_len[s] keys in the cache already (its
 * next token goes to that position) and table_len[s] block ids, consecutive in `tables`; spare
 * ids beyond what the context needs are kept for the positions to come. */
int rb200_decode_open(rb200_backend* b, int n_seqs, const int32_t* context_len, const int32_t* table_len,
                      const int32_t* tables);
/* Replaces the sequence in one slot (a finished request's slot taken by a new one). */
int rb200_decode_set_slot(rb200_backend* b, int slot, int context_len, int table_len, const int32_t* table);
/* One decode step over every slot. `tokens`: this step's token id per slot, or NULL to feed
 * each slot the token the previous step picked on the device (no token crosses to the host
 * and back). `new_block_seq[i]` / `new_block_id[i]`: block ids appended to slots' tables since
 * the last step (a slot whose context reaches a block boundary needs one: otherwise "block
 * table too short"). Outputs, each optional: token_out[n_seqs] (picked per `sampling`, host
 * array of n_seqs entries, NULL = greedy; same rules as rb200_forward_sample), logprob_out
 * [n_seqs], logits_out [n_seqs][vocab]. Every slot then stands one position further. Steps
 * of the same launch geometry are replayed as a CUDA graph from their second occurrence on
 * (RB200_DECODE_GRAPH=0 turns that off). Returns n_seqs, or -1. */
int rb200_decode_step(rb200_backend* b, const int32_t* tokens, int n_new_blocks, const int32_t* new_block_seq,
                      const int32_t* new_block_id, const rb200_sampling_params* sampling, int32_t* token_out,
                      double* logprob_out, float* logits_out, size_t cap_floats);
int rb200_decode_close(rb200_backend* b);

/* Backend::kv_block_bytes (engine/src/cuda_backend.cu:478): kv_heads * block_size * head_dim * 2. */
size_t rb200_kv_block_bytes(const rb200_backend* b);
/* Backend::read_kv_layer / write_kv_layer (backend.h:60-64; engine/src/cuda_backend.cu:630-664):
 * `buf` is host memory holding all K blocks then all V blocks in the order given. n = 1
 * with separate k/v pointers is read_kv_block / write_kv_block (backend.h:56-58). Safe to
 * call from another thread while rb200_forward runs. */
int rb200_read_kv_layer(rb200_backend* b, int layer, const int32_t* blocks, int n, void* k_out, void* v_out);
int rb200_write_kv_layer(rb200_backend* b, int layer, const int32_t* blocks, int n, const void* k_in,
                         const void* v_in);
/* Backend::wait_kv_written (engine/src/cuda_backend.cu:502). */
int rb200_wait_kv_written(rb200_backend* b, int layer);
/* Backend::update_weight (backend.h:72-80; engine/src/cuda_backend.cu:429-477): `src` is
 * n float32 values in relay's layout, in host memory or device memory of any GPU. Unlike
 * the reference, an int8 backend requantises the matrix on the device instead of refusing. */
int rb200_update_weight(rb200_backend* b, const char* name, const float* src, size_t n);

/* ---- measurement support (no counterpart in the reference: its benches time forward()
 *      from the host, tools/relay_attention_bench.cpp:82-95) ------------------------------ */

typedef struct rb200_profile {
  double total_ms;        /* device time of the profiled forward passes, first to last kernel */
  double decode_attn_ms;  /* of which split-context decode attention + merge */
  double prefill_attn_ms; /* of which flash prefill attention */
  uint64_t forwards, decode_attn_calls, prefill_attn_calls;
} rb200_profile;

/* While on, every forward pass brackets its attention launches with CUDA events on the
 * backend's stream and adds their times to the profile. */
int rb200_set_profiling(rb200_backend* b, int on);
/* Returns the profile accumulated so far and clears it. */
int rb200_get_profile(rb200_backend* b, rb200_profile* out);
/* Enqueues the kernels of the latest rb200_forward `iters` times from the metadata already
 * on the device (no host-to-device copy, logits stay on the device) and returns the device
 * time of all of them in ms_out. Every pass recomputes the same values. */
int rb200_forward_replay(rb200_backend* b, int iters, float* ms_out);
/* Fills both KV pools with N(0,1) values rounded to fp16 from a counter-based generator:
 * stands in for an untimed prefill when a benchmark needs a full cache. */
int rb200_debug_fill_kv(rb200_backend* b, uint64_t seed);
/* Kernels this library has launched in this process so far. */
uint64_t rb200_kernel_launches(void);

/* ---- the prefill -> decode KV hop over NCCL ------------------------------------------ */
/* Replaces the host-staged Layer payload of the transfer engine
 * (engine/src/kv_transfer.cpp:107-128 sender, :289-297 receiver) on the GPU->GPU hop:
 * gather kernel -> ncclSend on the sender, ncclRecv -> scatter kernel on the receiver,
 * both on the backend's copy stream. Payload order is the wire format's: all K blocks,
 * then all V blocks (engine/include/relay/kv_transfer.h:14-18). */

#define RB200_NCCL_ID_BYTES 128
/* Fills `id` (RB200_NCCL_ID_BYTES) on one rank; hand it to the others out of band. */
int rb200_nccl_unique_id(void* id);
/* Joins communicator of `nranks` as `rank`; collective across the ranks. */
int rb200_nccl_init(rb200_backend* b, const void* id, int nranks, int rank);
int rb200_nccl_finalize(rb200_backend* b);
/* Enqueue one layer's blocks to / from `peer`; returns once enqueued on the copy stream. */
int rb200_send_kv_layer(rb200_backend* b, int peer, int layer, const int32_t* blocks, int n);
int rb200_recv_kv_layer(rb200_backend* b, int peer, int layer, const int32_t* blocks, int n);
/* Waits for everything enqueued on the copy stream, at most timeout_ms (<= 0: 60 s); on
 * timeout the communicator is aborted and -1 returned. rb200_nccl_finalize and rb200_destroy
 * wait the same way with a 10 s limit, so an unmatched send or receive cannot block them. */
int rb200_kv_hop_sync(rb200_backend* b, int timeout_ms);

/* ---- the same hop over a K/V link: plain peer stores and two counters, no library kernel ---
 * A link joins one backend in each of two processes on one box. Each end creates its side (a
 * ring of n_slots landing slots of slot_bytes each in its own device memory) and gets a
 * handle; the ends swap handles out of band (the host connection that carries the transfer
 * engine's Hello frame, engine/src/kv_transfer.cpp:185-200) and connect. The k-th
 * rb200_kv_link_send_layer on one end pairs with the k-th rb200_kv_link_recv_layer on the
 * other: same payload and order as the Layer frames (engine/include/relay/kv_transfer.h:14-18;
 * sender engine/src/kv_transfer.cpp:107-128, receiver :269-301). The sender's gather kernel
 * stores the pages straight into the receiver's slot across NVLink (RB200_KV_LINK=ce: into its
 * own slot, which a copy engine then moves), the receiver scatters the slot into its own block
 * ids; slots are reused once the receiver has acknowledged them. Both calls only
 * enqueue (the send is ordered behind the layer's K/V append on the device);
 * rb200_kv_hop_sync waits for the links too, and on its deadline releases every wait the peer
 * has not satisfied and marks those links broken. A layer with more blocks than a slot holds
 * travels as several messages, cut the same way on both ends. */
#define RB200_KV_LINK_HANDLE_BYTES 128
/* Returns the link's id (>= 0) on this backend and fills handle_out (RB200_KV_LINK_HANDLE_BYTES). */
int rb200_kv_link_create(rb200_backend* b, int n_slots, size_t slot_bytes, void* handle_out);
/* Maps the other end's region; both ends must have been created with the same ring. */
int rb200_kv_link_connect(rb200_backend* b, int link, const void* peer_handle);
/* The same for two backends of one process (a process cannot open its own IPC handle): each end
 * takes the other's region by address; backends on different devices get peer access first.
 * A link orders its streams by counters the CUDA scheduler does not see, so its two ends belong
 * on two devices: on ONE device (tests) streams may share a hardware queue, and a wait enqueued
 * ahead of the work that satisfies it then holds that work back until the host deadline of
 * rb200_kv_link_wait / rb200_kv_hop_sync breaks the link. There, enqueue a message's send before
 * its receive and keep fewer messages in flight than the ring has slots, or give every stream its
 * own queue (CUDA_DEVICE_MAX_CONNECTIONS=32). */
int rb200_kv_link_connect_local(rb200_backend* a, int link_a, rb200_backend* b, int link_b);
int rb200_kv_link_send_layer(rb200_backend* b, int link, int layer, const int32_t* blocks, int n);
int rb200_kv_link_recv_layer(rb200_backend* b, int link, int layer, const int32_t* blocks, int n);
/* The same for n_layers consecutive layers of one request whose K/V is complete (a prompt handed
 * over after its prefill rather than streamed during it; relay's sender thread takes the queued
 * Layer jobs of such a request one frame at a time, engine/src/kv_transfer.cpp:130-150, each
 * through send_layer, :107-128): as many whole layers as a slot holds
 * travel as ONE message (one gather, one counter store), so a ring of slots of several layers
 * moves a prompt at NVLink's rate instead of the host's enqueue rate.
 * The receiver makes the matching call with the same first_layer, n_layers and n (the ends cut
 * messages by the same rule); rb200_kv_link_skip_layers is the dropping counterpart. With
 * n_layers == 1 these are the calls above. */
int rb200_kv_link_send_layers(rb200_backend* b, int link, int first_layer, int n_layers, const int32_t* blocks, int n);
int rb200_kv_link_recv_layers(rb200_backend* b, int link, int first_layer, int n_layers, const int32_t* blocks, int n);
int rb200_kv_link_skip_layers(rb200_backend* b, int link, int n_layers, int n);
/* How the calls above cut n_layers layers of n blocks of block_bytes (each block once for K and
 * once for V) into messages for a ring of slots of slot_bytes: the number of messages (returned;
 * -1 for arguments no link accepts) and the largest number of whole layers one message carries
 * (0 when a single layer already needs several messages). Pure host arithmetic, the same on
 * both ends; a sender may keep as many messages in flight as the ring has slots. */
int rb200_kv_link_plan(size_t slot_bytes, size_t block_bytes, int n_layers, int n, int32_t* layers_per_message_out);
/* Sender: waits until every layer sent so far has been read out of the cache (its gather has
 * run; the copy may still be under way), after which the sender's blocks may be rewritten. The
 * reference frees a request's blocks once its last frame is written
 * (engine/src/kv_transfer.cpp:139-160); its read_kv_layer is synchronous, this call restores
 * that guarantee. At most timeout_ms (<= 0: 60 s); on the deadline the link is broken, -1. */
int rb200_kv_link_wait_gathered(rb200_backend* b, int link, int timeout_ms);
/* Receiver: consumes a layer of n blocks from the link without landing it anywhere, the
 * counterpart of the transfer engine reading and dropping a Layer frame it has no room for
 * (engine/src/kv_transfer.cpp:284-288). */
int rb200_kv_link_skip_layer(rb200_backend* b, int link, int n);
/* Waits until everything enqueued on this link has run (write_kv_layer's contract is that the
 * pages are in the cache when it returns: engine/src/cuda_backend.cu:649-664), at most
 * timeout_ms (<= 0: 60 s); on the deadline the link is released, marked broken, and -1 returned. */
int rb200_kv_link_wait(rb200_backend* b, int link, int timeout_ms);
/* After rb200_kv_hop_sync; unmaps the peer's region and frees this end's. */
int rb200_kv_link_close(rb200_backend* b, int link);

/* ---- operators on device buffers ----------------------------------------------------- */
/* All pointers below are DEVICE pointers on the current device unless said otherwise;
 * `stream` is a cudaStream_t (NULL: the default stream). Calls return once enqueued. */

/* The batch's position metadata, engine/src/cuda_kernels.cuh:16-26 (TokenMeta): token t is
 * at position pos[t] of sequence seq[t], whose block ids start at tables[table_off[seq]]. */
typedef struct rb200_token_meta {
  const int32_t* pos;
  const int32_t* seq;
  const int32_t* table_off;
  const int32_t* tables;
} rb200_token_meta;

/* Geometry shared by the attention and KV operators. K and V pools are one layer's
 * [num_blocks][kv_heads][block_size][head_dim] fp16 (engine/src/cuda_backend.cu:368-371). */
typedef struct rb200_attn_shape {
  int32_t heads, kv_heads, head_dim, block_size;
  int32_t q_stride; /* floats between consecutive tokens' q rows (QKV in the model) */
  int32_t o_stride; /* halves between consecutive tokens' output rows */
} rb200_attn_shape;

#define RB200_DECODE_SLICE 512 /* keys per split-context slice (engine/src/cuda_kernels.cuh:180-190); slices grow in
                                  multiples of it when a batch has enough (token, KV head) pairs to fill the GPU */

/* Scratch that is always enough for the split decode of n_decode tokens whose longest context is
 * max_ctx: per (token, head, 512-key slice) D + 2 floats. Returns bytes. */
size_t rb200_decode_scratch_bytes(const rb200_attn_shape* s, int n_decode, int max_ctx);
/* What rb200_decode_attention will do with such a batch on the current device: keys per slice
 * (a multiple of RB200_DECODE_SLICE; the launch stand-in of the reference's fixed 512,
 * engine/src/cuda_backend.cu:560-565), slices per context, and (returned) the bytes of partial
 * results it will really park in the scratch: 0 when every context is one slice. */
size_t rb200_decode_plan(const rb200_attn_shape* s, int n_decode, int max_ctx, int32_t* slice_out, int32_t* parts_out);
/* Split-context decode attention + LSE merge (replaces decode_attention_kernel and
 * decode_combine_kernel, engine/src/cuda_kernels.cuh:223-362). q: fp32 rows of the batch
 * (token t's head h at q + t*q_stride + h*D); decode_tokens[i] is the batch row of the
 * i-th decode token, whose context is pos+1 keys; out: fp16 [T][o_stride]. */
int rb200_decode_attention(const rb200_attn_shape* s, const float* q, const rb200_token_meta* m,
                           const int32_t* decode_tokens, int n_decode, int max_ctx, const void* k_pool,
                           const void* v_pool, void* scratch, size_t scratch_bytes, void* out, void* stream);

/* No counterpart in the reference. The same split-context decode attention for callers
 * that cannot allocate device memory where they need it: a serving process that has
 * already handed every free byte of the GPU to its KV pool (a cudaMalloc there fails), or
 * a latency-critical loop that must not hit the device-wide stall of cudaMalloc/cudaFree.
 * The partial results live in a fixed RB200_STATIC_DECODE_SCRATCH_BYTES array inside the
 * library image (each GPU that loads the library carries it until the process exits);
 * inputs and outputs are still the caller's. This call allocates nothing, on the host side
 * or the device side. Limits and rules:
 *  - a batch whose partials (what rb200_decode_plan returns, never more than
 *    rb200_decode_scratch_bytes) exceed the array is rejected with an invalid-argument error
 *    naming both sizes;
 *  - the first call on each device looks up the array's device address and keeps it for the
 *    life of the process; make that first call before starting any stream capture on that
 *    device, and do not call cudaDeviceReset in a process that uses this entry point (the
 *    kept address would name memory of the destroyed context);
 *  - all calls share the one array, which keeps whatever the previous call left (nothing
 *    in it needs clearing: each call overwrites what it later reads); two calls that overlap
 *    on the GPU, e.g. on different streams, race on it and must be serialised by the caller. */
#define RB200_STATIC_DECODE_SCRATCH_BYTES (8u << 20)
int rb200_decode_attention_static(const rb200_attn_shape* s, const float* q, const rb200_token_meta* m,
                                  const int32_t* decode_tokens, int n_decode, int max_ctx, const void* k_pool,
                                  const void* v_pool, void* out, void* stream);

/* Causal flash attention for chunks of several tokens over the paged cache (replaces
 * flash_prefill_kernel, engine/src/cuda_kernels.cuh:51-178). tiles[i] = {first batch row,
 * row count <= RB200_PREFILL_ROWS} as built by engine/src/cuda_backend.cu:533-545. */
#define RB200_PREFILL_ROWS 64
int rb200_prefill_attention(const rb200_attn_shape* s, const float* q, const rb200_token_meta* m,
                            const int32_t* tiles, int n_tiles, const void* k_pool, const void* v_pool, void* out,
                            void* stream);

/* One CTA per (token, head) attention, any head_dim and group size (the role of the
 * reference's M0 attention_kernel, engine/src/cuda_backend.cu:202-243). */
int rb200_reference_attention(const rb200_attn_shape* s, const float* q, const rb200_token_meta* m, int n_tokens,
                              const void* k_pool, const void* v_pool, void* out, void* stream);

/* Weight-only int8 GEMV for 1..8 tokens (replaces gemv_int8_kernel,
 * engine/src/cuda_kernels.cuh:378-430): y[T,N] = scale[n] * sum_k Wq[n,k] x[t,k] + beta*y.
 * Wq int8 [N][ldw], x fp16 [T][ldx], y fp32 [T][N]; K a multiple of 64, ldw and ldx
 * multiples of 16 and 8 elements. `scratch` (rb200_gemv_scratch_bytes, 16-byte aligned)
 * holds two things: split-K partials of the register kernel, which must be zero before
 * the first use and are left zero again, and the activations rewritten as int8 digits
 * for the integer tensor-core kernel (no initial state). Calls that share a scratch
 * buffer must be ordered on one stream. */
size_t rb200_gemv_scratch_bytes(int N, int K);
int rb200_gemv_int8(const int8_t* wq, const float* scale, const void* x, float* y, int T, int K, int N, int ldw,
                    int ldx, float beta, void* scratch, size_t scratch_bytes, void* stream);
/* The same product for fp16 weights (the T <= 8 case of the reference's cublasGemmEx
 * call, engine/src/cuda_backend.cu:724-730). */
int rb200_gemv_f16(const void* w, const void* x, float* y, int T, int K, int N, int ldw, int ldx, float beta,
                   void* scratch, size_t scratch_bytes, void* stream);

/* y[T,N] = x[T,K] W[N,K]^T (+ beta*y) on tensor cores for any T: fp16 weights (replaces
 * cublasGemmEx, engine/src/cuda_backend.cu:724-730) or int8 weights (replaces
 * dequant_int8_kernel + cuBLAS, engine/src/cuda_kernels.cuh:432-436,
 * engine/src/cuda_backend.cu:719-721): multiplied as integers against int8 digits of the
 * activations for few tokens, widened to fp16 inside the main loop for more. Exactly one
 * of w_f16 / w_i8 is non-NULL. The int8 few-token path takes a temporary buffer from the
 * stream's memory pool (cudaMallocAsync / cudaFreeAsync on `stream`). */
int rb200_gemm(const void* w_f16, const int8_t* w_i8, const float* scale, const void* x, float* y, int T, int K,
               int N, int ldw, int ldx, float beta, void* stream);

/* 0, or the code that a bounded pipeline wait inside the tensor-core GEMM left on the
 * current device when it gave up (the launch then produced no valid output). */
int rb200_gemm_status(void);

/* rmsnorm_kernel (engine/src/cuda_backend.cu:157-167): out[r] = w * x[rows ? rows[r] : r] * rsqrt(mean(x^2)+eps),
 * fp32 -> fp16 rows of ld_out halves (columns H..ld_out-1 are written as zero). */
int rb200_rmsnorm(const float* x, const int32_t* rows, const float* w, void* out, int R, int H, int ld_out,
                  float eps, void* stream);
/* embed_kernel (engine/src/cuda_backend.cu:150-154): x[t] = float(table[tokens[t]]). */
int rb200_embed(const int32_t* tokens, const void* table, float* x, int T, int H, int ld_table, void* stream);
/* qkv_post_kernel (engine/src/cuda_backend.cu:171-198): bias, RoPE on q and k in place,
 * K/V append to the paged pools as fp16. bias may be NULL. */
int rb200_qkv_post(float* qkv, const float* bias, const float* inv_freq, const rb200_token_meta* m, int T,
                   void* k_pool, void* v_pool, int heads, int kv_heads, int head_dim, int block_size,
                   void* stream);
/* silu_mul_kernel (engine/src/cuda_backend.cu:245-253): act = silu(g) * u, fp32 [T][2I] -> fp16 [T][ld_act]. */
int rb200_silu_mul(const float* gu, void* act, int T, int I, int ld_act, void* stream);
/* f32_to_f16_kernel (engine/src/cuda_backend.cu:110-116): round to nearest even. */
int rb200_f32_to_f16(const float* in, void* out, size_t n, void* stream);
/* kv_gather_kernel / kv_scatter_kernel (engine/src/cuda_backend.cu:257-270): staging is
 * [K of each block][V of each block]; block_bytes a multiple of 16. */
int rb200_kv_gather(const void* k_pool, const void* v_pool, const int32_t* blocks, int n, size_t block_bytes,
                    void* staging, void* stream);
int rb200_kv_scatter(void* k_pool, void* v_pool, const int32_t* blocks, int n, size_t block_bytes,
                     const void* staging, void* stream);
/* Greedy token of each row of logits [R][V] (lowest id wins ties, engine/src/sampler.cpp:17-22). */
int rb200_argmax_rows(const float* logits, int R, int V, int32_t* token_out, float* logit_out, void* stream);
/* The device sampler on rows of logits [R][V] (engine/src/sampler.cpp:33-105): `params` is a
 * DEVICE array of R entries (see rb200_forward_sample); logprob_out (float64 [R]) may be NULL. */
int rb200_sample_rows(const float* logits, int R, int V, const rb200_sampling_params* params, int32_t* token_out,
                      double* logprob_out, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* RELAY_B200_H */
