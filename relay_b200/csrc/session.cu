// Decode sessions: a batch of single-token sequences whose positions, block tables and picked
// tokens stay on the device from one step to the next.
//
// The reference rebuilds and uploads every sequence's whole block table, position and token on
// every step (engine/src/cuda_backend.cu:508-566, called once per step by
// engine/src/engine.cpp:184-202). In steady-state decoding almost none of that changes: a
// sequence moves one position forward, its table gains one block id every block_size steps, and
// its next token is the one the previous step picked. A session keeps that state in device
// memory in exactly the packed layout Backend::forward builds, so the same kernels run on it;
// a step uploads only what changed (the caller's token ids unless the device feeds its own,
// the block ids appended since the last step, the rows' sampling parameters) in one small copy.
//
// Steps with the same launch geometry (the decode-attention slice plan and the way tokens are
// picked) are captured once as a CUDA graph and replayed, which takes the ~300 kernel launches
// of a step off the host. Everything a captured kernel points at is owned by the session or by
// the backend's persistent buffers; if one of those is regrown the graphs are dropped.
#include <cstdlib>
#include <cstring>

#include "backend.h"

namespace rb200 {

namespace {

// Applies a step's delta to the resident state: this step's tokens (the caller's, or the ones
// the previous step picked), the block ids appended to the tables.
__global__ void session_advance_kernel(int* __restrict__ meta, const int* __restrict__ picked, int S, int cap, int T4,
                                       int tables_off, int delta_off, int tokens_off, int blocks_off) {
  // No pdl_trigger(): the kernels of the step read this metadata before their own dependency
  // wait, so none of them may start before this kernel (and session_finish_kernel of the step
  // before it, which it waits for) has completed.
  pdl_wait();
  const int* hdr = meta + delta_off;
  const int n_new = hdr[0], feed_own = hdr[1];
  for (int s = threadIdx.x; s < S; s += blockDim.x) meta[s] = feed_own ? picked[s] : meta[tokens_off + s];
  for (int i = threadIdx.x; i < n_new; i += blockDim.x) {
    const int* t = meta + blocks_off + 3 * i;
    meta[tables_off + t[0] * cap + t[1]] = t[2];
  }
  (void)T4;
}

// Every sequence has consumed one position.
__global__ void session_finish_kernel(int* __restrict__ pos, int S) {
  pdl_trigger();
  pdl_wait();
  for (int s = threadIdx.x; s < S; s += blockDim.x) pos[s] += 1;
}

bool graphs_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("RB200_DECODE_GRAPH");
    return !(e && e[0] == '0');
  }();
  return on;
}

}  // namespace

void Backend::decode_open(int n_seqs, const int32_t* context_len, const int32_t* table_len, const int32_t* tables) {
  set_device();
  RB_REQUIRE(n_seqs > 0, "decode_open: needs at least one sequence");
  if (n_seqs > max_tokens_) fail(RB200_ERR_INVALID_ARGUMENT, "batch has more tokens than max_batch_tokens");
  RB_REQUIRE(context_len && table_len && tables, "decode_open: null argument");
  RB_REQUIRE(fast_attention_, "decode_open: this head layout runs on the reference attention kernel; use rb200_forward");
  const int bs = block_size_;
  auto s = std::make_unique<DecodeSession>();
  s->S = n_seqs;
  s->cap = round_up(div_up(max_context_, bs), 4);
  s->T4 = static_cast<size_t>(round_up(n_seqs, 4));
  s->S4 = s->T4;
  s->ctx.assign(context_len, context_len + n_seqs);
  s->tlen.assign(table_len, table_len + n_seqs);
  const size_t tables_off = 7 * s->T4 + s->S4;
  s->delta_off = tables_off + static_cast<size_t>(n_seqs) * s->cap;
  s->tokens_off = s->delta_off + 4;
  s->blocks_off = s->tokens_off + s->S4;
  s->sampling_off = s->blocks_off + static_cast<size_t>(round_up(3 * n_seqs, 4));
  s->delta_ints = s->sampling_off + static_cast<size_t>(n_seqs) * 8 - s->delta_off;
  const size_t total = s->delta_off + s->delta_ints;
  std::vector<int> hm(total, 0);
  int *h_pos = hm.data() + s->T4, *h_seq = hm.data() + 2 * s->T4, *h_rows = hm.data() + 3 * s->T4, *h_dec = hm.data() + 4 * s->T4;
  int* h_toff = hm.data() + 7 * s->T4;
  int* h_tables = hm.data() + tables_off;
  long long tb = 0;
  for (int i = 0; i < n_seqs; ++i) {
    RB_REQUIRE(context_len[i] >= 0 && table_len[i] >= 0, "decode_open: negative field");
    if (context_len[i] + 1 > max_context_) fail(RB200_ERR_INVALID_ARGUMENT, "sequence longer than max_context");
    if (table_len[i] < div_up(context_len[i], bs)) fail(RB200_ERR_INVALID_ARGUMENT, "block table too short");
    RB_REQUIRE(table_len[i] <= s->cap, "decode_open: block table longer than max_context allows");
    for (int j = 0; j < table_len[i]; ++j) {
      const int id = tables[tb + j];
      if (id < 0 || id >= num_blocks_) fail(RB200_ERR_INVALID_ARGUMENT, "block id out of range");
      h_tables[static_cast<size_t>(i) * s->cap + j] = id;
    }
    tb += table_len[i];
    h_pos[i] = context_len[i];  // the position this step's token will take
    h_seq[i] = i;
    h_rows[i] = i;
    h_dec[i] = i;
    h_toff[i] = i * s->cap;
  }
  s->meta = DeviceBuf(total * 4);
  s->delta_host.ensure(s->delta_ints * 4);
  RB_CUDA(cudaMemcpyAsync(s->meta.p, hm.data(), total * 4, cudaMemcpyHostToDevice, stream_));
  RB_CUDA(cudaStreamSynchronize(stream_));  // hm is pageable and about to go out of scope
  if (!pass_done_) RB_CUDA(cudaEventCreateWithFlags(&pass_done_, cudaEventDisableTiming));
  session_ = std::move(s);
}

void Backend::decode_set_slot(int slot, int context_len, int table_len, const int32_t* table) {
  set_device();
  RB_REQUIRE(session_ != nullptr, "decode_set_slot: no open session");
  DecodeSession& s = *session_;
  RB_REQUIRE(slot >= 0 && slot < s.S, "decode_set_slot: no such slot");
  RB_REQUIRE(context_len >= 0 && table_len >= 0 && (table || table_len == 0), "decode_set_slot: bad arguments");
  if (context_len + 1 > max_context_) fail(RB200_ERR_INVALID_ARGUMENT, "sequence longer than max_context");
  if (table_len < div_up(context_len, block_size_)) fail(RB200_ERR_INVALID_ARGUMENT, "block table too short");
  RB_REQUIRE(table_len <= s.cap, "decode_set_slot: block table longer than max_context allows");
  for (int j = 0; j < table_len; ++j)
    if (table[j] < 0 || table[j] >= num_blocks_) fail(RB200_ERR_INVALID_ARGUMENT, "block id out of range");
  std::vector<int> row(static_cast<size_t>(s.cap), 0);
  std::memcpy(row.data(), table, static_cast<size_t>(table_len) * 4);
  int* dm = s.meta.as<int>();
  const size_t tables_off = 7 * s.T4 + s.S4;
  RB_CUDA(cudaMemcpyAsync(dm + tables_off + static_cast<size_t>(slot) * s.cap, row.data(), row.size() * 4, cudaMemcpyHostToDevice, stream_));
  RB_CUDA(cudaMemcpyAsync(dm + s.T4 + slot, &context_len, 4, cudaMemcpyHostToDevice, stream_));
  RB_CUDA(cudaStreamSynchronize(stream_));
  s.ctx[slot] = context_len;
  s.tlen[slot] = table_len;
  s.have_picked = false;  // the new sequence's first token has to come from the caller
}

void Backend::decode_close() {
  if (!session_) return;
  set_device();
  RB_CUDA(cudaStreamSynchronize(stream_));
  session_.reset();
}

int Backend::decode_step(const int32_t* tokens, int n_new, const int32_t* new_seq, const int32_t* new_id, const Outputs& out) {
  set_device();
  RB_REQUIRE(session_ != nullptr, "decode_step: no open session (rb200_decode_open)");
  DecodeSession& s = *session_;
  const int S = s.S, bs = block_size_, V = c_.vocab;
  RB_REQUIRE(n_new >= 0 && n_new <= S && (n_new == 0 || (new_seq && new_id)), "decode_step: bad new-block list");
  const bool feed_own = tokens == nullptr;
  if (feed_own && !s.have_picked)
    fail(RB200_ERR_INVALID_ARGUMENT, "decode_step: no token ids given and the previous step picked none on the device");
  if (!feed_own)
    for (int i = 0; i < S; ++i)
      if (tokens[i] < 0 || tokens[i] >= V) fail(RB200_ERR_OUT_OF_RANGE, "token id out of range");
  if (out.logits && static_cast<size_t>(S) * V > out.cap_floats) fail(RB200_ERR_INVALID_ARGUMENT, "logits buffer too small");
  const PickSpec pick = pick_of(Outputs{nullptr, 0, out.tokens, nullptr, out.sampling, out.logprobs, static_cast<size_t>(S)}, S);

  // Validate against a copy of the table lengths, so that a refused step changes nothing.
  std::vector<int> tlen = s.tlen;
  int* hd = s.delta_host.as<int>();
  int* h_tok = hd + (s.tokens_off - s.delta_off);
  int* h_blk = hd + (s.blocks_off - s.delta_off);
  for (int i = 0; i < n_new; ++i) {
    RB_REQUIRE(new_seq[i] >= 0 && new_seq[i] < S, "decode_step: new block for a slot that does not exist");
    if (new_id[i] < 0 || new_id[i] >= num_blocks_) fail(RB200_ERR_INVALID_ARGUMENT, "block id out of range");
    RB_REQUIRE(tlen[new_seq[i]] < s.cap, "decode_step: block table longer than max_context allows");
    h_blk[3 * i] = new_seq[i];
    h_blk[3 * i + 1] = tlen[new_seq[i]]++;
    h_blk[3 * i + 2] = new_id[i];
  }
  int max_ctx = 0;
  for (int i = 0; i < S; ++i) {
    const int end = s.ctx[i] + 1;
    if (tlen[i] < div_up(end, bs)) fail(RB200_ERR_INVALID_ARGUMENT, "block table too short");
    if (end > max_context_) fail(RB200_ERR_INVALID_ARGUMENT, "sequence longer than max_context");
    max_ctx = std::max(max_ctx, end);
  }
  hd[0] = n_new;
  hd[1] = feed_own ? 1 : 0;
  hd[2] = hd[3] = 0;
  if (!feed_own) std::memcpy(h_tok, tokens, static_cast<size_t>(S) * 4);
  if (pick.kind == Pick::Sample) {
    auto* sp = reinterpret_cast<rb200_sampling_params*>(hd + (s.sampling_off - s.delta_off));
    for (int r = 0; r < S; ++r) sp[r] = out.sampling ? out.sampling[r] : rb200_sampling_params{0.0f, 1.0f, 0, 0, 0, 0};
  }

  const int D = c_.head_dim, QKV = (c_.heads + 2 * c_.kv_heads) * D;
  const AttnShape shape{c_.heads, c_.kv_heads, D, bs, QKV, Qp_, pool_rows()};
  decode_scratch_.ensure(decode_scratch_bytes(shape, S, max_ctx));
  ensure_row_buffers(S, PickSpec{pick.kind == Pick::None ? Pick::Greedy : pick.kind, pick.logprobs});  // picked tokens always have a home
  const uintptr_t sig = reinterpret_cast<uintptr_t>(decode_scratch_.p) ^ (reinterpret_cast<uintptr_t>(logits_.p) << 1) ^
                        (reinterpret_cast<uintptr_t>(argmax_tok_.p) << 2) ^ (reinterpret_cast<uintptr_t>(argmax_val_.p) << 3) ^
                        (reinterpret_cast<uintptr_t>(logprob_.p) << 4);
  if (sig != s.buffers_sig) {  // a buffer the captured kernels point at was regrown: the graphs are stale
    for (auto& g : s.graphs) cudaGraphExecDestroy(g.second);
    s.graphs.clear();
    s.seen.clear();
    s.buffers_sig = sig;
  }

  int* dm = s.meta.as<int>();
  RB_CUDA(cudaMemcpyAsync(dm + s.delta_off, hd, s.delta_ints * 4, cudaMemcpyHostToDevice, stream_));
  Plan p{S, S, S, 0, max_ctx, s.T4, s.S4, pick.kind == Pick::Sample ? s.sampling_off : 0};
  const int tables_off = static_cast<int>(7 * s.T4 + s.S4);
  auto run = [&](bool layer_events) {
    count_launch();
    launch_pdl(session_advance_kernel, dim3(1), dim3(256), 0, stream_, dm, argmax_tok_.as<int>(), S, s.cap, static_cast<int>(s.T4),
               tables_off, static_cast<int>(s.delta_off), static_cast<int>(s.tokens_off), static_cast<int>(s.blocks_off));
    enqueue(dm, p, nullptr, nullptr, pick, nullptr, layer_events);
    count_launch();
    launch_pdl(session_finish_kernel, dim3(1), dim3(256), 0, stream_, dm + s.T4, S);
  };

  const DecodePlan dp = plan_decode(shape, S, max_ctx);
  const uint64_t key = (static_cast<uint64_t>(dp.parts) << 40) ^ (static_cast<uint64_t>(dp.slice) << 8) ^
                       (static_cast<uint64_t>(pick.kind) << 2) ^ (pick.truncated ? 2u : 0u) ^ (pick.logprobs ? 1u : 0u);
  bool as_graph = false;
  if (graphs_enabled()) {
    auto it = s.graphs.find(key);
    if (it != s.graphs.end()) {
      RB_CUDA(cudaGraphLaunch(it->second, stream_));
      count_launch();
      as_graph = true;
    } else if (s.seen[key]++ >= 1) {
      // This geometry has run once in the ordinary way (first-use set-up of every kernel is done):
      // capture it. A capture that fails leaves the step to the ordinary path, for good.
      cudaGraph_t g = nullptr;
      cudaGraphExec_t exec = nullptr;
      bool ok = cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
      if (ok) {
        try {
          run(false);
        } catch (...) {
          ok = false;
        }
        if (cudaStreamEndCapture(stream_, &g) != cudaSuccess || g == nullptr) ok = false;
      }
      if (ok && cudaGraphInstantiate(&exec, g, 0) != cudaSuccess) ok = false;
      if (g) cudaGraphDestroy(g);
      if (ok) {
        s.graphs[key] = exec;
        RB_CUDA(cudaGraphLaunch(exec, stream_));
        count_launch();
        as_graph = true;
      } else {
        cudaGetLastError();
        s.seen[key] = -(1 << 30);  // never try this geometry again
      }
    }
  }
  if (!as_graph) run(true);
  if (as_graph) RB_CUDA(cudaEventRecord(pass_done_, stream_));
  layer_events_stale_ = as_graph;
  plan_ = Plan{};  // rb200_forward_replay replays forward passes, not session steps

  fetch_outputs(out, S, pick);
  result_host_.ensure(sizeof(int));
  RB_CUDA(cudaMemcpyAsync(result_host_.p, umma_status_word(), sizeof(int), cudaMemcpyDeviceToHost, stream_));
  RB_CUDA(cudaGetLastError());
  RB_CUDA(cudaStreamSynchronize(stream_));
  // The step ran: the mirror follows the device.
  s.tlen = tlen;
  for (int i = 0; i < S; ++i) s.ctx[i] += 1;
  s.have_picked = pick.kind != Pick::None;
  check_pipeline_status();
  return S;
}

}  // namespace rb200
