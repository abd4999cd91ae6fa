// TEST INFRASTRUCTURE, not product code: a flat C face over relay's own, unmodified
// float32 CPU backend (engine/src/cpu_backend.cpp), so that Python tests and the
// benchmark's cpu_baseline leg can drive the real reference through ctypes. It is compiled
// by oracle/Makefile together with the reference's sources, where they lie, into
// oracle/_ref/librelay_ref.so. Nothing under relay_b200/ may link or load it.
#include <omp.h>

#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "relay/backend.h"
#include "relay/engine.h"
#include "relay/safetensors.h"
#include "relay/sampler.h"
#include "relay_b200.h"

namespace {

thread_local std::string g_err;

struct Ref {
  relay::HostWeights w;
  std::unique_ptr<relay::Backend> be;
};

template <class F>
int guarded(F&& f) {
  try {
    return f();
  } catch (const std::exception& e) {
    g_err = e.what();
    return -1;
  }
}

std::vector<float> vec(const float* p, std::size_t n) { return p ? std::vector<float>(p, p + n) : std::vector<float>(); }

relay::ModelConfig to_config(const rb200_model_config& c) {
  relay::ModelConfig m;
  m.model_type = c.qkv_bias ? "qwen2" : "llama";
  m.hidden = c.hidden;
  m.intermediate = c.intermediate;
  m.layers = c.layers;
  m.heads = c.heads;
  m.kv_heads = c.kv_heads;
  m.head_dim = c.head_dim;
  m.vocab = c.vocab;
  m.max_position = c.max_position;
  m.rms_eps = c.rms_eps;
  m.rope_theta = c.rope_theta;
  if (c.rope_scaling_type == 1) {
    m.rope_scaling.type = "llama3";
    m.rope_scaling.factor = c.rope_factor;
    m.rope_scaling.low_freq_factor = c.rope_low_freq_factor;
    m.rope_scaling.high_freq_factor = c.rope_high_freq_factor;
    m.rope_scaling.original_max_position = c.rope_original_max_position;
  }
  m.tie_embeddings = c.tie_embeddings != 0;
  m.qkv_bias = c.qkv_bias != 0;
  return m;
}

void from_config(const relay::ModelConfig& m, rb200_model_config* c) {
  std::memset(c, 0, sizeof(*c));
  c->hidden = m.hidden;
  c->intermediate = m.intermediate;
  c->layers = m.layers;
  c->heads = m.heads;
  c->kv_heads = m.kv_heads;
  c->head_dim = m.head_dim;
  c->vocab = m.vocab;
  c->max_position = m.max_position;
  c->rms_eps = m.rms_eps;
  c->rope_theta = m.rope_theta;
  c->rope_scaling_type = m.rope_scaling.type == "llama3" ? 1 : 0;
  c->rope_factor = m.rope_scaling.factor;
  c->rope_low_freq_factor = m.rope_scaling.low_freq_factor;
  c->rope_high_freq_factor = m.rope_scaling.high_freq_factor;
  c->rope_original_max_position = m.rope_scaling.original_max_position;
  c->tie_embeddings = m.tie_embeddings;
  c->qkv_bias = m.qkv_bias;
}

relay::ForwardBatch to_batch(int n_seqs, const int* tokens, const int* chunk_len, const int* start_pos,
                             const int* table_len, const int* tables, const unsigned char* want, int all_logits) {
  relay::ForwardBatch b;
  b.all_logits = all_logits != 0;
  std::size_t t = 0, tb = 0;
  for (int s = 0; s < n_seqs; ++s) {
    relay::SeqChunk ch;
    ch.tokens.assign(tokens + t, tokens + t + chunk_len[s]);
    ch.start_pos = start_pos[s];
    ch.block_table.assign(tables + tb, tables + tb + table_len[s]);
    ch.want_logits = want ? want[s] != 0 : true;
    t += chunk_len[s];
    tb += table_len[s];
    b.seqs.push_back(std::move(ch));
  }
  return b;
}

}  // namespace

extern "C" {

const char* ref_last_error() { return g_err.c_str(); }

// A CPU backend over a copy of the given float32 weights (relay's fused layout).
void* ref_create(const rb200_model_config* cfg, const rb200_weights* w, int num_blocks, int block_size) {
  try {
    auto r = std::make_unique<Ref>();
    r->w.config = to_config(*cfg);
    const relay::ModelConfig& c = r->w.config;
    const std::size_t H = c.hidden, Q = c.q_dim(), KV = c.kv_dim(), I = c.intermediate, V = c.vocab;
    r->w.embed = vec(w->embed, V * H);
    r->w.final_norm = vec(w->final_norm, H);
    r->w.lm_head = vec(w->lm_head, V * H);
    for (int l = 0; l < c.layers; ++l) {
      const rb200_layer_weights& s = w->layers[l];
      relay::LayerWeights L;
      L.attn_norm = vec(s.attn_norm, H);
      L.wqkv = vec(s.wqkv, (Q + 2 * KV) * H);
      L.bqkv = vec(s.bqkv, Q + 2 * KV);
      L.wo = vec(s.wo, H * Q);
      L.mlp_norm = vec(s.mlp_norm, H);
      L.w_gate_up = vec(s.w_gate_up, 2 * I * H);
      L.w_down = vec(s.w_down, H * I);
      r->w.layers.push_back(std::move(L));
    }
    r->be = relay::make_cpu_backend(r->w, num_blocks, block_size);
    return r.release();
  } catch (const std::exception& e) {
    g_err = e.what();
    return nullptr;
  }
}

// A CPU backend over a Hugging Face model directory (config.json + safetensors).
void* ref_load(const char* dir, int num_blocks, int block_size) {
  try {
    auto r = std::make_unique<Ref>();
    r->w = relay::HostWeights::load(dir);
    r->be = relay::make_cpu_backend(r->w, num_blocks, block_size);
    return r.release();
  } catch (const std::exception& e) {
    g_err = e.what();
    return nullptr;
  }
}

void ref_destroy(void* h) { delete static_cast<Ref*>(h); }

int ref_get_config(void* h, rb200_model_config* out) {
  from_config(static_cast<Ref*>(h)->w.config, out);
  return 0;
}

// The loaded model's float32 tensors by relay's names (c_api.cpp's relay_model_tensor).
const float* ref_tensor(void* h, const char* name, long long* numel) {
  Ref* r = static_cast<Ref*>(h);
  std::string n = name;
  const std::vector<float>* v = nullptr;
  if (n == "embed") v = &r->w.embed;
  else if (n == "final_norm") v = &r->w.final_norm;
  else if (n == "lm_head") v = &r->w.lm_head;
  else if (n.rfind("layers.", 0) == 0) {
    std::size_t dot = n.find('.', 7);
    if (dot == std::string::npos) return nullptr;
    int i = std::stoi(n.substr(7, dot - 7));
    if (i < 0 || i >= static_cast<int>(r->w.layers.size())) return nullptr;
    relay::LayerWeights& L = r->w.layers[i];
    std::string f = n.substr(dot + 1);
    if (f == "attn_norm") v = &L.attn_norm;
    else if (f == "wqkv") v = &L.wqkv;
    else if (f == "bqkv") v = &L.bqkv;
    else if (f == "wo") v = &L.wo;
    else if (f == "mlp_norm") v = &L.mlp_norm;
    else if (f == "w_gate_up") v = &L.w_gate_up;
    else if (f == "w_down") v = &L.w_down;
  }
  if (!v || v->empty()) return nullptr;
  if (numel) *numel = static_cast<long long>(v->size());
  return v->data();
}

int ref_forward(void* h, int n_seqs, const int* tokens, const int* chunk_len, const int* start_pos,
                const int* table_len, const int* tables, const unsigned char* want, int all_logits, float* out,
                std::size_t cap) {
  return guarded([&] {
    Ref* r = static_cast<Ref*>(h);
    relay::ForwardBatch b = to_batch(n_seqs, tokens, chunk_len, start_pos, table_len, tables, want, all_logits);
    std::vector<float> lg = r->be->forward(b);
    if (lg.size() > cap) throw std::invalid_argument("logits buffer too small");
    std::memcpy(out, lg.data(), lg.size() * 4);
    return static_cast<int>(lg.size() / r->w.config.vocab);
  });
}

// forward() with a LayerObserver that records the order of kv_written calls.
int ref_forward_observed(void* h, int n_seqs, const int* tokens, const int* chunk_len, const int* start_pos,
                         const int* table_len, const int* tables, int* layers_seen, int cap_layers) {
  return guarded([&] {
    struct Obs : relay::LayerObserver {
      std::vector<int> seen;
      void kv_written(int l) override { seen.push_back(l); }
    } obs;
    Ref* r = static_cast<Ref*>(h);
    relay::ForwardBatch b = to_batch(n_seqs, tokens, chunk_len, start_pos, table_len, tables, nullptr, 0);
    r->be->forward(b, &obs);
    int n = static_cast<int>(obs.seen.size());
    for (int i = 0; i < n && i < cap_layers; ++i) layers_seen[i] = obs.seen[i];
    return n;
  });
}

std::size_t ref_kv_block_bytes(void* h) { return static_cast<Ref*>(h)->be->kv_block_bytes(); }

int ref_read_kv_block(void* h, int layer, int block, void* k, void* v) {
  return guarded([&] {
    static_cast<Ref*>(h)->be->read_kv_block(layer, block, k, v);
    return 0;
  });
}

int ref_write_kv_block(void* h, int layer, int block, const void* k, const void* v) {
  return guarded([&] {
    static_cast<Ref*>(h)->be->write_kv_block(layer, block, k, v);
    return 0;
  });
}

int ref_rope_inv_freq(const rb200_model_config* cfg, float* out) {
  std::vector<float> f = to_config(*cfg).rope_inv_freq();
  std::memcpy(out, f.data(), f.size() * 4);
  return static_cast<int>(f.size());
}

unsigned short ref_f32_to_f16(float f) { return relay::f32_to_f16(f); }
float ref_f16_to_f32(unsigned short h) { return relay::f16_to_f32(h); }
int ref_argmax(const float* logits, int vocab) { return relay::argmax(logits, vocab); }

// relay's sampler (engine/src/sampler.cpp) on one row of logits: the token it picks for
// (seed, index) and, when lp_out is given, the log-probability Engine reports with it
// (engine/src/engine.cpp:270-282).
int ref_sample(const float* logits, int vocab, float temperature, float top_p, int top_k, unsigned long long seed,
               unsigned long long index, double* lp_out) {
  relay::SamplingParams p;
  p.temperature = temperature;
  p.top_p = top_p;
  p.top_k = top_k;
  p.seed = seed;
  if (lp_out) return relay::sample_with_log_prob(logits, vocab, p, index, lp_out);
  return relay::sample(logits, vocab, p, index);
}
double ref_uniform01(unsigned long long seed, unsigned long long index) { return relay::uniform01(seed, index); }

// OpenMP threads of this library's parallel loops (a launcher may have exported
// OMP_NUM_THREADS=1 to the process); returns the count now in force.
int ref_set_threads(int n) {
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
}

// Greedy generation through relay's own Engine (continuous batching scheduler) on the CPU
// backend: the prompt, then `steps` tokens; writes the tokens and each step's logits.
int ref_generate_greedy(void* h, const int* prompt, int n_prompt, int steps, int* tokens_out, float* logits_out) {
  return guarded([&] {
    Ref* r = static_cast<Ref*>(h);
    relay::Engine engine(*r->be, {512, 8});
    const int V = r->w.config.vocab;
    int seen = 0;
    engine.on_logits = [&](std::uint64_t, int, const float* lg) {
      if (logits_out && seen < steps) std::memcpy(logits_out + static_cast<std::size_t>(seen) * V, lg, V * 4);
      ++seen;
    };
    relay::SamplingParams sp;
    sp.max_new_tokens = steps;
    sp.ignore_eos = true;
    engine.add({1, std::vector<int>(prompt, prompt + n_prompt), sp});
    auto out = engine.run_all();
    const std::vector<int>& g = out[1];
    for (std::size_t i = 0; i < g.size(); ++i) tokens_out[i] = g[i];
    return static_cast<int>(g.size());
  });
}

}  // extern "C"
