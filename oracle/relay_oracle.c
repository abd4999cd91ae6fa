/* TEST INFRASTRUCTURE — see relay_oracle.h. A plain-C restatement of relay's float32 CPU
 * algorithm for the per-token compute path. Written from the behaviour of the reference
 * lines cited at each function; it shares no code with them. Every floating-point
 * expression keeps the reference's operand order so that, compiled with the same flags,
 * the results are bit-identical to relay's CPU backend (tests/test_oracle.py checks that).
 */
#include "relay_oracle.h"

#include <math.h>
#include <omp.h>
#include <stdlib.h>
#include <string.h>

/* ---- fp16 <-> fp32 (engine/src/safetensors.cpp:38-88) -------------------------------- */

static uint32_t bits_of(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}

static float float_of(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* Round to nearest, ties to even, with subnormals, overflow to infinity and NaN kept NaN
 * (quiet bit set), as the reference's f32_to_f16 does. */
uint16_t ro_f32_to_f16(float f) {
  const uint32_t u = bits_of(f);
  const uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
  const uint32_t absu = u & 0x7FFFFFFFu;
  if (absu >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | (absu > 0x7F800000u ? 0x200u : 0u));
  if (absu >= 0x47800000u) return (uint16_t)(sign | 0x7C00u); /* >= 65536: past the largest half even before rounding */
  if (absu < 0x33000000u) return sign;                        /* < 2^-25: rounds to zero */
  const int e = (int)(absu >> 23) - 127;                      /* unbiased exponent */
  uint32_t mant = (absu & 0x7FFFFFu) | 0x800000u;             /* 24-bit significand */
  int drop = e >= -14 ? 13 : 13 + (-14 - e);                  /* bits that fall off the end */
  uint32_t kept = mant >> drop;
  const uint32_t rest = mant & ((1u << drop) - 1u), halfway = 1u << (drop - 1);
  if (rest > halfway || (rest == halfway && (kept & 1u))) ++kept;
  if (e >= -14) {
    /* kept has the implicit bit at position 10; adding the biased exponent minus one lets a
     * carry out of the mantissa bump the exponent (and reach infinity) by itself. */
    return (uint16_t)(sign | (uint16_t)(((uint32_t)(e + 15 - 1) << 10) + kept));
  }
  return (uint16_t)(sign | kept); /* subnormal (a carry makes the smallest normal) */
}

float ro_f16_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  const uint32_t e = (h >> 10) & 0x1Fu, m = h & 0x3FFu;
  if (e == 0x1Fu) return float_of(sign | 0x7F800000u | (m << 13));
  if (e != 0) return float_of(sign | ((e + 112u) << 23) | (m << 13));
  if (m == 0) return float_of(sign);
  /* subnormal: m * 2^-24, exact in float */
  float v = (float)m * 5.9604644775390625e-08f;
  return (sign ? -v : v);
}

void ro_round_to_f16(const float* in, float* out, size_t n) {
  for (size_t i = 0; i < n; ++i) out[i] = ro_f16_to_f32(ro_f32_to_f16(in[i]));
}

/* ---- dot / matmul / rmsnorm (engine/src/cpu_backend.cpp:20-52) ------------------------ */

/* Eight running sums over k = l (mod 8), combined pairwise in a fixed tree, plus a scalar
 * tail: the order is part of the contract (same bits for any batch or thread count). */
float ro_dot(const float* a, const float* b, int n) {
  float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int i = 0;
  for (; i + 8 <= n; i += 8)
    for (int l = 0; l < 8; ++l) s[l] += a[i + l] * b[i + l];
  float tail = 0;
  for (; i < n; ++i) tail += a[i] * b[i];
  return ((s[0] + s[1]) + (s[2] + s[3])) + ((s[4] + s[5]) + (s[6] + s[7])) + tail;
}

void ro_matmul(const float* x, const float* W, float* y, int T, int K, int N, int accumulate) {
#pragma omp parallel for schedule(static)
  for (int nb = 0; nb < N; nb += 16) {
    const int ne = nb + 16 < N ? nb + 16 : N;
    for (int t = 0; t < T; ++t) {
      const float* xt = x + (int64_t)t * K;
      float* yt = y + (int64_t)t * N;
      for (int n = nb; n < ne; ++n) {
        float v = ro_dot(xt, W + (int64_t)n * K, K);
        yt[n] = accumulate ? yt[n] + v : v;
      }
    }
  }
}

/* Sum of squares in double; inv = 1 / sqrtf(float(sum / n) + eps); out = w * (x * inv). */
void ro_rmsnorm(const float* x, const float* w, float* out, int n, float eps) {
  double ss = 0;
  for (int i = 0; i < n; ++i) ss += (double)x[i] * x[i];
  const float inv = 1.0f / sqrtf((float)(ss / n) + eps);
  for (int i = 0; i < n; ++i) out[i] = w[i] * (x[i] * inv);
}

/* ---- RoPE (engine/src/config.cpp:79-109, engine/src/cpu_backend.cpp:223-235) ---------- */

int ro_rope_inv_freq(const ro_config* c, float* out) {
  const int half = c->head_dim / 2;
  for (int i = 0; i < half; ++i) {
    float exponent = (float)(2 * i) / (float)c->head_dim;
    out[i] = 1.0f / powf((float)c->rope_theta, exponent);
  }
  if (c->rope_scaling_type == 1) { /* "llama3": long wavelengths divided by factor, a smooth band between */
    const double pi = 3.14159265358979323846;
    const double low_wavelen = c->rope_original_max_position / c->rope_low_freq_factor;
    const double high_wavelen = c->rope_original_max_position / c->rope_high_freq_factor;
    for (int i = 0; i < half; ++i) {
      const float f = out[i];
      const float wavelen = 2.0f * (float)pi / f;
      float scaled = wavelen > low_wavelen ? f / (float)c->rope_factor : f;
      if (!(wavelen < high_wavelen) && !(wavelen > low_wavelen)) {
        float smooth = (float)((c->rope_original_max_position / wavelen - c->rope_low_freq_factor) /
                               (c->rope_high_freq_factor - c->rope_low_freq_factor));
        scaled = (1 - smooth) * f / (float)c->rope_factor + smooth * f;
      }
      out[i] = scaled;
    }
  }
  return half;
}

void ro_rope(float* v, int nheads, int D, int p, const float* inv_freq) {
  const int half = D / 2;
  for (int i = 0; i < half; ++i) {
    float angle = (float)p * inv_freq[i];
    float cs = cosf(angle), sn = sinf(angle);
    for (int h = 0; h < nheads; ++h) {
      float* x = v + h * D;
      float a = x[i], b = x[i + half];
      x[i] = a * cs - b * sn;
      x[i + half] = b * cs + a * sn;
    }
  }
}

/* ---- SwiGLU (engine/src/cpu_backend.cpp:189-194) ------------------------------------- */

void ro_swiglu(const float* gu, float* act, int T, int I) {
#pragma omp parallel for
  for (int t = 0; t < T; ++t) {
    const float* g = gu + (int64_t)t * 2 * I;
    const float* u = g + I;
    float* a = act + (int64_t)t * I;
    for (int i = 0; i < I; ++i) a[i] = g[i] / (1.0f + expf(-g[i])) * u[i];
  }
}

/* ---- paged attention (engine/src/cpu_backend.cpp:153-180) ----------------------------- */

static int64_t page_offset(int block, int kv_heads, int kv_head, int block_size, int slot, int D) {
  /* KVLayout::offset, engine/include/relay/kv_cache.h:32-35 */
  return ((int64_t)block * kv_heads + kv_head) * block_size * D + (int64_t)slot * D;
}

void ro_attention(const float* q, int q_stride, const int32_t* pos, const int32_t* seq, const int32_t* table_off,
                  const int32_t* tables, int T, const float* k_pool, const float* v_pool, int heads, int kv_heads,
                  int D, int block_size, float* out) {
  const float scale = 1.0f / sqrtf((float)D);
  const int group = heads / kv_heads, Q = heads * D;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int t = 0; t < T; ++t) {
    for (int h = 0; h < heads; ++h) {
      const int32_t* table = tables + table_off[seq[t]];
      const float* qv = q + (int64_t)t * q_stride + h * D;
      const int kvh = h / group, n = pos[t] + 1;
      float* score = (float*)malloc(sizeof(float) * (size_t)n);
      float mx = -INFINITY;
      for (int j = 0; j < n; ++j) {
        int64_t off = page_offset(table[j / block_size], kv_heads, kvh, block_size, j % block_size, D);
        score[j] = ro_dot(qv, k_pool + off, D) * scale;
        mx = mx > score[j] ? mx : score[j]; /* std::max(mx, score[j]) */
      }
      float sum = 0;
      for (int j = 0; j < n; ++j) {
        score[j] = expf(score[j] - mx);
        sum += score[j];
      }
      float* o = out + (int64_t)t * Q + h * D;
      for (int d = 0; d < D; ++d) o[d] = 0.0f;
      for (int j = 0; j < n; ++j) {
        int64_t off = page_offset(table[j / block_size], kv_heads, kvh, block_size, j % block_size, D);
        const float* v = v_pool + off;
        float p = score[j] / sum;
        for (int d = 0; d < D; ++d) o[d] += p * v[d];
      }
      free(score);
    }
  }
}

/* ---- bias + RoPE + KV append (engine/src/cpu_backend.cpp:132-147) --------------------- */

void ro_qkv_post(float* qkv, const float* bias, const float* inv_freq, const int32_t* pos, const int32_t* seq,
                 const int32_t* table_off, const int32_t* tables, int T, float* k_pool, float* v_pool, int heads,
                 int kv_heads, int D, int block_size) {
  const int Q = heads * D, KV = kv_heads * D, QKV = Q + 2 * KV;
#pragma omp parallel for
  for (int t = 0; t < T; ++t) {
    float* row = qkv + (int64_t)t * QKV;
    if (bias)
      for (int i = 0; i < QKV; ++i) row[i] += bias[i];
    ro_rope(row, heads, D, pos[t], inv_freq);
    ro_rope(row + Q, kv_heads, D, pos[t], inv_freq);
    const int32_t* table = tables + table_off[seq[t]];
    const int block = table[pos[t] / block_size], slot = pos[t] % block_size;
    for (int h = 0; h < kv_heads; ++h) {
      int64_t off = page_offset(block, kv_heads, h, block_size, slot, D);
      memcpy(k_pool + off, row + Q + h * D, (size_t)D * 4);
      memcpy(v_pool + off, row + Q + KV + h * D, (size_t)D * 4);
    }
  }
}

/* ---- weight-only int8 (engine/src/cuda_backend.cu:282-304, cuda_kernels.cuh:364-427) -- */

void ro_quantize_rows_int8(const float* w, int N, int K, int8_t* q, float* scale) {
#pragma omp parallel for
  for (int n = 0; n < N; ++n) {
    const float* row = w + (int64_t)n * K;
    float mx = 0.0f;
    for (int k = 0; k < K; ++k) {
      float a = fabsf(row[k]);
      mx = mx > a ? mx : a;
    }
    scale[n] = mx > 0.0f ? mx / 127.0f : 1.0f;
    for (int k = 0; k < K; ++k) q[(int64_t)n * K + k] = (int8_t)lrintf(row[k] / scale[n]);
  }
}

/* The reference kernel sums q*x in float32 in a lane-strided order that is not part of its
 * contract (its own test compares it only loosely to fp16); this restatement accumulates
 * in double and rounds once, which every float32 summation order approximates. */
void ro_gemv_int8(const int8_t* q, const float* scale, const float* x, float* y, int T, int K, int N, float beta) {
#pragma omp parallel for
  for (int n = 0; n < N; ++n) {
    const int8_t* row = q + (int64_t)n * K;
    for (int t = 0; t < T; ++t) {
      const float* xt = x + (int64_t)t * K;
      double s = 0;
      for (int k = 0; k < K; ++k) s += (double)row[k] * xt[k];
      float v = (float)s * scale[n];
      float* dst = y + (int64_t)t * N + n;
      *dst = beta != 0.0f ? v + beta * *dst : v;
    }
  }
}

/* ---- LSE merge of decode slices (engine/src/cuda_kernels.cuh:341-362) ------------------ */

void ro_lse_merge(const float* part_o, const float* part_ml, int parts, int D, float* out) {
  float M = -INFINITY;
  for (int p = 0; p < parts; ++p) M = M > part_ml[2 * p] ? M : part_ml[2 * p];
  float L = 0.0f;
  for (int p = 0; p < parts; ++p)
    if (part_ml[2 * p] != -INFINITY) L += expf(part_ml[2 * p] - M) * part_ml[2 * p + 1];
  for (int d = 0; d < D; ++d) {
    float acc = 0.0f;
    for (int p = 0; p < parts; ++p)
      if (part_ml[2 * p] != -INFINITY) acc += expf(part_ml[2 * p] - M) * part_o[(int64_t)p * D + d];
    out[d] = acc / L;
  }
}

/* ---- greedy token (engine/src/sampler.cpp:17-22): strict >, so the lowest id wins ties -- */

int ro_argmax(const float* logits, int vocab) {
  int best = 0;
  for (int i = 1; i < vocab; ++i)
    if (logits[i] > logits[best]) best = i;
  return best;
}

/* ---- KV page moves (engine/src/cuda_backend.cu:257-270) -------------------------------- */

void ro_kv_gather(const uint8_t* k_pool, const uint8_t* v_pool, const int32_t* blocks, int n, size_t block_bytes,
                  uint8_t* staging) {
  for (int i = 0; i < n; ++i) {
    memcpy(staging + (size_t)i * block_bytes, k_pool + (size_t)blocks[i] * block_bytes, block_bytes);
    memcpy(staging + ((size_t)n + i) * block_bytes, v_pool + (size_t)blocks[i] * block_bytes, block_bytes);
  }
}

void ro_kv_scatter(uint8_t* k_pool, uint8_t* v_pool, const int32_t* blocks, int n, size_t block_bytes,
                   const uint8_t* staging) {
  for (int i = 0; i < n; ++i) {
    memcpy(k_pool + (size_t)blocks[i] * block_bytes, staging + (size_t)i * block_bytes, block_bytes);
    memcpy(v_pool + (size_t)blocks[i] * block_bytes, staging + ((size_t)n + i) * block_bytes, block_bytes);
  }
}

/* ---- the whole forward pass (engine/src/cpu_backend.cpp:55-218) ------------------------ */

struct ro_model {
  ro_config c;
  ro_weights w;
  ro_layer* layers;
  int num_blocks, block_size;
  int64_t block_elems, layer_elems;
  float *k, *v, *inv_freq;
};

ro_model* ro_model_new(const ro_config* c, const ro_weights* w, int num_blocks, int block_size) {
  ro_model* m = (ro_model*)calloc(1, sizeof(ro_model));
  m->c = *c;
  m->w = *w;
  m->layers = (ro_layer*)malloc(sizeof(ro_layer) * (size_t)c->layers);
  memcpy(m->layers, w->layers, sizeof(ro_layer) * (size_t)c->layers);
  m->w.layers = m->layers;
  m->num_blocks = num_blocks;
  m->block_size = block_size;
  m->block_elems = (int64_t)c->kv_heads * block_size * c->head_dim;
  m->layer_elems = m->block_elems * num_blocks;
  m->k = (float*)calloc((size_t)(m->layer_elems * c->layers), 4);
  m->v = (float*)calloc((size_t)(m->layer_elems * c->layers), 4);
  m->inv_freq = (float*)malloc(sizeof(float) * (size_t)(c->head_dim / 2 + 1));
  ro_rope_inv_freq(c, m->inv_freq);
  return m;
}

void ro_model_free(ro_model* m) {
  if (!m) return;
  free(m->layers);
  free(m->k);
  free(m->v);
  free(m->inv_freq);
  free(m);
}

size_t ro_kv_block_bytes(const ro_model* m) { return (size_t)m->block_elems * 4; }

void ro_read_kv_block(const ro_model* m, int layer, int block, float* k_out, float* v_out) {
  int64_t off = layer * m->layer_elems + block * m->block_elems;
  memcpy(k_out, m->k + off, (size_t)m->block_elems * 4);
  memcpy(v_out, m->v + off, (size_t)m->block_elems * 4);
}

void ro_write_kv_block(ro_model* m, int layer, int block, const float* k_in, const float* v_in) {
  int64_t off = layer * m->layer_elems + block * m->block_elems;
  memcpy(m->k + off, k_in, (size_t)m->block_elems * 4);
  memcpy(m->v + off, v_in, (size_t)m->block_elems * 4);
}

int ro_forward(ro_model* m, int n_seqs, const int32_t* tokens, const int32_t* chunk_len, const int32_t* start_pos,
               const int32_t* table_len, const int32_t* tables, const uint8_t* want_logits, int all_logits,
               float* logits_out, size_t cap_floats) {
  const ro_config* c = &m->c;
  const int H = c->hidden, D = c->head_dim, Q = c->heads * D, KV = c->kv_heads * D, I = c->intermediate;
  const int QKV = Q + 2 * KV, V = c->vocab, bs = m->block_size;
  int T = 0;
  for (int s = 0; s < n_seqs; ++s) {
    int need = (start_pos[s] + chunk_len[s] + bs - 1) / bs;
    if (table_len[s] < need) return -1;
    T += chunk_len[s];
  }
  if (T == 0) return 0;
  for (int t = 0; t < T; ++t)
    if (tokens[t] < 0 || tokens[t] >= V) return -2;

  int32_t* pos = (int32_t*)malloc(sizeof(int32_t) * (size_t)T);
  int32_t* seq = (int32_t*)malloc(sizeof(int32_t) * (size_t)T);
  int32_t* toff = (int32_t*)malloc(sizeof(int32_t) * (size_t)n_seqs);
  int32_t* rows = (int32_t*)malloc(sizeof(int32_t) * (size_t)T);
  int R = 0;
  for (int s = 0, t = 0, tb = 0; s < n_seqs; ++s) {
    toff[s] = tb;
    tb += table_len[s];
    for (int i = 0; i < chunk_len[s]; ++i, ++t) {
      pos[t] = start_pos[s] + i;
      seq[t] = s;
      if (all_logits) rows[R++] = t;
    }
    if (!all_logits && chunk_len[s] > 0 && (want_logits ? want_logits[s] : 1)) rows[R++] = t - 1;
  }
  if ((size_t)R * V > cap_floats) {
    free(pos); free(seq); free(toff); free(rows);
    return -3;
  }

  float* x = (float*)malloc(sizeof(float) * (size_t)T * H);
  float* xn = (float*)malloc(sizeof(float) * (size_t)T * H);
  float* qkv = (float*)malloc(sizeof(float) * (size_t)T * QKV);
  float* attn = (float*)malloc(sizeof(float) * (size_t)T * Q);
  float* gu = (float*)malloc(sizeof(float) * (size_t)T * 2 * I);
  float* act = (float*)malloc(sizeof(float) * (size_t)T * I);
  for (int t = 0; t < T; ++t) memcpy(x + (int64_t)t * H, m->w.embed + (int64_t)tokens[t] * H, (size_t)H * 4);
  const float eps = (float)c->rms_eps;

  for (int l = 0; l < c->layers; ++l) {
    const ro_layer* L = &m->layers[l];
    float* Kc = m->k + l * m->layer_elems;
    float* Vc = m->v + l * m->layer_elems;
#pragma omp parallel for
    for (int t = 0; t < T; ++t) ro_rmsnorm(x + (int64_t)t * H, L->attn_norm, xn + (int64_t)t * H, H, eps);
    ro_matmul(xn, L->wqkv, qkv, T, H, QKV, 0);
    ro_qkv_post(qkv, L->bqkv, m->inv_freq, pos, seq, toff, tables, T, Kc, Vc, c->heads, c->kv_heads, D, bs);
    ro_attention(qkv, QKV, pos, seq, toff, tables, T, Kc, Vc, c->heads, c->kv_heads, D, bs, attn);
    ro_matmul(attn, L->wo, x, T, Q, H, 1);
#pragma omp parallel for
    for (int t = 0; t < T; ++t) ro_rmsnorm(x + (int64_t)t * H, L->mlp_norm, xn + (int64_t)t * H, H, eps);
    ro_matmul(xn, L->w_gate_up, gu, T, H, 2 * I, 0);
    ro_swiglu(gu, act, T, I);
    ro_matmul(act, L->w_down, x, T, I, H, 1);
  }

  float* xr = (float*)malloc(sizeof(float) * (size_t)(R > 0 ? R : 1) * H);
  for (int r = 0; r < R; ++r) ro_rmsnorm(x + (int64_t)rows[r] * H, m->w.final_norm, xr + (int64_t)r * H, H, eps);
  ro_matmul(xr, m->w.lm_head ? m->w.lm_head : m->w.embed, logits_out, R, H, V, 0);

  free(xr); free(act); free(gu); free(attn); free(qkv); free(xn); free(x);
  free(rows); free(toff); free(seq); free(pos);
  return R;
}

/* ---- the sampler (engine/src/sampler.cpp) ------------------------------------------------ */

/* uniform01 (sampler.cpp:9-15): splitmix64 of (seed, index), 53 random bits. */
double ro_uniform01(uint64_t seed, uint64_t index) {
  uint64_t z = seed + 0x9E3779B97F4A7C15ULL * (index + 1);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  z ^= z >> 31;
  return (double)(z >> 11) * (1.0 / 9007199254740992.0);
}

/* log_prob (sampler.cpp:24-31): log softmax(logits / t)[token] in double; t <= 0 means 1. */
static double log_prob(const float* logits, int vocab, float temperature, int token) {
  const double t = temperature > 0.0f ? temperature : 1.0;
  double mx = logits[0];
  for (int i = 1; i < vocab; ++i) mx = mx > (double)logits[i] ? mx : (double)logits[i];
  double sum = 0;
  for (int i = 0; i < vocab; ++i) sum += exp((logits[i] - mx) / t);
  return (logits[token] - mx) / t - log(sum);
}

static const float* g_sort_logits; /* qsort has no context argument; sampling rows is not re-entrant here */
#pragma omp threadprivate(g_sort_logits)
static int by_logit(const void* a, const void* b) {
  const int ia = *(const int*)a, ib = *(const int*)b;
  if (g_sort_logits[ia] > g_sort_logits[ib]) return -1;
  if (g_sort_logits[ia] < g_sort_logits[ib]) return 1;
  return ia < ib ? -1 : (ia > ib ? 1 : 0); /* ties by id: the order is fully determined */
}

/* sample / sample_with_log_prob (sampler.cpp:33-105). lp_out may be NULL. */
int ro_sample(const float* logits, int vocab, float temperature, float top_p, int top_k, uint64_t seed, uint64_t index,
              double* lp_out) {
  int tok;
  if (!(temperature > 0.0f)) {
    tok = ro_argmax(logits, vocab);
    if (lp_out) *lp_out = log_prob(logits, vocab, temperature, tok);
    return tok;
  }
  if ((top_k <= 0 || top_k >= vocab) && top_p >= 1.0f) {
    /* no truncation: inverse CDF in id order, float terms, double sum (sampler.cpp:35-59) */
    const float inv_t = 1.0f / temperature;
    float mx = logits[0];
    for (int i = 1; i < vocab; ++i) mx = mx > logits[i] ? mx : logits[i];
    float* e = (float*)malloc(sizeof(float) * (size_t)vocab);
    double total = 0;
    for (int i = 0; i < vocab; ++i) total += e[i] = expf((logits[i] - mx) * inv_t);
    double r = ro_uniform01(seed, index) * total;
    tok = vocab - 1;
    for (int i = 0; i < vocab; ++i) {
      r -= e[i];
      if (r < 0) {
        tok = i;
        break;
      }
    }
    if (r >= 0)
      while (tok > 0 && e[tok] == 0.0f) --tok;
    if (lp_out) *lp_out = ((double)logits[tok] - mx) * inv_t - log(total);
    free(e);
    return tok;
  }
  /* candidates in order of decreasing logit, the k best kept (sampler.cpp:77-104) */
  int* ids = (int*)malloc(sizeof(int) * (size_t)vocab);
  for (int i = 0; i < vocab; ++i) ids[i] = i;
  const int k = (top_k > 0 && top_k < vocab) ? top_k : vocab;
  g_sort_logits = logits;
  qsort(ids, (size_t)vocab, sizeof(int), by_logit);
  double* prob = (double*)malloc(sizeof(double) * (size_t)k);
  double mx = logits[ids[0]] / temperature, total = 0;
  for (int i = 0; i < k; ++i) total += prob[i] = exp(logits[ids[i]] / temperature - mx);
  int keep = k;
  if (top_p < 1.0f) {
    double cum = 0;
    for (int i = 0; i < k; ++i) {
      cum += prob[i] / total;
      if (cum >= top_p) {
        keep = i + 1;
        break;
      }
    }
  }
  double kept = 0;
  for (int i = 0; i < keep; ++i) kept += prob[i];
  double r = ro_uniform01(seed, index) * kept;
  tok = ids[keep - 1];
  for (int i = 0; i < keep; ++i) {
    r -= prob[i];
    if (r < 0) {
      tok = ids[i];
      break;
    }
  }
  free(prob);
  free(ids);
  if (lp_out) *lp_out = log_prob(logits, vocab, temperature, tok);
  return tok;
}

int ro_set_threads(int n) {
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
}
