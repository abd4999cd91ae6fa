/* TEST INFRASTRUCTURE — a plain-C restatement of relay's float32 CPU algorithm for the
 * per-token compute path, used only as the checker by tests/, __graft_entry__.smoke() and
 * bench.py's cpu_baseline / reference legs. The product (relay_b200/) never links, loads
 * or calls it. Each function names the reference lines it restates.
 *
 * Parity status: PINNED. tests/test_oracle.py checks it (a) against the transformers
 * logits of the reference's five tiny-model fixtures (tests/golden/, converted from
 * tests/fixtures of the reference), (b) against relay's own CPU backend compiled from its
 * sources (oracle/_ref, where present) bit for bit, and (c) against the reference's
 * fp16 round-trip known answers.
 */
#ifndef RELAY_ORACLE_H
#define RELAY_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Same field order as rb200_model_config (include/relay_b200.h). */
typedef struct ro_config {
  int32_t hidden, intermediate, layers, heads, kv_heads, head_dim, vocab, max_position;
  double rms_eps, rope_theta;
  int32_t rope_scaling_type;
  double rope_factor, rope_low_freq_factor, rope_high_freq_factor, rope_original_max_position;
  int32_t tie_embeddings, qkv_bias;
} ro_config;

typedef struct ro_layer {
  const float *attn_norm, *wqkv, *bqkv, *wo, *mlp_norm, *w_gate_up, *w_down;
} ro_layer;

typedef struct ro_weights {
  const float *embed, *final_norm, *lm_head;
  const ro_layer* layers;
} ro_weights;

/* engine/src/safetensors.cpp:38-88 */
uint16_t ro_f32_to_f16(float f);
float ro_f16_to_f32(uint16_t h);
void ro_round_to_f16(const float* in, float* out, size_t n); /* out = f16_to_f32(f32_to_f16(in)) */

/* engine/src/cpu_backend.cpp:20-28, 31-45, 47-52 */
float ro_dot(const float* a, const float* b, int n);
void ro_matmul(const float* x, const float* W, float* y, int T, int K, int N, int accumulate);
void ro_rmsnorm(const float* x, const float* w, float* out, int n, float eps);

/* engine/src/config.cpp:79-109 */
int ro_rope_inv_freq(const ro_config* c, float* out);
/* engine/src/cpu_backend.cpp:223-235: rotate pairs (i, i + D/2) of nheads heads at position p */
void ro_rope(float* v, int nheads, int D, int p, const float* inv_freq);

/* engine/src/cpu_backend.cpp:189-194 */
void ro_swiglu(const float* gu, float* act, int T, int I);

/* engine/src/cpu_backend.cpp:153-180: causal attention of tokens over a paged fp32 cache.
 * q row of token t, head h: q + t*q_stride + h*D. k_pool/v_pool: one layer,
 * [num_blocks][kv_heads][block_size][D]. out: [T][heads*D]. */
void ro_attention(const float* q, int q_stride, const int32_t* pos, const int32_t* seq, const int32_t* table_off,
                  const int32_t* tables, int T, const float* k_pool, const float* v_pool, int heads, int kv_heads,
                  int D, int block_size, float* out);

/* engine/src/cpu_backend.cpp:136-146: bias, RoPE on q and k, append k and v to the cache. */
void ro_qkv_post(float* qkv, const float* bias, const float* inv_freq, const int32_t* pos, const int32_t* seq,
                 const int32_t* table_off, const int32_t* tables, int T, float* k_pool, float* v_pool, int heads,
                 int kv_heads, int D, int block_size);

/* engine/src/cuda_backend.cu:282-304 */
void ro_quantize_rows_int8(const float* w, int N, int K, int8_t* q, float* scale);
/* engine/src/cuda_kernels.cuh:364-369, 412-427: y = scale[n] * sum_k q[n,k] x[t,k] + beta*y, fp32 sum */
void ro_gemv_int8(const int8_t* q, const float* scale, const float* x, float* y, int T, int K, int N, float beta);

/* engine/src/cuda_kernels.cuh:341-362: out = sum_p e^(m_p-M) O_p / sum_p e^(m_p-M) l_p over
 * the slices with m_p > -inf. part_o [parts][D], part_ml [parts][2]. */
void ro_lse_merge(const float* part_o, const float* part_ml, int parts, int D, float* out);

/* engine/src/sampler.cpp:17-22 */
int ro_argmax(const float* logits, int vocab);

/* engine/src/cuda_backend.cu:257-270: staging = [K of each block][V of each block] */
void ro_kv_gather(const uint8_t* k_pool, const uint8_t* v_pool, const int32_t* blocks, int n, size_t block_bytes,
                  uint8_t* staging);
void ro_kv_scatter(uint8_t* k_pool, uint8_t* v_pool, const int32_t* blocks, int n, size_t block_bytes,
                   const uint8_t* staging);

/* The whole forward pass, engine/src/cpu_backend.cpp:90-218, over a model that owns an
 * fp32 paged cache [layers][num_blocks][kv_heads][block_size][D]. */
typedef struct ro_model ro_model;
ro_model* ro_model_new(const ro_config* c, const ro_weights* w, int num_blocks, int block_size);
void ro_model_free(ro_model* m);
/* Returns rows written to logits_out ([rows][vocab]), or -1: block table too short (-1),
 * token id out of range (-2), logits buffer too small (-3). */
int ro_forward(ro_model* m, int n_seqs, const int32_t* tokens, const int32_t* chunk_len, const int32_t* start_pos,
               const int32_t* table_len, const int32_t* tables, const uint8_t* want_logits, int all_logits,
               float* logits_out, size_t cap_floats);
size_t ro_kv_block_bytes(const ro_model* m);
void ro_read_kv_block(const ro_model* m, int layer, int block, float* k_out, float* v_out);
void ro_write_kv_block(ro_model* m, int layer, int block, const float* k_in, const float* v_in);

/* engine/src/sampler.cpp:9-15 and :33-105: the random number of (seed, index); the token
 * sample() picks from one row and, in *lp_out when not NULL, the log-probability
 * sample_with_log_prob() / log_prob() report for it. */
double ro_uniform01(uint64_t seed, uint64_t index);
int ro_sample(const float* logits, int vocab, float temperature, float top_p, int top_k, uint64_t seed, uint64_t index,
              double* lp_out);

/* OpenMP threads of this library's parallel loops (a launcher may have exported
 * OMP_NUM_THREADS=1 to the process); returns the count now in force. */
int ro_set_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
