// Internal launch interface between the kernels (small_ops.cu, attention.cu, gemm.cu) and
// the backend that sequences them (backend.cu). Everything here enqueues on a stream and
// returns; callers check cudaGetLastError().
#pragma once

#include <algorithm>

#include "common.cuh"

namespace rb200 {

// Where each token of the flattened batch sits: position pos[t] of sequence seq[t], whose
// block ids start at tables[table_off[seq[t]]] (engine/src/cuda_kernels.cuh:16-26).
struct TokenMeta {
  const int* pos;
  const int* seq;
  const int* table_off;
  const int* tables;
};

struct AttnShape {
  int heads, kv_heads, D, block_size;
  int q_stride;  // floats between tokens' q rows
  int o_stride;  // halves between tokens' output rows
  // Rows ([block][kv head][slot]) of one layer's pool, when the caller knows them (the backend
  // does; the operator entry points do not): the TMA descriptors of the tcgen05 prefill kernel
  // then end where the pool ends, so a page the block table should not name reads as zeros
  // instead of memory behind the pool. 0: unknown.
  long long pool_rows = 0;
};

constexpr int kDecodeSlice = RB200_DECODE_SLICE;  // keys per split-context CTA
constexpr int kPrefillRows = RB200_PREFILL_ROWS;  // query rows per prefill tile

// ---- small_ops.cu ----
void launch_embed(const int* tokens, const __half* table, float* x, int T, int H, int ld_table, cudaStream_t st);
// Where a kernel ahead of an int8 linear may leave the activation rows as int8 digits
// (i8_digits.cuh); null members: nobody does, the linear makes them itself.
struct I8Digits {
  int8_t* digits = nullptr;
  float* tscale = nullptr;
};
// `dg` (from linear_digits_dest for the linear that reads `out` next): also write the rows as digits.
void launch_rmsnorm(const float* x, const int* rows, const float* w, __half* out, int R, int H, int ld_out, float eps,
                    cudaStream_t st, I8Digits dg = {});
void launch_qkv_post(float* qkv, const float* bias, const float* inv_freq, const TokenMeta& m, int T, __half* kc,
                     __half* vc, int heads, int kv_heads, int D, int block_size, cudaStream_t st);
// `dg` (from linear_digits_dest for the linear that reads `act` next; needs I a multiple of 4 and
// ld_act of 32): also write the rows as digits.
void launch_silu_mul(const float* gu, __half* act, int T, int I, int ld_act, cudaStream_t st, I8Digits dg = {});
void launch_f32_to_f16(const float* in, __half* out, size_t n, cudaStream_t st);
void launch_convert_rows_f16(const float* in, __half* out, int rows, int K, int ld, cudaStream_t st);
void launch_quantize_rows_int8(const float* in, int8_t* out, float* scale, int rows, int K, int ld, cudaStream_t st);
void launch_kv_gather(const void* k, const void* v, const int* blocks, int n, size_t block_bytes, void* staging,
                      cudaStream_t st);
void launch_kv_scatter(void* k, void* v, const int* blocks, int n, size_t block_bytes, const void* staging,
                       cudaStream_t st);
void launch_argmax_rows(const float* logits, int R, int V, int* token_out, float* logit_out, cudaStream_t st);

// ---- sampler.cu ----
// True when these parameters ask for top-k or nucleus truncation (temperature > 0 and top_k in
// (0, V) or top_p < 1). `params` of launch_sample_rows is a device array, one per row;
// `any_truncated`: some row may be truncated, so the second kernel (which takes those rows) is
// launched behind the first.
bool sampling_truncated(const rb200_sampling_params& p, int V);
void launch_sample_rows(const float* logits, int R, int V, const rb200_sampling_params* params, int* token_out,
                        double* logprob_out, cudaStream_t st, bool any_truncated);

// ---- attention.cu ----
// True when the tensor-core decode / prefill kernels cover this head layout; otherwise the
// backend routes every token through launch_reference_attention.
bool fast_attention_supported(const AttnShape& s);
// Upper bound of the split decode's partial results (512-key slices), for sizing a buffer once.
size_t decode_scratch_bytes(const AttnShape& s, int n_decode, int max_ctx);
// What launch_decode_attention does with a batch: keys per slice, slices per context, and the
// bytes of partial results it parks in its scratch (0 with one slice).
struct DecodePlan {
  int slice = 0, parts = 0;
  bool cluster_merge = false;  // the slices of a (token, KV head) run as one cluster and merge on chip
  size_t scratch_bytes = 0;
};
DecodePlan plan_decode(const AttnShape& s, int n_decode, int max_ctx);
void launch_decode_attention(const AttnShape& s, const float* q, const TokenMeta& m, const int* decode_tokens,
                             int n_decode, int max_ctx, const __half* kc, const __half* vc, float* scratch,
                             __half* out, cudaStream_t st);
void launch_prefill_attention(const AttnShape& s, const float* q, const TokenMeta& m, const int2* tiles, int n_tiles,
                              const __half* kc, const __half* vc, __half* out, cudaStream_t st);
void launch_reference_attention(const AttnShape& s, const float* q, const TokenMeta& m, int T, const __half* kc,
                                const __half* vc, __half* out, cudaStream_t st);

// ---- gemm.cu ----
// A weight matrix [N][ld] in device memory: fp16, or int8 with one fp32 scale per row.
// ld >= K is the row stride in elements; columns K..ld-1 hold zeros.
struct WeightView {
  const __half* f16 = nullptr;
  const int8_t* i8 = nullptr;
  const float* scale = nullptr;
  int N = 0, K = 0, ld = 0;
};
// Scratch of the few-token kernels for an [N][K] matrix: split-K counters and partials of the
// register GEMV, then room for `max_tokens` activation rows as int8 digits (umma_i8_gemm.cu).
size_t gemv_scratch_bytes(int N, int K, int max_tokens = 8);
// y[T,N] = x[T,K] W^T (+ beta*y); routes T <= 8 to the GEMV and larger T to the GEMM.
// `digits_ready`: the kernel ahead has written the rows of x as digits where
// linear_digits_dest(same arguments) said (non-null result only).
void launch_linear(const WeightView& W, const __half* x, int ldx, float* y, int T, float beta, void* scratch,
                   size_t scratch_bytes, cudaStream_t st, bool digits_ready = false);
I8Digits linear_digits_dest(const WeightView& W, const __half* x, int ldx, int T, void* scratch, size_t scratch_bytes);
void launch_gemv(const WeightView& W, const __half* x, int ldx, float* y, int T, float beta, void* scratch,
                 size_t scratch_bytes, cudaStream_t st, bool digits_ready = false);
// `scratch` (may be null) is the buffer gemv_scratch_bytes(N, K, 64) sizes; without it the int8
// path for up to 64 tokens takes its digit buffer from the stream's memory pool.
void launch_gemm(const WeightView& W, const __half* x, int ldx, float* y, int T, float beta, cudaStream_t st,
                 void* scratch = nullptr, size_t scratch_bytes = 0, bool digits_ready = false);
// The same product with legacy mma.sync tiles (any alignment); launch_gemm prefers the
// tcgen05 kernel of umma_gemm.cu and falls back to this one.
void launch_gemm_mma_sync(const WeightView& W, const __half* x, int ldx, float* y, int T, float beta, cudaStream_t st);

// ---- umma_prefill.cu ----
// The tcgen05 flash prefill kernel covers head sizes 64 and 128 with an even number of query
// heads per KV head and block sizes that are multiples of 16; launch_prefill_attention
// prefers it and keeps prefill_flash_kernel (mma.sync) for everything else.
bool umma_prefill_usable(const AttnShape& s, const float* q, const __half* kc, const __half* vc, const __half* out);
void launch_umma_prefill(const AttnShape& s, const float* q, const TokenMeta& m, const int2* tiles, int n_tiles,
                         const __half* kc, const __half* vc, __half* out, cudaStream_t st);

// ---- umma_gemm.cu ----
bool umma_gemm_usable(const WeightView& W, const __half* x, int ldx);
void launch_umma_gemm(const WeightView& W, const __half* x, int ldx, float* y, int T, float beta, cudaStream_t st);
// 0, or the code a bounded pipeline wait of a tcgen05 kernel left on the current device. The
// word is sticky: it keeps the code until umma_status_clear() zeroes it.
int umma_gemm_status();
// The status word's device address (one int per device), for callers that read it back in a
// copy of their own, and its reset, enqueued on `st`.
const int* umma_status_word();
void umma_status_clear(cudaStream_t st);

// ---- umma_i8_gemm.cu ----
// int8 weights x up to 64 tokens on the integer tensor cores: the activations are rewritten
// as three int8 digits per element into `scratch` (i8_digits_bytes(T, K) bytes, 16-byte
// aligned) by a first kernel, the second multiplies the raw int8 weight tiles by them.
size_t i8_digits_bytes(int T, int K);
bool umma_i8_usable(const WeightView& W, const __half* x, int ldx, int T);
// Up to this many tokens the GEMM makes the digits itself and `scratch` may be null (0 when
// RB200_I8_FUSED=0 turns that off).
int umma_i8_fused_tokens();
// `digits_ready`: `scratch` already holds the digits and token scales of x (no pass over x).
void launch_umma_i8(const WeightView& W, const __half* x, int ldx, float* y, int T, float beta, void* scratch, cudaStream_t st,
                    bool digits_ready = false);
// The token scales' place behind the three digit planes of a buffer of i8_digits_bytes(T, K).
float* i8_tscale(int8_t* digits, int T, int K);

}  // namespace rb200
