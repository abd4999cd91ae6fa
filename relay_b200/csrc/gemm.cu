// The linear layers: y[T,N] = x[T,K] W[N,K]^T (+ beta*y), W fp16 or weight-only int8 with
// one fp32 scale per output row, x fp16, y fp32.
//
// Dispatch (launch_linear): fp16 weights go to the tcgen05 kernel of umma_gemm.cu for every
// token count; int8 weights go to the integer tensor-core kernel of umma_i8_gemm.cu up to 16
// tokens (32 on large matrices) and to umma_gemm.cu's int8 instantiation (widening into TMEM)
// above. The two kernels of this file are what remains for operands those cannot take:
//
//  * gemv_kernel (T <= 8) — the register-path form of gemv_int8_kernel
//    (engine/src/cuda_kernels.cuh:378-430), used for matrices under 2 MB, callers without
//    scratch for the digit buffer, and pointers TMA cannot address.
//    Bound by weight bandwidth: every weight byte is read from HBM exactly once, straight
//    into registers with 256-bit loads (the four lanes of a quad cover a whole 128-byte line
//    of a row), int8 spliced under an fp16 exponent with two byte permutes (the constant
//    bias this leaves, 1152 * sum of the activations, is removed once per output), and
//    multiplied on the tensor cores with the 8 tokens on the N axis of m16n8k16, so the
//    arithmetic never competes with the load stream. The k order inside an instruction is
//    permuted (legal for a dot product) so that a lane's 32 contiguous weight bytes feed
//    eight instructions. Small N is split along K across CTAs; the last CTA of a row block to
//    finish adds the partials in a fixed order, so results are deterministic.
//    fp16 weights with up to 8 tokens go to the tcgen05 kernel of umma_gemm.cu (a 16-token
//    tile): TMA streams them faster than per-lane loads do. This kernel keeps an fp16
//    instantiation for operands TMA cannot address.
//  * gemm_kernel (T > 8, mma.sync; RB200_GEMM=mma_sync forces it) — the legacy-tile form of dequant_int8_kernel + cuBLAS (engine/src/cuda_kernels.cuh:432-436,
//    engine/src/cuda_backend.cu:719-721) and cublasGemmEx for fp16 weights: weights on the M
//    axis, tokens on N, int8 dequantised on its way into shared memory (the fp16 copy of the
//    matrix is never materialised in HBM), scale and residual applied in the epilogue.
#include <cstdlib>

#include "kernels.h"

namespace rb200 {

namespace {

// ---- int8 -> fp16 -----------------------------------------------------------------------

// Four signed bytes -> two half2 (exact): flip the sign bit (v + 128 as an unsigned byte),
// splice the byte under the exponent of 1024.0 (0x6400 | b = 1024 + b), subtract 1152.
__device__ __forceinline__ void cvt_s8x4_f16x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t u = w ^ 0x80808080u;
  uint32_t a, b;
  asm("prmt.b32 %0, %1, %2, 0x4140;" : "=r"(a) : "r"(u), "r"(0x64646464u));
  asm("prmt.b32 %0, %1, %2, 0x4342;" : "=r"(b) : "r"(u), "r"(0x64646464u));
  const __half2 bias = __half2half2(__ushort_as_half(0x6480));  // 1152.0
  __half2 ha = __hsub2(*reinterpret_cast<__half2*>(&a), bias);
  __half2 hb = __hsub2(*reinterpret_cast<__half2*>(&b), bias);
  lo = *reinterpret_cast<uint32_t*>(&ha);
  hi = *reinterpret_cast<uint32_t*>(&hb);
}

// 32 bytes per lane in one instruction (sm_100 has 256-bit global loads), streaming cache
// policy; lanes past the end of the k range get zeros.
__device__ __forceinline__ void ld_global_256(uint32_t (&r)[8], const void* p, bool valid) {
  if (valid) {
    asm volatile("ld.global.cs.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "l"(p));
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) r[i] = 0u;
  }
}

// Four signed bytes -> two half2 holding w + 1152 (exact, 1024..1279): the byte, with its
// sign bit flipped, spliced under the exponent of 1024.0. Two instructions cheaper per call
// than cvt_s8x4_f16x4; the caller removes the bias once per output (1152 * sum of x).
__device__ __forceinline__ void cvt_s8x4_biased(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t u = w ^ 0x80808080u;
  asm("prmt.b32 %0, %1, %2, 0x4140;" : "=r"(lo) : "r"(u), "r"(0x64646464u));
  asm("prmt.b32 %0, %1, %2, 0x4342;" : "=r"(hi) : "r"(u), "r"(0x64646464u));
}

// ---- GEMV (T <= 8) -------------------------------------------------------------------------

constexpr int kGemvWarps = 4;            // 16 output rows each
constexpr int kGemvRows = kGemvWarps * 16;
constexpr int kGemvMaxChunk = 1024;      // K values of x staged per CTA

constexpr __host__ __device__ int gemv_x_pad(bool int8) { return int8 ? 8 : 32; }
__host__ __device__ inline int round_up_dev(int a, int b) { return (a + b - 1) / b * b; }

struct GemvPlan {
  int row_blocks, splits, chunk;
};

GemvPlan plan_gemv(int N, int K) {
  GemvPlan p;
  p.row_blocks = div_up(N, kGemvRows);
  // about four resident CTAs per SM in total; k ranges of at most kGemvMaxChunk, shorter
  // (down to 256) only when the rows alone cannot occupy the GPU
  const int slots = 4 * sm_count();
  const int want = std::max(div_up(slots, p.row_blocks), div_up(K, kGemvMaxChunk));
  const int splits = std::max(1, std::min(want, std::max(1, K / 256)));
  p.chunk = round_up(div_up(K, splits), 64);
  p.splits = div_up(K, p.chunk);
  return p;
}

// Scratch: [row_blocks] arrival counters (padded to 256 B), then partials [splits][N][8] floats.
size_t gemv_counter_bytes(int N) { return static_cast<size_t>(round_up(div_up(N, kGemvRows) * 4, 256)); }

// What every GEMV variant does with a warp's accumulator (m16n8: acc[0], acc[1] = row g,
// tokens 2*t4 and 2*t4+1; acc[2], acc[3] = row g + 8): scale, add beta*y and store, or, when
// K is split, park the partial sums and let the last CTA of the row block add them in order.
template <bool INT8>
__device__ __forceinline__ void gemv_finish(const float (&acc)[4], int rb, int split, int splits, int warp, int g, int t4,
                                            int T, int N, const float* __restrict__ scale, float* __restrict__ y,
                                            float beta, unsigned* __restrict__ counters, float* __restrict__ partials,
                                            unsigned* s_last) {
  // acc[0], acc[1]: row g, tokens 2*t4, 2*t4+1; acc[2], acc[3]: row g + 8.
  const int n_a = rb * kGemvRows + warp * 16 + g, n_b = n_a + 8;
  const int tok = 2 * t4;
  auto finish = [&](int n, float v0, float v1) {
    if (n >= N) return;
    const float sc = INT8 ? scale[n] : 1.0f;
    if (tok < T) {
      float* d = y + static_cast<long long>(tok) * N + n;
      *d = beta != 0.f ? v0 * sc + beta * *d : v0 * sc;
    }
    if (tok + 1 < T) {
      float* d = y + static_cast<long long>(tok + 1) * N + n;
      *d = beta != 0.f ? v1 * sc + beta * *d : v1 * sc;
    }
  };
  if (splits == 1) {
    finish(n_a, acc[0], acc[1]);
    finish(n_b, acc[2], acc[3]);
    return;
  }
  // Split K: park this CTA's partial sums, then the last CTA of the row block to arrive
  // adds all of them in split order.
  float* mine = partials + static_cast<long long>(split) * N * 8;
  if (n_a < N) *reinterpret_cast<float2*>(mine + static_cast<long long>(n_a) * 8 + tok) = make_float2(acc[0], acc[1]);
  if (n_b < N) *reinterpret_cast<float2*>(mine + static_cast<long long>(n_b) * 8 + tok) = make_float2(acc[2], acc[3]);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned seen = atomicAdd(&counters[rb], 1u);
    *s_last = seen == static_cast<unsigned>(splits - 1);
    if (*s_last) counters[rb] = 0;  // ready for the next launch
  }
  __syncthreads();
  if (!*s_last) return;
  __threadfence();
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float* p = partials + static_cast<long long>(s) * N * 8;
    if (n_a < N) {
      const float2 v = __ldcg(reinterpret_cast<const float2*>(p + static_cast<long long>(n_a) * 8 + tok));
      s0 += v.x;
      s1 += v.y;
    }
    if (n_b < N) {
      const float2 v = __ldcg(reinterpret_cast<const float2*>(p + static_cast<long long>(n_b) * 8 + tok));
      s2 += v.x;
      s3 += v.y;
    }
  }
  finish(n_a, s0, s1);
  finish(n_b, s2, s3);
}

template <bool INT8>
__global__ void __launch_bounds__(kGemvWarps * 32)
gemv_kernel(const void* __restrict__ wv, const float* __restrict__ scale, const __half* __restrict__ x,
            float* __restrict__ y, int T, int K, int N, int ldw, int ldx, float beta, int chunk, int splits,
            unsigned* __restrict__ counters, float* __restrict__ partials) {
  pdl_trigger();
  pdl_wait();
  // x[8][chunk] halves, each row padded (16 bytes for int8 weights, 64 for fp16) so that the
  // token rows a quarter-warp reads with 16-byte loads fall into different bank groups.
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ unsigned s_last;
  __shared__ float s_xsum[8];  // int8 only: sum of each token's activations over this CTA's k range
  const int xs_stride = round_up_dev(chunk, 128) + gemv_x_pad(INT8);  // halves
  __half* xs = reinterpret_cast<__half*>(smem_raw);

  const int rb = blockIdx.x, split = blockIdx.y;
  const int kb0 = split * chunk, kb1 = min(K, kb0 + chunk);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  constexpr int KB = INT8 ? 128 : 64;  // k values per block: each lane of a quad loads 32 bytes, a full 128-byte line per row
  constexpr int U = 4;                 // 32-byte loads in flight per thread and row

  const int row_a = min(rb * kGemvRows + warp * 16 + g, N - 1);      // clamped: extra rows are never stored
  const int row_b = min(rb * kGemvRows + warp * 16 + g + 8, N - 1);
  const size_t esz = INT8 ? 1 : 2;
  const unsigned char* wa = static_cast<const unsigned char*>(wv) + (static_cast<size_t>(row_a) * ldw + kb0) * esz + 32 * t4;
  const unsigned char* wb = static_cast<const unsigned char*>(wv) + (static_cast<size_t>(row_b) * ldw + kb0) * esz + 32 * t4;
  const int span = (kb1 - kb0) * static_cast<int>(esz);  // bytes of one row this CTA covers (a multiple of 64)
  const int nblk = (span + 127) / 128;

  // Start the weight stream before anything else: the first U blocks are in flight while the
  // activations are staged.
  uint32_t ra[U][8], rbv[U][8];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    if (u < nblk) {
      ld_global_256(ra[u], wa + u * 128, u * 128 + 32 * t4 < span);
      ld_global_256(rbv[u], wb + u * 128, u * 128 + 32 * t4 < span);
    }
  }

  // stage x[:, kb0:kb1) (rows >= T and the tail of the last block are zero)
  const int xcols = round_up_dev(kb1 - kb0, 128);
  float xsum = 0.f;  // this thread's share of its token's sum (idx -> token is fixed per warp pass below)
  if (threadIdx.x < 8) s_xsum[threadIdx.x] = 0.f;
  __syncthreads();
  for (int t = warp; t < 8; t += kGemvWarps) {  // a warp stages whole token rows, so it can sum them too
    xsum = 0.f;
    for (int c = lane; c < xcols / 8; c += 32) {
      uint4 v = make_uint4(0, 0, 0, 0);
      if (t < T && kb0 + c * 8 < kb1) v = *reinterpret_cast<const uint4*>(x + static_cast<long long>(t) * ldx + kb0 + c * 8);
      *reinterpret_cast<uint4*>(xs + t * xs_stride + c * 8) = v;
      if constexpr (INT8) {
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __half22float2(h[i]);
          xsum += f.x + f.y;
        }
      }
    }
    if constexpr (INT8) {
      xsum = warp_sum(xsum);
      if (lane == 0) s_xsum[t] = xsum;
    }
  }
  __syncthreads();

  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const __half* xg = xs + g * xs_stride + (INT8 ? 32 : 16) * t4;
  for (int b0 = 0; b0 < nblk; b0 += U) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int b = b0 + u;
      if (b < nblk) {
        uint32_t wra[8], wrb[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          wra[i] = ra[u][i];
          wrb[i] = rbv[u][i];
        }
        if (b + U < nblk) {  // refill this slot at once: U loads stay in flight
          ld_global_256(ra[u], wa + (b + U) * 128, (b + U) * 128 + 32 * t4 < span);
          ld_global_256(rbv[u], wb + (b + U) * 128, (b + U) * 128 + 32 * t4 < span);
        }
        if constexpr (INT8) {
          uint32_t xb[16];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint4 xv = *reinterpret_cast<const uint4*>(xg + b * KB + 8 * c);
            xb[4 * c] = xv.x;
            xb[4 * c + 1] = xv.y;
            xb[4 * c + 2] = xv.z;
            xb[4 * c + 3] = xv.w;
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {  // four consecutive k per instruction and lane
            uint32_t a[4];
            cvt_s8x4_biased(wra[i], a[0], a[2]);
            cvt_s8x4_biased(wrb[i], a[1], a[3]);
            mma_f16(acc, a, xb[2 * i], xb[2 * i + 1]);
          }
        } else {
          const uint4 x0 = *reinterpret_cast<const uint4*>(xg + b * KB);
          const uint4 x1 = *reinterpret_cast<const uint4*>(xg + b * KB + 8);
          const uint32_t xb[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t a[4] = {wra[2 * i], wrb[2 * i], wra[2 * i + 1], wrb[2 * i + 1]};
            mma_f16(acc, a, xb[2 * i], xb[2 * i + 1]);
          }
        }
      }
    }
  }
  if constexpr (INT8) {
    // The multiplicand fed to the tensor core was w + 1152 (see cvt_s8x4_biased): take the
    // surplus 1152 * sum_k x[t][k] back out, in fp32, per token.
    const float c0 = 1152.0f * s_xsum[2 * t4], c1 = 1152.0f * s_xsum[2 * t4 + 1];
    acc[0] -= c0;
    acc[1] -= c1;
    acc[2] -= c0;
    acc[3] -= c1;
  }
  gemv_finish<INT8>(acc, rb, split, splits, warp, g, t4, T, N, scale, y, beta, counters, partials, &s_last);
}

// ---- GEMV for small int8 matrices (T <= 8) ---------------------------------------------------
//
// A matrix of a few megabytes is read in about a microsecond; what a kernel for it has to avoid
// is everything else: a K split across CTAs (partials through global memory, a counter, a last
// CTA), staging the activations through shared memory behind block barriers, set-up of tensor
// memory and descriptors. Here a CTA owns 16 output rows for the whole of K: its eight warps
// take an eighth of K each, load their weight bytes (32 bytes per lane and row, four blocks in
// flight) BEFORE waiting for the kernel ahead (weights are never written by a forward pass), read
// the activation fragments straight from global memory (a few KB per warp, L1 / L2 resident),
// multiply on m16n8k16 with the tokens on N as gemv_kernel does, and add the partial
// accumulators in warp order through 4 KB of shared memory: one block barrier, no atomics,
// the same sum on every run. WPG = warps that share a group of 16 rows (8, 4 or 2: a CTA then
// owns 16, 32 or 64 rows, and a warp an eighth, a quarter or half of K); the host picks the
// largest WPG whose grid still fits the SMs in one wave of two CTAs each, so that no second
// wave trails behind.
constexpr int kRowsWarps = 8;

template <int WPG>
__global__ void __launch_bounds__(kRowsWarps * 32, 2)
gemv_rows_i8_kernel(const int8_t* __restrict__ w, const float* __restrict__ scale, const __half* __restrict__ x,
                    float* __restrict__ y, int T, int K, int N, int ldw, int ldx, float beta) {
  pdl_trigger();
  __shared__ float red[kRowsWarps][32][4];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  constexpr int U = 4;          // 32-byte loads in flight per lane and row
  constexpr int kGroups = kRowsWarps / WPG;
  const int group = warp / WPG, part = warp % WPG;
  const int kw = K / WPG;  // this warp's k range: a multiple of 128
  const int k0 = part * kw, nblk = kw / 128;
  const int n_a = (blockIdx.x * kGroups + group) * 16 + g, n_b = n_a + 8;
  const unsigned char* wa = reinterpret_cast<const unsigned char*>(w) + static_cast<size_t>(min(n_a, N - 1)) * ldw + k0 + 32 * t4;
  const unsigned char* wb = reinterpret_cast<const unsigned char*>(w) + static_cast<size_t>(min(n_b, N - 1)) * ldw + k0 + 32 * t4;
  uint32_t ra[U][8], rbv[U][8];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    if (u < nblk) {
      ld_global_256(ra[u], wa + u * 128, true);
      ld_global_256(rbv[u], wb + u * 128, true);
    }
  }
  // the row scales are weights too; what y holds (read with beta) is fetched right behind the wait,
  // so that neither is a round trip to memory after the last multiply
  const float sc_a = scale[min(n_a, N - 1)], sc_b = scale[min(n_b, N - 1)];
  pdl_wait();  // x and y belong to the kernels ahead until they complete
  const int tok = 2 * t4;
  float old[4] = {0.f, 0.f, 0.f, 0.f};  // y at (tok, n_a), (tok + 1, n_a), (tok, n_b), (tok + 1, n_b)
  if (part == 0 && beta != 0.f) {
    if (n_a < N && tok < T) old[0] = y[static_cast<long long>(tok) * N + n_a];
    if (n_a < N && tok + 1 < T) old[1] = y[static_cast<long long>(tok + 1) * N + n_a];
    if (n_b < N && tok < T) old[2] = y[static_cast<long long>(tok) * N + n_b];
    if (n_b < N && tok + 1 < T) old[3] = y[static_cast<long long>(tok + 1) * N + n_b];
  }
  // token g's 32 activations of a block, at the same k as this lane's 32 weight bytes
  const __half* xg = x + static_cast<long long>(min(g, T - 1)) * ldx + k0 + 32 * t4;
  const bool tok_live = g < T;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int b0 = 0; b0 < nblk; b0 += U) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int b = b0 + u;
      if (b < nblk) {
        // two mma per 16-byte piece of the token's activations, so only four registers of x are live
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint4 xv = make_uint4(0u, 0u, 0u, 0u);
          if (tok_live) xv = __ldg(reinterpret_cast<const uint4*>(xg + b * 128 + 8 * c));
          uint32_t a[4];
          cvt_s8x4_f16x4(ra[u][2 * c], a[0], a[2]);
          cvt_s8x4_f16x4(rbv[u][2 * c], a[1], a[3]);
          mma_f16(acc, a, xv.x, xv.y);
          cvt_s8x4_f16x4(ra[u][2 * c + 1], a[0], a[2]);
          cvt_s8x4_f16x4(rbv[u][2 * c + 1], a[1], a[3]);
          mma_f16(acc, a, xv.z, xv.w);
        }
        if (b + U < nblk) {  // refill the slot: U loads stay in flight
          ld_global_256(ra[u], wa + (b + U) * 128, true);
          ld_global_256(rbv[u], wb + (b + U) * 128, true);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) red[warp][lane][i] = acc[i];
  __syncthreads();
  if (part != 0) return;
  float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int wv = 0; wv < WPG; ++wv)
#pragma unroll
    for (int i = 0; i < 4; ++i) s[i] += red[group * WPG + wv][lane][i];
  // s[0], s[1]: row n_a, tokens 2 t4 and 2 t4 + 1; s[2], s[3]: row n_b
  auto finish = [&](int n, float sc, float v0, float v1, float o0, float o1) {
    if (n >= N) return;
    if (tok < T) y[static_cast<long long>(tok) * N + n] = beta != 0.f ? v0 * sc + beta * o0 : v0 * sc;
    if (tok + 1 < T) y[static_cast<long long>(tok + 1) * N + n] = beta != 0.f ? v1 * sc + beta * o1 : v1 * sc;
  };
  finish(n_a, sc_a, s[0], s[1], old[0], old[1]);
  finish(n_b, sc_b, s[2], s[3], old[2], old[3]);
}

// ---- GEMM (T > 8) --------------------------------------------------------------------------

constexpr int kBM = 128;  // weight rows per CTA
constexpr int kBN = 64;   // tokens per CTA
constexpr int kBK = 64;   // k per shared-memory tile (128-byte fp16 rows)

template <bool INT8>
__global__ void __launch_bounds__(256)
gemm_kernel(const void* __restrict__ wv, const float* __restrict__ scale, const __half* __restrict__ x,
            float* __restrict__ y, int T, int K, int N, int ldw, int ldx, float beta) {
  // two stages of: A tile [kBM][kBK] fp16, B tile [kBN][kBK] fp16, both swizzled (8 chunks per row)
  __shared__ __align__(128) __half sA[2][kBM * kBK];
  __shared__ __align__(128) __half sB[2][kBN * kBK];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
  const int wm = warp >> 1, wn = warp & 1;  // 4 x 2 warps, each 32 rows x 32 tokens
  const int n0 = blockIdx.x * kBM, tok0 = blockIdx.y * kBN;

  // Global -> register prefetch of one k tile; int8 weights are widened on the way to shared memory.
  uint4 ra[INT8 ? 2 : 4];
  uint4 rx[2];
  auto fetch = [&](int kt) {
    const int k0 = kt * kBK;
    if constexpr (INT8) {
      // 128 rows x 64 bytes: thread -> row tid/2, 32-byte half (tid & 1)
      const int r = tid >> 1, h = tid & 1;
      const int8_t* src = static_cast<const int8_t*>(wv) + static_cast<long long>(min(n0 + r, N - 1)) * ldw + k0 + h * 32;
      ra[0] = *reinterpret_cast<const uint4*>(src);
      ra[1] = *reinterpret_cast<const uint4*>(src + 16);
    } else {
      // 128 rows x 128 bytes: thread -> row tid/2, 64-byte half
      const int r = tid >> 1, h = tid & 1;
      const __half* src = static_cast<const __half*>(wv) + static_cast<long long>(min(n0 + r, N - 1)) * ldw + k0 + h * 32;
#pragma unroll
      for (int i = 0; i < 4; ++i) ra[i] = *reinterpret_cast<const uint4*>(src + i * 8);
    }
    // x: 64 tokens x 128 bytes: thread -> token tid/4, 32-byte quarter
    const int r = tid >> 2, qd = tid & 3;
    if (tok0 + r < T) {
      const __half* src = x + static_cast<long long>(tok0 + r) * ldx + k0 + qd * 16;
      rx[0] = *reinterpret_cast<const uint4*>(src);
      rx[1] = *reinterpret_cast<const uint4*>(src + 8);
    } else {
      rx[0] = rx[1] = make_uint4(0, 0, 0, 0);
    }
  };
  auto stash = [&](int stage) {
    const int r = tid >> 1, h = tid & 1;
    uint4* a = reinterpret_cast<uint4*>(sA[stage]);
    if constexpr (INT8) {
      const uint32_t w8[8] = {ra[0].x, ra[0].y, ra[0].z, ra[0].w, ra[1].x, ra[1].y, ra[1].z, ra[1].w};
#pragma unroll
      for (int c = 0; c < 4; ++c) {  // 8 weights per 16-byte fp16 chunk
        uint4 o;
        cvt_s8x4_f16x4(w8[2 * c], o.x, o.y);
        cvt_s8x4_f16x4(w8[2 * c + 1], o.z, o.w);
        a[swz<8>(r, h * 4 + c)] = o;
      }
    } else {
#pragma unroll
      for (int c = 0; c < 4; ++c) a[swz<8>(r, h * 4 + c)] = ra[c];
    }
    const int rr = tid >> 2, qd = tid & 3;
    uint4* b = reinterpret_cast<uint4*>(sB[stage]);
    b[swz<8>(rr, qd * 2)] = rx[0];
    b[swz<8>(rr, qd * 2 + 1)] = rx[1];
  };

  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;

  const int nkt = K / kBK;
  fetch(0);
  stash(0);
  __syncthreads();
  for (int kt = 0; kt < nkt; ++kt) {
    const int stage = kt & 1;
    if (kt + 1 < nkt) fetch(kt + 1);
    const uint32_t a_base = smem_u32(sA[stage]), b_base = smem_u32(sB[stage]);
#pragma unroll
    for (int ks = 0; ks < kBK / 16; ++ks) {
      uint32_t af[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        // A fragment of rows wm*32 + i*16 ..: matrices (rows 0-7, k lo), (rows 8-15, k lo), (rows 0-7, k hi), (rows 8-15, k hi)
        const int row = wm * 32 + i * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
        ldmatrix_x4(af[i], a_base + swz<8>(row, 2 * ks + (lane >> 4)) * 16);
      }
#pragma unroll
      for (int jp = 0; jp < 2; ++jp) {
        uint32_t bf[4];
        const int row = wn * 32 + jp * 16 + (lane & 7) + ((lane >> 4) << 3);
        ldmatrix_x4(bf, b_base + swz<8>(row, 2 * ks + ((lane >> 3) & 1)) * 16);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          mma_f16(acc[i][2 * jp], af[i], bf[0], bf[1]);
          mma_f16(acc[i][2 * jp + 1], af[i], bf[2], bf[3]);
        }
      }
    }
    if (kt + 1 < nkt) stash(stage ^ 1);
    __syncthreads();
  }

  // epilogue: acc[i][j][0,1] = (row g, tokens 2*t4, +1), [2,3] = row g + 8
#pragma unroll
  for (int i = 0; i < 2; ++i) {
#pragma unroll
    for (int hrow = 0; hrow < 2; ++hrow) {
      const int n = n0 + wm * 32 + i * 16 + g + hrow * 8;
      if (n >= N) continue;
      const float sc = INT8 ? scale[n] : 1.0f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int tok = tok0 + wn * 32 + j * 8 + 2 * t4 + e;
          if (tok >= T) continue;
          float* d = y + static_cast<long long>(tok) * N + n;
          const float v = acc[i][j][hrow * 2 + e] * sc;
          *d = beta != 0.f ? v + beta * *d : v;
        }
      }
    }
  }
}

}  // namespace

static size_t gemv_partials_bytes(int N, int K) {
  const int splits = plan_gemv(N, K).splits;
  const size_t bytes = gemv_counter_bytes(N) + (splits > 1 ? static_cast<size_t>(splits) * N * 8 * sizeof(float) : 0);
  return (bytes + 255) / 256 * 256;
}

size_t gemv_scratch_bytes(int N, int K, int max_tokens) {
  return gemv_partials_bytes(N, K) + i8_digits_bytes(max_tokens, K);
}

// The digits of an int8 linear sit at the END of the caller's scratch (256-byte aligned), the
// register GEMV's counters and partials at its start: a buffer shared by several matrices (sized
// for the largest of each) never has one matrix's digits on top of another's counters.
static size_t digits_offset(size_t scratch_bytes, int T, int K) {
  return (scratch_bytes - i8_digits_bytes(T, K)) / 256 * 256;
}

// int8 weights with few tokens: the integer tensor-core kernel once the matrix is large enough
// to pay for its activation pass (a second small launch); smaller ones stay on the register GEMV.
static bool i8_digits_preferred(const WeightView& W) {
  static const long long min_bytes = [] {
    const char* e = std::getenv("RB200_I8_MIN_MB");
    return (e ? std::atoll(e) : 2) << 20;
  }();
  return static_cast<long long>(W.N) * W.K >= min_bytes;
}

// Up to umma_i8_fused_tokens() tokens the kernel can make the digits itself (every CTA then reads
// the activation rows for their largest magnitude). Measured against the separate digit pass it
// wins where a CTA streams much more weight data than activations: 58.7 MB, 1 / 2 / 4 tokens,
// K = 4096: 12.1 / 12.4 / 12.7 us against 13.0 / 13.1 / 13.2; K = 14336: 13.2 / 14.0 / 15.6 against
// 13.5 / 14.2 / 15.2; 16.8 MB (K split over a cluster of four): 7.0 against 6.5.
static bool i8_fused_preferred(const WeightView& W, int T) {
  return T <= umma_i8_fused_tokens() && static_cast<long long>(W.N) * W.K >= (32ll << 20) && static_cast<long long>(T) * W.K <= 32768;
}

// Small int8 matrices with up to 8 tokens: gemv_rows_i8_kernel (no K split across CTAs, no set-up).
// RB200_I8_ROWS_MB: the largest matrix (MB) that takes it; 0 turns it off.
static bool i8_rows_preferred(const WeightView& W, int T) {
  static const long long max_bytes = [] {
    const char* e = std::getenv("RB200_I8_ROWS_MB");
    return (e ? std::atoll(e) : 20) << 20;
  }();
  return W.i8 != nullptr && T >= 1 && T <= 8 && W.K % (kRowsWarps * 128) == 0 && static_cast<long long>(W.N) * W.K <= max_bytes &&
         W.ld % 32 == 0 && (reinterpret_cast<uintptr_t>(W.i8) & 31) == 0;
}

static void launch_gemv_rows_i8(const WeightView& W, const __half* x, int ldx, float* y, int T, float beta, cudaStream_t st) {
  // rows per CTA: 16 unless that needs more CTAs than fit the SMs at once (two per SM by registers)
  const int slots = 2 * sm_count();
  count_launch();
  if (div_up(W.N, 16) <= slots)
    launch_pdl(gemv_rows_i8_kernel<8>, dim3(div_up(W.N, 16)), dim3(kRowsWarps * 32), 0, st, W.i8, W.scale, x, y, T, W.K, W.N, W.ld, ldx, beta);
  else if (div_up(W.N, 32) <= slots)
    launch_pdl(gemv_rows_i8_kernel<4>, dim3(div_up(W.N, 32)), dim3(kRowsWarps * 32), 0, st, W.i8, W.scale, x, y, T, W.K, W.N, W.ld, ldx, beta);
  else
    launch_pdl(gemv_rows_i8_kernel<2>, dim3(div_up(W.N, 64)), dim3(kRowsWarps * 32), 0, st, W.i8, W.scale, x, y, T, W.K, W.N, W.ld, ldx, beta);
}

static bool gemm_forced_legacy() {
  static const bool v = [] {
    const char* e = std::getenv("RB200_GEMM");
    return e && std::string(e) == "mma_sync";
  }();
  return v;
}

static void check_linear(const WeightView& W, int ldx, int T) {
  RB_REQUIRE((W.f16 != nullptr) != (W.i8 != nullptr), "linear: exactly one of fp16 / int8 weights");
  RB_REQUIRE(W.i8 == nullptr || W.scale != nullptr, "linear: int8 weights need row scales");
  RB_REQUIRE(W.N > 0 && W.K > 0 && W.K % 64 == 0, "linear: K must be a positive multiple of 64 (pad with zeros)");
  RB_REQUIRE(W.ld >= W.K && W.ld % 16 == 0 && ldx >= W.K && ldx % 8 == 0, "linear: row strides must be 16-byte aligned");
  RB_REQUIRE(T >= 0, "linear: bad token count");
}

I8Digits linear_digits_dest(const WeightView& W, const __half* x, int ldx, int T, void* scratch, size_t scratch_bytes) {
  static const bool off = [] {
    const char* e = std::getenv("RB200_NORM_DIGITS");
    return e && std::string(e) == "0";
  }();
  // The conditions under which launch_linear reads digits from `scratch` (below), and rows whose
  // pitch is the digit planes' pitch.
  if (off || !W.i8 || gemm_forced_legacy() || T < 1 || T > 16 || ldx != W.K || !umma_i8_usable(W, x, ldx, T)) return {};
  if (i8_rows_preferred(W, T) && (reinterpret_cast<uintptr_t>(x) & 15) == 0) return {};  // that kernel reads x itself
  if (T <= 8 && !i8_digits_preferred(W)) return {};
  const size_t po = gemv_partials_bytes(W.N, W.K);
  const bool room = scratch != nullptr && (reinterpret_cast<uintptr_t>(scratch) & 15) == 0 && scratch_bytes >= po + i8_digits_bytes(T, W.K);
  if (!room) return {};  // (digits a producer writes on its way beat the GEMM making its own: 3.55 against 3.65 ms per 4-sequence step)
  I8Digits d;
  d.digits = reinterpret_cast<int8_t*>(static_cast<char*>(scratch) + digits_offset(scratch_bytes, T, W.K));
  d.tscale = i8_tscale(d.digits, T, W.K);
  return d;
}

void launch_gemv(const WeightView& W, const __half* x, int ldx, float* y, int T, float beta, void* scratch,
                 size_t scratch_bytes, cudaStream_t st, bool digits_ready) {
  check_linear(W, ldx, T);
  RB_REQUIRE(T <= 8, "gemv: at most 8 tokens");
  if (T == 0) return;
  // fp16 weights stream faster through TMA (whole 128-byte row pieces) than through per-lane
  // 16-byte loads, so the few-token case uses the tcgen05 kernel with a 16-token tile.
  if (W.f16 && !gemm_forced_legacy() && umma_gemm_usable(W, x, ldx)) return launch_umma_gemm(W, x, ldx, y, T, beta, st);
  if (!digits_ready && i8_rows_preferred(W, T) && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && ldx % 8 == 0) {
    launch_gemv_rows_i8(W, x, ldx, y, T, beta, st);
    return;
  }
  if (W.i8 && !gemm_forced_legacy() && i8_digits_preferred(W) && umma_i8_usable(W, x, ldx, T)) {
    const bool room = scratch != nullptr && (reinterpret_cast<uintptr_t>(scratch) & 15) == 0 &&
                      scratch_bytes >= gemv_partials_bytes(W.N, W.K) + i8_digits_bytes(T, W.K);
    if (!(digits_ready && room) && (i8_fused_preferred(W, T) || (!room && T <= umma_i8_fused_tokens())))
      return launch_umma_i8(W, x, ldx, y, T, beta, nullptr, st);  // digits made in the kernel
    if (room) return launch_umma_i8(W, x, ldx, y, T, beta, static_cast<char*>(scratch) + digits_offset(scratch_bytes, T, W.K), st, digits_ready);
  }
  unsigned* counters = static_cast<unsigned*>(scratch);
  float* partials = scratch ? reinterpret_cast<float*>(static_cast<char*>(scratch) + gemv_counter_bytes(W.N)) : nullptr;
  const GemvPlan p = plan_gemv(W.N, W.K);
  RB_REQUIRE(p.splits == 1 || (scratch != nullptr && scratch_bytes >= gemv_partials_bytes(W.N, W.K)),
             "gemv: scratch too small");
  const size_t smem = static_cast<size_t>(8) * (round_up(p.chunk, 128) + gemv_x_pad(W.i8 != nullptr)) * sizeof(__half);
  RB_REQUIRE((static_cast<size_t>(W.ld) * (W.i8 ? 1 : 2)) % 32 == 0 && (reinterpret_cast<uintptr_t>(W.i8 ? static_cast<const void*>(W.i8) : static_cast<const void*>(W.f16)) & 31) == 0,
             "gemv: weight rows must be 32-byte aligned");
  dim3 grid(p.row_blocks, p.splits);
  count_launch();
  if (W.i8)
    launch_pdl(gemv_kernel<true>, grid, dim3(kGemvWarps * 32), smem, st, W.i8, W.scale, x, y, T, W.K, W.N, W.ld, ldx, beta,
               p.chunk, p.splits, counters, partials);
  else
    launch_pdl(gemv_kernel<false>, grid, dim3(kGemvWarps * 32), smem, st, W.f16, static_cast<const float*>(nullptr), x, y, T, W.K,
               W.N, W.ld, ldx, beta, p.chunk, p.splits, counters, partials);
}

void launch_gemm(const WeightView& W, const __half* x, int ldx, float* y, int T, float beta, cudaStream_t st, void* scratch,
                 size_t scratch_bytes, bool digits_ready) {
  check_linear(W, ldx, T);
  if (T == 0) return;
  // Above 16 tokens the digit tiles (three bytes per activation) crowd the weight tiles out of
  // shared memory and L2 bandwidth, and the kernel that widens int8 into TMEM takes over
  // (58.7 MB matrix, 32 tokens: 15.3 us against 14.5 us).
  const bool digits = T <= 16;
  if (W.i8 && digits && !gemm_forced_legacy() && umma_i8_usable(W, x, ldx, T)) {
    const size_t off = gemv_partials_bytes(W.N, W.K), need = i8_digits_bytes(T, W.K);
    const bool room = scratch != nullptr && (reinterpret_cast<uintptr_t>(scratch) & 15) == 0 && scratch_bytes >= off + need;
    if (!(digits_ready && room) && (i8_fused_preferred(W, T) || (!room && T <= umma_i8_fused_tokens()))) return launch_umma_i8(W, x, ldx, y, T, beta, nullptr, st);
    if (room) return launch_umma_i8(W, x, ldx, y, T, beta, static_cast<char*>(scratch) + digits_offset(scratch_bytes, T, W.K), st, digits_ready);
    void* tmp = nullptr;  // no caller buffer: stream-ordered allocation, released behind the kernels
    RB_CUDA(cudaMallocAsync(&tmp, need, st));
    launch_umma_i8(W, x, ldx, y, T, beta, tmp, st);
    RB_CUDA(cudaFreeAsync(tmp, st));
    return;
  }
  if (!gemm_forced_legacy() && umma_gemm_usable(W, x, ldx)) return launch_umma_gemm(W, x, ldx, y, T, beta, st);
  launch_gemm_mma_sync(W, x, ldx, y, T, beta, st);
}

void launch_gemm_mma_sync(const WeightView& W, const __half* x, int ldx, float* y, int T, float beta, cudaStream_t st) {
  check_linear(W, ldx, T);
  if (T == 0) return;
  dim3 grid(div_up(W.N, kBM), div_up(T, kBN));
  count_launch();
  if (W.i8)
    gemm_kernel<true><<<grid, 256, 0, st>>>(W.i8, W.scale, x, y, T, W.K, W.N, W.ld, ldx, beta);
  else
    gemm_kernel<false><<<grid, 256, 0, st>>>(W.f16, nullptr, x, y, T, W.K, W.N, W.ld, ldx, beta);
}

void launch_linear(const WeightView& W, const __half* x, int ldx, float* y, int T, float beta, void* scratch,
                   size_t scratch_bytes, cudaStream_t st, bool digits_ready) {
  if (T <= 8) launch_gemv(W, x, ldx, y, T, beta, scratch, scratch_bytes, st, digits_ready);
  else launch_gemm(W, x, ldx, y, T, beta, st, scratch, scratch_bytes, digits_ready);
}

}  // namespace rb200

// ---- C boundary -----------------------------------------------------------------------

using namespace rb200;

extern "C" {

size_t rb200_gemv_scratch_bytes(int N, int K) {
  if (N <= 0 || K < 64) return 256;
  return gemv_scratch_bytes(N, K, 8);
}

int rb200_gemv_int8(const int8_t* wq, const float* scale, const void* x, float* y, int T, int K, int N, int ldw, int ldx,
                    float beta, void* scratch, size_t scratch_bytes, void* stream) {
  return guarded([&] {
    WeightView W;
    W.i8 = wq;
    W.scale = scale;
    W.N = N;
    W.K = K;
    W.ld = ldw;
    launch_gemv(W, static_cast<const __half*>(x), ldx, y, T, beta, scratch, scratch_bytes, as_stream(stream));
    RB_CUDA(cudaGetLastError());
    return 0;
  });
}

int rb200_gemv_f16(const void* w, const void* x, float* y, int T, int K, int N, int ldw, int ldx, float beta,
                   void* scratch, size_t scratch_bytes, void* stream) {
  return guarded([&] {
    WeightView W;
    W.f16 = static_cast<const __half*>(w);
    W.N = N;
    W.K = K;
    W.ld = ldw;
    launch_gemv(W, static_cast<const __half*>(x), ldx, y, T, beta, scratch, scratch_bytes, as_stream(stream));
    RB_CUDA(cudaGetLastError());
    return 0;
  });
}

int rb200_gemm_status(void) {
  int v = -1;
  const int rc = guarded([&] {
    v = umma_gemm_status();
    return 0;
  });
  return rc == 0 ? v : -1;
}

int rb200_gemm(const void* w_f16, const int8_t* w_i8, const float* scale, const void* x, float* y, int T, int K, int N,
               int ldw, int ldx, float beta, void* stream) {
  return guarded([&] {
    WeightView W;
    W.f16 = static_cast<const __half*>(w_f16);
    W.i8 = w_i8;
    W.scale = scale;
    W.N = N;
    W.K = K;
    W.ld = ldw;
    launch_gemm(W, static_cast<const __half*>(x), ldx, y, T, beta, as_stream(stream));
    RB_CUDA(cudaGetLastError());
    return 0;
  });
}

}  // extern "C"
