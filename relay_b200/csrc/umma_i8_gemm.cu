// Weight-only int8 linear for up to 64 tokens on the integer tensor cores:
//   y[T,N] = scale[n] * (Wq[N,K] . x[T,K]) (+ beta*y)
// (the reference's gemv_int8_kernel and, above 8 tokens, its dequantise-then-cuBLAS path:
// engine/src/cuda_kernels.cuh:391-436, engine/src/cuda_backend.cu:712-730).
//
// The int8 rows are never widened. Each activation row is written once as three signed base-128
// digits of a fixed-point number, x = 2^(e-20) * (d0 + 128 d1 + 128^2 d2) with 2^e above the
// row's largest magnitude: elements within 2^-10 of the largest are exact, the rest are
// rounded at 2^-21 of it, which is finer than their fp16 rounding matters to the sum. Then
//   Wq . x = 2^(e-20) * (Wq.d0 + 128 Wq.d1 + 128^2 Wq.d2)
// and the three integer products are exact in int32: tcgen05.mma kind::i8 takes the raw weight
// tile (A, 128 rows x 128 bytes straight from TMA) and the digit tile (B, three digits x BN
// tokens = 3 BN accumulator columns) and needs no conversion work in the main loop, so the
// kernel is the plain TMA -> shared-memory ring -> MMA -> TMEM pipeline and runs at the speed
// the int8 bytes arrive from HBM.
//
// Up to four tokens the GEMM can also make the digit tiles itself (FUSED below): no kernel
// ahead of it, no digit buffer.
//
// Warp roles as in umma_gemm.cu: warp 0 TMA producer, warp 1 MMA issuer and TMEM owner,
// warps 2-5 epilogue (combine the digits in fp32, row scale x token scale, beta*y). Matrices
// with few 128-row tiles split K over a thread-block cluster and add the partial tiles over
// DSMEM in rank order. Every mbarrier wait is bounded; a wait that gives up records a code in
// the device's status word and the CTA still releases its TMEM.
#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <string>
#include <unordered_map>
#include <utility>

#include "i8_digits.cuh"
#include "kernels.h"
#include "tcgen05.cuh"

namespace rb200 {

using namespace tc;

namespace {

constexpr int kTileM = 128;
constexpr int kBlockKB = 128;  // int8 per k block: one 128-byte swizzle atom
constexpr int kI8Threads = 192;
using namespace i8d;

template <int BN>
struct I8Smem {
  static constexpr int kABytes = kTileM * kBlockKB;
  static constexpr int kBBytes = kDigits * BN * kBlockKB;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = 196 * 1024 / kStageBytes > 10 ? 10 : 196 * 1024 / kStageBytes;
  static constexpr int kAccCols = kDigits * BN;
  static constexpr int kTmemCols = kAccCols <= 64 ? 64 : (kAccCols <= 128 ? 128 : 256);
  static constexpr int kBarBytes = 512;  // barriers, the TMEM slot, the fused digit pass's row maxima
  static constexpr size_t kTotal = static_cast<size_t>(kStages) * kStageBytes + kBarBytes + 1024;
};

// kind::i8: int32 accumulator (bits 4-5 = 2), signed 8-bit A and B (bits 7-9, 10-12 = 1), both
// K-major, N / 8 in bits 17-22, M / 16 in bits 24-28.
__host__ __device__ constexpr uint32_t umma_idesc_i8(int M, int N) {
  return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 16 consecutive 32-bit columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}

// A 3-D load: digit tile = [digit][token][k].
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z)
               : "memory");
}

// ---- activation rows -> digits ----------------------------------------------------------
// Programmatic dependent launch (common.cuh): the GEMM that follows is launched while this kernel
// runs (its weight loads do not depend on the digits) and waits for this grid before its first
// digit load.

constexpr int kQuantThreads = 512;
constexpr int kQuantHeld = 4;  // 16-byte pieces of the row a thread keeps in registers between the passes

__device__ __forceinline__ void store_digits8(const uint4& v, float up, int8_t* out, long long plane) {
  uint32_t w[kDigits][2];
  digits8(v, up, w);
#pragma unroll
  for (int g = 0; g < kDigits; ++g) *reinterpret_cast<uint2*>(out + g * plane) = make_uint2(w[g][0], w[g][1]);
}

// One block per token. digits[d][t][k] (row pitch K), tscale[t] = 2^(e-20). K is a multiple of 8.
__global__ void __launch_bounds__(kQuantThreads) quantize_tokens_kernel(const __half* __restrict__ x, int ldx, int K, int T,
                                                                        int8_t* __restrict__ digits, float* __restrict__ tscale) {
  pdl_trigger();
  pdl_wait();  // the activations come from the kernel ahead
  const int t = blockIdx.x;
  const uint4* row = reinterpret_cast<const uint4*>(x + static_cast<long long>(t) * ldx);
  const int pieces = K / 8;
  __shared__ float s_max[kQuantThreads / 32];
  uint4 held[kQuantHeld];
  float mx = 0.f;
#pragma unroll
  for (int c = 0; c < kQuantHeld; ++c) {
    const int i = threadIdx.x + c * kQuantThreads;
    held[c] = i < pieces ? row[i] : make_uint4(0, 0, 0, 0);
    mx = fmaxf(mx, abs_max8(held[c]));
  }
  for (int i = threadIdx.x + kQuantHeld * kQuantThreads; i < pieces; i += kQuantThreads) mx = fmaxf(mx, abs_max8(row[i]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = s_max[0];
#pragma unroll
  for (int w = 1; w < kQuantThreads / 32; ++w) mx = fmaxf(mx, s_max[w]);
  float up, down;
  digit_scales(mx, up, down);
  if (threadIdx.x == 0) tscale[t] = down;
  const long long plane = static_cast<long long>(T) * K;
  int8_t* out = digits + static_cast<long long>(t) * K;
#pragma unroll
  for (int c = 0; c < kQuantHeld; ++c) {
    const int i = threadIdx.x + c * kQuantThreads;
    if (i < pieces) store_digits8(held[c], up, out + 8 * i, plane);
  }
  for (int i = threadIdx.x + kQuantHeld * kQuantThreads; i < pieces; i += kQuantThreads) store_digits8(row[i], up, out + 8 * i, plane);
}

// ---- the GEMM -----------------------------------------------------------------------------
// FUSED (at most kFusedTokens tokens): no digit buffer and no kernel ahead. The four epilogue
// warps, idle during the main loop otherwise, find each token row's largest magnitude (every
// CTA reads the few activation rows from L2) and then write the digit tile of each k block
// straight into the ring in the 128-byte-swizzled layout the MMA reads, one warp per k block
// in turn; the stage's barrier takes the weight tile's bytes and that warp's arrival.
constexpr int kFusedTokens = 4;

template <int BN, bool FUSED>
__global__ void __launch_bounds__(kI8Threads, 1)
umma_i8_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_q,
               const float* __restrict__ scale, const float* __restrict__ tscale, const __half* __restrict__ x, int ldx,
               float* __restrict__ y, int T, int N, int K, int rows, float beta, int* __restrict__ status) {
  using S = I8Smem<BN>;
  constexpr int NS = S::kStages;
  constexpr uint32_t kTmemCols = S::kTmemCols;
  pdl_trigger();
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  const uint32_t sA = base;
  const uint32_t sB = sA + NS * S::kABytes;
  const uint32_t bars = sB + NS * S::kBBytes;
  const uint32_t full_bar = bars;            // NS x 8 bytes: TMA landed
  const uint32_t empty_bar = bars + 8 * NS;  // NS x 8: the MMAs have read the stage
  const uint32_t accum_bar = bars + 16 * NS;
  const uint32_t tmem_slot = accum_bar + 8;
  const uint32_t rowmax_slot = accum_bar + 16;  // FUSED: [4 warps][kFusedTokens] floats
  unsigned char* gen_base = smem_dyn + (base - smem_u32(smem_dyn));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // `rows` (at most 128) weight rows per CTA: the host shrinks the tile so that
  // the grid fills the SMs evenly; the MMA still spans 128 lanes and the rest is ignored.
  const int m0 = blockIdx.x * rows, tok0 = blockIdx.y * BN;
  const uint32_t stage_tx = static_cast<uint32_t>(rows) * kBlockKB + (FUSED ? 0 : S::kBBytes);
  const int splits = gridDim.z, split = blockIdx.z;  // the cluster spans z: split == rank in the cluster
  const int nk_all = (K + kBlockKB - 1) / kBlockKB;  // a last half block reads zeros past K
  const int kb_begin = static_cast<int>(static_cast<long long>(nk_all) * split / splits);
  const int nk = static_cast<int>(static_cast<long long>(nk_all) * (split + 1) / splits) - kb_begin;

  const int pre = min(nk, NS);  // the ring starts empty: stages the producer fills without waiting
  if (warp == 0 && lane == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
    if (!FUSED) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_q)) : "memory");
    for (int s = 0; s < NS; ++s) {
      mbar_init(full_bar + 8 * s, FUSED ? 2 : 1);
      mbar_init(empty_bar + 8 * s, 1);
    }
    mbar_init(accum_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
    // The first weight tiles leave for HBM before anything else is set up (TMEM, the block
    // barrier): the barriers they complete on are this thread's own work above.
    for (int kb = 0; kb < pre; ++kb) {
      mbar_expect_tx(full_bar + 8 * kb, stage_tx);
      tma_load_2d(sA + kb * S::kABytes, &map_w, (kb_begin + kb) * kBlockKB, m0, full_bar + 8 * kb);
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(gen_base + (tmem_slot - base));

  bool ok = true;
  float ts[kFusedTokens] = {};  // FUSED: the token scales, known to warps 2-5
  if (warp == 0) {
    if (elect_one()) {
      // The weight tiles of the first stages are already in flight; their digit tiles follow once
      // the kernel that writes the digits (it may still be running) has finished.
      if (!FUSED) {
        pdl_wait();
        for (int kb = 0; kb < pre; ++kb)
          tma_load_3d(sB + kb * S::kBBytes, &map_q, (kb_begin + kb) * kBlockKB, tok0, 0, full_bar + 8 * kb);
      }
      for (int kb = pre; kb < nk && ok; ++kb) {
        const int s = kb % NS;
        ok = mbar_wait(empty_bar + 8 * s, ((kb / NS) & 1) ^ 1);
        if (!ok) break;
        mbar_expect_tx(full_bar + 8 * s, stage_tx);
        const int kx = (kb_begin + kb) * kBlockKB;
        tma_load_2d(sA + s * S::kABytes, &map_w, kx, m0, full_bar + 8 * s);
        if (!FUSED) tma_load_3d(sB + s * S::kBBytes, &map_q, kx, tok0, 0, full_bar + 8 * s);
      }
      if (!ok) atomicExch(status, 21);
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_i8(kTileM, kDigits * BN);
      for (int kb = 0; kb < nk && ok; ++kb) {
        const int s = kb % NS;
        ok = mbar_wait(full_bar + 8 * s, (kb / NS) & 1);
        if (!ok) break;
        tc_fence_after();
        const uint64_t da = smem_desc_sw128(sA + s * S::kABytes), db = smem_desc_sw128(sB + s * S::kBBytes);
#pragma unroll
        for (int k4 = 0; k4 < kBlockKB / 32; ++k4)  // 32 int8 = 32 bytes = 2 descriptor units per step
          umma_i8(tmem_base, da + 2 * k4, db + 2 * k4, idesc, (kb | k4) != 0);
        umma_commit(empty_bar + 8 * s);
      }
      umma_commit(accum_bar);
      if (!ok) atomicExch(status, 22);
    }
  } else {
    if (FUSED) {
      const int pw = warp - 2, ptid = static_cast<int>(threadIdx.x) - 64;
      // Token rows T..BN-1 of every digit tile stay zero; rows below T are rewritten per k block.
      uint4* bz = reinterpret_cast<uint4*>(gen_base + (sB - base));
      for (int i = ptid; i < NS * S::kBBytes / 16; i += 128) bz[i] = make_uint4(0u, 0u, 0u, 0u);
      fence_async_smem();
      pdl_wait();  // the activations (and, with beta, y) come from kernels before this one
      float* rowmax = reinterpret_cast<float*>(gen_base + (rowmax_slot - base));
      // A lane owns 16 consecutive k of one token: one 16-byte chunk of each digit's row.
      const int tok = lane >> 3, ch = lane & 7;
      const bool has = tok < T;
      const __half* xrow = x + static_cast<long long>(tok) * ldx + ch * 16;
      uint4 a = make_uint4(0u, 0u, 0u, 0u), b = a;
      auto fetch = [&](int kb, uint4& lo, uint4& hi) {
        const int k = (kb_begin + kb) * kBlockKB;
        lo = hi = make_uint4(0u, 0u, 0u, 0u);
        if (has && k + ch * 16 < K) {  // a last half block: nothing past K is read
          const uint4* p = reinterpret_cast<const uint4*>(xrow + k);
          lo = p[0];
          hi = p[1];
        }
      };
      if (pw < nk) fetch(pw, a, b);  // in flight with the loads of the pass below
      const int pieces = K / 8;
      {
        // Largest magnitude of each token row; the loads of all rows go out together (L2 latency,
        // not bandwidth, is what this pass costs).
        float mx[kFusedTokens] = {};
        const uint4* row0 = reinterpret_cast<const uint4*>(x);
        const long long pitch = ldx / 8;
        for (int i0 = ptid; i0 < pieces; i0 += 128 * 8) {
          uint4 v[8][kFusedTokens];
#pragma unroll
          for (int u = 0; u < 8; ++u)
#pragma unroll
            for (int t = 0; t < kFusedTokens; ++t) {
              const int i = i0 + u * 128;
              v[u][t] = (t < T && i < pieces) ? row0[t * pitch + i] : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
          for (int u = 0; u < 8; ++u)
#pragma unroll
            for (int t = 0; t < kFusedTokens; ++t) mx[t] = fmaxf(mx[t], abs_max8(v[u][t]));
        }
#pragma unroll
        for (int t = 0; t < kFusedTokens; ++t) {
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) mx[t] = fmaxf(mx[t], __shfl_xor_sync(0xffffffffu, mx[t], o));
          if (lane == 0) rowmax[pw * kFusedTokens + t] = mx[t];
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");  // warps 2-5: the zeroed tiles and the row maxima
      float ups[kFusedTokens];
#pragma unroll
      for (int t = 0; t < kFusedTokens; ++t) {
        float mx = 0.f;
        mx = fmaxf(fmaxf(rowmax[t], rowmax[kFusedTokens + t]), fmaxf(rowmax[2 * kFusedTokens + t], rowmax[3 * kFusedTokens + t]));
        digit_scales(mx, ups[t], ts[t]);
      }
      const float up = tok == 0 ? ups[0] : tok == 1 ? ups[1] : tok == 2 ? ups[2] : ups[3];
      const uint32_t dst0 = sB + static_cast<uint32_t>(tok) * kBlockKB + static_cast<uint32_t>((ch ^ (tok & 7)) << 4);
      for (int kb = pw; kb < nk; kb += 4) {
        uint4 na = make_uint4(0u, 0u, 0u, 0u), nb = na;
        if (kb + 4 < nk) fetch(kb + 4, na, nb);
        const int s = kb % NS;
        if (kb >= NS) ok = mbar_wait(empty_bar + 8 * s, ((kb / NS) & 1) ^ 1);  // the MMAs have read the tile this overwrites
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (has) {
          uint32_t lo[kDigits][2], hi[kDigits][2];
          digits8(a, up, lo);
          digits8(b, up, hi);
#pragma unroll
          for (int g = 0; g < kDigits; ++g)
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst0 + s * S::kBBytes + g * BN * kBlockKB), "r"(lo[g][0]),
                         "r"(lo[g][1]), "r"(hi[g][0]), "r"(hi[g][1])
                         : "memory");
        }
        fence_async_smem();  // generic-proxy writes, read by the MMA through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(full_bar + 8 * s);
        a = na;
        b = nb;
      }
      if (!ok && lane == 0) atomicExch(status, 25);
    } else {
      pdl_wait();  // token scales (and, with beta, y) come from kernels before this one
    }
    // What the epilogue needs besides the accumulator is in memory already (the row scales are
    // weights; the token scales and y come from kernels that have completed): the first 16 token
    // columns' worth is fetched while the MMAs still run, not behind them.
    const int quarter = warp & 3;  // the TMEM lane quarter this warp may read
    const int row = quarter * 32 + lane;
    const int n = m0 + row;
    const bool live = row < rows && n < N;
    const float sc = live ? scale[n] : 0.f;
    const int nt0 = min(16, T - tok0);
    float old0[16], ts0[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      old0[j] = (splits == 1 && live && beta != 0.f && j < nt0) ? y[static_cast<long long>(tok0 + j) * N + n] : 0.f;
      ts0[j] = FUSED ? ts[j & (kFusedTokens - 1)] : (j < nt0 ? tscale[tok0 + j] : 0.f);
    }
    const bool done = mbar_wait(accum_bar, 0);
    if (!done) atomicExch(status, 24);
    tc_fence_after();
    const uint32_t trow = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    float* red = reinterpret_cast<float*>(gen_base);  // split K: this CTA's partial tile, red[token][row]
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 16) {
      uint32_t d0[16], d1[16], d2[16];
      tmem_ld16(trow + c0, d0);
      tmem_ld16(trow + BN + c0, d1);
      tmem_ld16(trow + 2 * BN + c0, d2);
      tmem_ld_wait();
      float v[16];
#pragma unroll
      for (int j = 0; j < 16; ++j)
        v[j] = fmaf(16384.f, static_cast<float>(static_cast<int>(d2[j])),
                    fmaf(128.f, static_cast<float>(static_cast<int>(d1[j])), static_cast<float>(static_cast<int>(d0[j]))));
      if (splits > 1) {
#pragma unroll
        for (int j = 0; j < 16; ++j) red[(c0 + j) * kTileM + row] = v[j];
      } else if (done && live) {
        const int nt = min(16, T - tok0 - c0);  // valid token columns of this chunk
        float* dst = y + static_cast<long long>(tok0 + c0) * N + n;
        float old[16], tsv[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          old[j] = c0 == 0 ? old0[j] : ((beta != 0.f && j < nt) ? dst[static_cast<long long>(j) * N] : 0.f);
          tsv[j] = c0 == 0 ? ts0[j] : (FUSED ? ts[j & (kFusedTokens - 1)] : (j < nt ? tscale[tok0 + c0 + j] : 0.f));
        }
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (j < nt) dst[static_cast<long long>(j) * N] = v[j] * (sc * tsv[j]) + beta * old[j];
      }
    }
  }
  if (splits > 1) {
    // What this CTA's share of the columns needs from memory (row scale, token scales, y) is
    // fetched before the cluster barrier, not behind it.
    const int per = (BN + splits - 1) / splits;  // token columns this CTA finishes
    const int c_begin = split * per, c_end = min(min(BN, c_begin + per), T - tok0);
    constexpr int kPre = 8;
    float old_pre[kPre], ts_pre[kPre];
    float sc_pre = 0.f;
    if (warp >= 2) {
      const int row = (warp & 3) * 32 + lane;
      const int n = m0 + row;
      const bool live = row < rows && n < N;
      sc_pre = live ? scale[n] : 0.f;
#pragma unroll
      for (int i = 0; i < kPre; ++i) {
        const int c = c_begin + i;
        const bool in = c < c_end;
        old_pre[i] = (in && live && beta != 0.f) ? y[static_cast<long long>(tok0 + c) * N + n] : 0.f;
        ts_pre[i] = !in ? 0.f : !FUSED ? tscale[tok0 + c] : c == 0 ? ts[0] : c == 1 ? ts[1] : c == 2 ? ts[2] : ts[3];
      }
    }
    cluster_sync_all();  // every member's partial tile is in its shared memory
    if (warp >= 2) {
      const int row = (warp & 3) * 32 + lane;
      const int n = m0 + row;
      const bool live = row < rows && n < N;
      const float sc = sc_pre;
      uint32_t peer[8];
#pragma unroll
      for (int r = 0; r < 8; ++r)
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer[r]) : "r"(base + static_cast<uint32_t>(row) * 4), "r"(r < splits ? r : 0));
      auto finish_column = [&](int c, float old, float tsc) {
        float acc = 0.f;
#pragma unroll
        for (int r = 0; r < 8; ++r) {  // members in rank order: the sum is the same on every run
          if (r >= splits) break;
          float part;
          asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(part) : "r"(peer[r] + static_cast<uint32_t>(c * kTileM) * 4) : "memory");
          acc += part;
        }
        if (live) y[static_cast<long long>(tok0 + c) * N + n] = acc * (sc * tsc) + beta * old;
      };
#pragma unroll
      for (int i = 0; i < kPre; ++i)
        if (c_begin + i < c_end) finish_column(c_begin + i, old_pre[i], ts_pre[i]);
      for (int c = c_begin + kPre; c < c_end; ++c) {  // wider token tiles with few members: fetched here
        const float old = (live && beta != 0.f) ? y[static_cast<long long>(tok0 + c) * N + n] : 0.f;
        const float tsc = !FUSED ? tscale[tok0 + c] : c == 0 ? ts[0] : c == 1 ? ts[1] : c == 2 ? ts[2] : ts[3];
        finish_column(c, old, tsc);
      }
    }
    cluster_sync_all();  // nobody leaves while a peer may still read its shared memory
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int BN, bool FUSED>
void launch_i8_t(const WeightView& W, const int8_t* digits, const float* tscale, const __half* x, int ldx, float* y, int T,
                 float beta, cudaStream_t st) {
  using S = I8Smem<BN>;
  static PerDeviceOnce once;
  auto kernel = umma_i8_kernel<BN, FUSED>;
  if (once.first())
    RB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(S::kTotal)));
  // Rows per CTA and the K split: the pair that needs the fewest (waves x bytes per CTA), where a
  // CTA's fixed cost (prologue, pipeline fill, epilogue) counts like 48 KB of weights. A cluster
  // needs its CTAs on SMs of one GPC at the same time, so fewer clusters than SMs / size are
  // resident together: the occupancy query says how many.
  const int ttiles = div_up(T, BN), nk = div_up(W.K, kBlockKB);
  static const std::array<int, 9> capacity = cluster_capacity(kernel, kI8Threads, S::kTotal);
  // The search is per (N, K, token tiles) and remembered: it runs once per matrix shape.
  static std::mutex plan_mu;
  static std::unordered_map<uint64_t, std::pair<int, int>> plans;
  const uint64_t key = (static_cast<uint64_t>(W.N) << 36) ^ (static_cast<uint64_t>(W.K) << 12) ^ static_cast<uint64_t>(ttiles);
  int rows = kTileM, splits = 1;
  {
    std::lock_guard<std::mutex> lock(plan_mu);
    auto it = plans.find(key);
    if (it == plans.end()) {
      // Any row count works (the TMA box is `rows` high, the MMA spans 128 lanes and the epilogue
      // ignores the rest), but a stage of the ring holds `rows` x 128 bytes, and with much fewer
      // than 128 rows a CTA no longer has enough bytes in flight: 56-row tiles in 74 clusters of
      // two measured 20.7 us on the 14336 -> 4096 matrix against 13.3 us for 128-row tiles in 32
      // clusters of four, 42-row tiles 9.4 against 8.4 us on 4096 -> 6144; 97-row tiles (148 CTAs
      // instead of 138 of 104 rows) gain 3 % on 4096 -> 14336. Hence: any count from 96 up,
      // multiples of 8 below. RB200_I8_ROW_STEP=8: multiples of 8 only.
      static const int step = [] {
        const char* e = std::getenv("RB200_I8_ROW_STEP");
        return e && std::atoi(e) == 8 ? 8 : 1;
      }();
      double best = 1e30;
      for (int r = kTileM; r >= 64; --r) {
        if (r % 8 != 0 && (step == 8 || r < 96)) continue;
        for (int sp = 1; sp <= 8; ++sp) {
          if (sp > 1 && (nk / sp < 4 || static_cast<size_t>(BN) * kTileM * 4 > static_cast<size_t>(S::kStages) * S::kStageBytes)) break;
          const long long clusters = static_cast<long long>(div_up(W.N, r)) * ttiles;
          // below about 1.25 x BN rows a CTA is bound by its MMAs (3 x BN columns per k block
          // whatever the row count), not by its weight bytes
          const double eff_rows = std::max<double>(r, 1.25 * BN);
          // A grid of exactly as many clusters as fit at once only starts together on an empty
          // GPU; under the tail of the kernel ahead its last cluster waits for a whole GPC's worth
          // of slots. Filling the last slot measured no faster (33 clusters of four against 32 on
          // 14336 -> 4096, 74 of two against 70 on 4096 -> 6144: within the run-to-run spread), so
          // one cluster of room is kept.
          const long long room = sp > 1 ? std::max(1, capacity[sp] - 1) : capacity[sp];
          const double cost = static_cast<double>(div_up(clusters, room)) *
                              (eff_rows * W.K / sp + 48.0 * 1024 + (sp > 1 ? 8.0 * 1024 : 0.0));
          if (cost < best - 1e-9) {
            best = cost;
            rows = r;
            splits = sp;
          }
        }
      }
      plans.emplace(key, std::make_pair(rows, splits));
    } else {
      rows = it->second.first;
      splits = it->second.second;
    }
  }
  static const int forced = [] {
    const char* e = std::getenv("RB200_GEMM_SPLITS");
    return e ? std::atoi(e) : 0;
  }();
  if (forced > 0) splits = std::min({forced, 8, std::max(1, nk)});
  const CUtensorMap mw = make_map(W.i8, 1, W.N, W.K, W.ld, rows, kBlockKB, true);
  CUtensorMap mq{};  // FUSED: the kernel makes the digit tiles itself
  if (!FUSED) mq = make_map_3d(digits, W.K, T, kDigits, W.K, static_cast<long long>(T) * W.K, kBlockKB, BN, kDigits);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(div_up(W.N, rows), ttiles, splits);
  cfg.blockDim = dim3(kI8Threads);
  cfg.dynamicSmemBytes = S::kTotal;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = splits;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // may start under the kernel ahead
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  count_launch();
  int* status = status_word();
  const float* scale = W.scale;
  const int N = W.N, K = W.K;
  RB_CUDA(cudaLaunchKernelEx(&cfg, kernel, mw, mq, scale, tscale, x, ldx, y, T, N, K, rows, beta, status));
}

}  // namespace

size_t i8_digits_bytes(int T, int K) {
  // three digit planes, then the token scales (kept 16-byte aligned)
  return (static_cast<size_t>(kDigits) * T * K + 15) / 16 * 16 + static_cast<size_t>(T) * sizeof(float);
}

bool umma_i8_usable(const WeightView& W, const __half* x, int ldx, int T) {
  static const bool off = [] {
    const char* e = std::getenv("RB200_INT8_GEMM");
    return e && std::string(e) == "widen";
  }();
  return !off && W.i8 && T >= 1 && T <= 64 && W.K % 64 == 0 && W.ld % 16 == 0 && ldx % 8 == 0 &&
         (reinterpret_cast<uintptr_t>(W.i8) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
}

int umma_i8_fused_tokens() {
  static const bool off = [] {
    const char* e = std::getenv("RB200_I8_FUSED");
    return e && std::string(e) == "0";
  }();
  return off ? 0 : kFusedTokens;
}

float* i8_tscale(int8_t* digits, int T, int K) {
  return reinterpret_cast<float*>(digits + (static_cast<size_t>(kDigits) * T * K + 15) / 16 * 16);
}

void launch_umma_i8(const WeightView& W, const __half* x, int ldx, float* y, int T, float beta, void* scratch, cudaStream_t st,
                    bool digits_ready) {
  if (T == 0) return;
  // Without a digit buffer the GEMM makes the digits itself (few tokens only).
  if (scratch == nullptr) {
    RB_REQUIRE(T <= umma_i8_fused_tokens(), "int8 linear: the digit buffer is missing");
    return launch_i8_t<16, true>(W, nullptr, nullptr, x, ldx, y, T, beta, st);
  }
  int8_t* digits = static_cast<int8_t*>(scratch);
  float* tscale = i8_tscale(digits, T, W.K);
  if (!digits_ready) {
    count_launch();
    launch_pdl(quantize_tokens_kernel, dim3(T), dim3(kQuantThreads), 0, st, x, ldx, W.K, T, digits, tscale);
  }
  if (T <= 16) launch_i8_t<16, false>(W, digits, tscale, x, ldx, y, T, beta, st);
  else if (T <= 32) launch_i8_t<32, false>(W, digits, tscale, x, ldx, y, T, beta, st);
  else launch_i8_t<64, false>(W, digits, tscale, x, ldx, y, T, beta, st);
}

}  // namespace rb200
