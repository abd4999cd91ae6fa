// Causal flash attention for prompt chunks on tcgen05 tensor cores (replaces the WMMA
// flash_prefill_kernel of the reference, engine/src/cuda_kernels.cuh:51-178, for head sizes
// 64 and 128 with an even number of query heads per KV head and block sizes that are
// multiples of 16; other layouts stay on prefill_flash_kernel in attention.cu).
//
// One CTA = one prefill tile (up to 64 query positions, engine/src/cuda_backend.cu:533-545)
// of TWO query heads that share a KV head: 128 rows on the M axis of tcgen05.mma, so every
// K/V tile fetched is used by both heads. Per 128-key tile:
//   S = Q K^T    A = Q (fp16, shared memory, K-major, 128-byte swizzle), B = K pages as TMA
//                lands them (K-major), D = S in TMEM (128 lanes x 128 columns, fp32);
//   softmax      four warps, one thread per row: tcgen05.ld the row of S, scale, causal mask,
//                running max / sum, P = exp2(.) as fp16 into shared memory in the A layout;
//   O_t = P V    A = P, B = V pages as TMA lands them ([key][d] = MN-major), D = O_t in TMEM;
//   O = O * corr + O_t   in the softmax threads' registers (tcgen05.ld of O_t).
// Warp roles: warp 0 producer (one lane issues one TMA box per KV page, 16 keys x 64 dims, from
// a tensor map over the whole layer pool, following the block table), warp 1 issues the MMAs
// and owns TMEM, warps 2-5 softmax / accumulate / epilogue. QK^T of tile j+1 is issued right
// after P V of tile j, so it runs while the softmax warps fold O_t in.
//
// Every mbarrier wait is bounded in time; a wait that gives up records a code in the
// device's status word (tc::status_word) and the CTA still frees its TMEM and exits.
#include <cstdlib>
#include <mutex>
#include <string>

#include "kernels.h"
#include "tcgen05.cuh"

namespace rb200 {

using namespace tc;

namespace {

constexpr int kKeys = 128;      // keys per tile (N of the first MMA, K of the second)
constexpr int kRows = 128;      // 2 heads x 64 query positions
constexpr int kPfThreads = 192;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Descriptor of an MN-major operand (V: [key][d], d contiguous) in the layout TMA's 128-byte
// swizzle writes: 8-key groups 1024 bytes apart (stride byte offset), 64-wide d atoms
// `lbo_bytes` apart (leading byte offset), version 1, layout type SWIZZLE_128B.
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

template <int D>
struct PfSmem {
  static constexpr int kQBytes = kRows * D * 2;
  static constexpr int kKBytes = kKeys * D * 2;          // one K (or V) tile
  static constexpr int kPBytes = kRows * kKeys * 2;
  static constexpr int kStages = D == 64 ? 2 : 1;
  static constexpr int kBarBytes = 256;
  static constexpr size_t kTotal = kQBytes + static_cast<size_t>(kStages) * 2 * kKBytes + kPBytes + kBarBytes + 1024;
};

template <int D>
__global__ void __launch_bounds__(kPfThreads, D == 64 ? 2 : 1)
umma_prefill_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                    const float* __restrict__ q, TokenMeta m, const int2* __restrict__ tiles,
                    __half* __restrict__ out, int heads, int kv_heads, int bs, int q_stride, int o_stride,
                    float scale_log2e, int* __restrict__ status) {
  using S = PfSmem<D>;
  constexpr int NS = S::kStages;
  constexpr uint32_t kTmemCols = 256;  // S: columns 0..127, O_t: columns 128..128+D-1
  constexpr int kAtoms = D / 64;       // 64-wide d atoms per K/V row
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  unsigned char* gen = smem_dyn + (base - smem_u32(smem_dyn));
  const uint32_t sQ = base;
  const uint32_t sK = sQ + S::kQBytes;                 // NS stages of [K tile][V tile]
  const uint32_t sP = sK + NS * 2 * S::kKBytes;
  const uint32_t bars = sP + S::kPBytes;
  const uint32_t kv_full = bars, kv_empty = bars + 16;  // 2 x 8 bytes each
  const uint32_t q_ready = bars + 32, s_ready = bars + 40, p_ready = bars + 48, o_ready = bars + 56, o_free = bars + 64;
  const uint32_t tmem_slot = bars + 72;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int2 tile = tiles[blockIdx.x];
  const int t0 = tile.x, nrows = tile.y;
  const int G = heads / kv_heads, pairs = G / 2;
  const int kvh = blockIdx.y / pairs, h0 = kvh * G + 2 * (blockIdx.y % pairs);
  const int pos0 = m.pos[t0];
  const int nk = pos0 + nrows;                 // keys the tile's last row sees
  const int ntiles = (nk + kKeys - 1) / kKeys;
  const int* table = m.tables + m.table_off[m.seq[t0]];

  if (warp == 0 && lane == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(kv_full + 8 * s, 1);
      mbar_init(kv_empty + 8 * s, 1);
    }
    mbar_init(q_ready, 4);
    mbar_init(s_ready, 1);
    mbar_init(p_ready, 4);
    mbar_init(o_ready, 1);
    mbar_init(o_free, 4);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(gen + (tmem_slot - base));
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + kKeys;

  bool ok = true;
  if (warp == 0) {
    // ---- producer: one TMA box per page (16 keys x 64 dims), K tile then V tile ----
    if (elect_one()) {
      const int last_page = (nk - 1) / 16;  // pages are 16-key runs; a block of bs keys holds bs / 16 of them
      for (int j = 0; j < ntiles && ok; ++j) {
        const int s = j % NS;
        ok = mbar_wait(kv_empty + 8 * s, ((j / NS) & 1) ^ 1);
        if (!ok) break;
        mbar_expect_tx(kv_full + 8 * s, 2 * S::kKBytes);
        const uint32_t kdst = sK + s * 2 * S::kKBytes, vdst = kdst + S::kKBytes;
#pragma unroll 1
        for (int pg = 0; pg < kKeys / 16; ++pg) {
          // pages past the context repeat the last valid one: finite values, masked to zero weight
          const int page = min(j * (kKeys / 16) + pg, last_page);
          const int key = page * 16;
          const int blk = table[key / bs], slot = key % bs;
          const int row = (blk * kv_heads + kvh) * bs + slot;  // row of the [blocks*kv_heads*bs, D] pool view
#pragma unroll
          for (int a = 0; a < kAtoms; ++a) {
            tma_load_2d(kdst + a * (kKeys * 128) + pg * 2048, &map_k, a * 64, row, kv_full + 8 * s);
            tma_load_2d(vdst + a * (kKeys * 128) + pg * 2048, &map_v, a * 64, row, kv_full + 8 * s);
          }
        }
      }
      if (!ok) atomicExch(status, 11);
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    if (elect_one()) {
      constexpr uint32_t idesc_qk = umma_idesc(kRows, kKeys);
      constexpr uint32_t idesc_pv = umma_idesc(kRows, D) | (1u << 16);  // B (V) is MN-major
      auto issue_qk = [&](int j) {
        const uint32_t kt = sK + (j % NS) * 2 * S::kKBytes;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * (kRows * 128) + (k % 4) * 32;  // 64-wide atom, then 32 bytes per 16 dims
          umma_f16(tmem_s, smem_desc_sw128(sQ + off), smem_desc_sw128(kt + off), idesc_qk, k != 0);
        }
        umma_commit(s_ready);
      };
      ok = mbar_wait(q_ready, 0) && mbar_wait(kv_full, 0);
      if (ok) {
        tc_fence_after();
        issue_qk(0);
      }
      for (int j = 0; j < ntiles && ok; ++j) {
        ok = mbar_wait(p_ready, j & 1);
        if (ok && j > 0) ok = mbar_wait(o_free, (j - 1) & 1);
        if (!ok) break;
        tc_fence_after();
        const uint32_t vt = sK + (j % NS) * 2 * S::kKBytes + S::kKBytes;
#pragma unroll
        for (int k = 0; k < kKeys / 16; ++k) {
          const uint32_t poff = (k / 4) * (kRows * 128) + (k % 4) * 32;  // P: keys are its K axis
          umma_f16(tmem_o, smem_desc_sw128(sP + poff), smem_desc_mn_sw128(vt + k * 2048, kKeys * 128), idesc_pv, k != 0);
        }
        umma_commit(o_ready);
        umma_commit(kv_empty + 8 * (j % NS));
        if (j + 1 < ntiles) {
          ok = mbar_wait(kv_full + 8 * ((j + 1) % NS), ((j + 1) / NS) & 1);
          if (!ok) break;
          tc_fence_after();
          issue_qk(j + 1);
        }
      }
      if (!ok) atomicExch(status, 12);
    }
  } else {
    // ---- softmax, accumulation, epilogue: one thread per row ----
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int head = h0 + (row >> 6);
    const int rr = min(row & 63, nrows - 1);
    const int p = pos0 + rr;
    {  // Q row -> fp16 -> swizzled A operand
      const float* src = q + static_cast<long long>(t0 + rr) * q_stride + head * D;
#pragma unroll
      for (int c = 0; c < D / 8; ++c) {
        const float4 a = *reinterpret_cast<const float4*>(src + c * 8);
        const float4 b = *reinterpret_cast<const float4*>(src + c * 8 + 4);
        uint4 v;
        v.x = pack_half2(a.x, a.y);
        v.y = pack_half2(a.z, a.w);
        v.z = pack_half2(b.x, b.y);
        v.w = pack_half2(b.z, b.w);
        *reinterpret_cast<uint4*>(gen + (sQ - base) + (c / 8) * (kRows * 128) + row * 128 + (((c & 7) ^ (row & 7)) << 4)) = v;
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(q_ready);
    }
    float acc[D];
#pragma unroll
    for (int d = 0; d < D; ++d) acc[d] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    for (int j = 0; j < ntiles && ok; ++j) {
      ok = mbar_wait(s_ready, j & 1);
      if (!ok) break;
      tc_fence_after();
      const int key0 = j * kKeys;
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < kKeys / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_s + lane_sel + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (key0 + c * 32 + i <= p) mx = fmaxf(mx, __uint_as_float(v[i]));
      }
      const float m_new = fmaxf(m_run, mx * scale_log2e);
      const float corr = ex2(m_run - m_new);  // first tile: exp2(-inf) = 0
      float sum = 0.f;
#pragma unroll 1
      for (int c = 0; c < kKeys / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_s + lane_sel + c * 32, v);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int k = key0 + c * 32 + 2 * i;
          const float a = k <= p ? ex2(__uint_as_float(v[2 * i]) * scale_log2e - m_new) : 0.f;
          const float b = k + 1 <= p ? ex2(__uint_as_float(v[2 * i + 1]) * scale_log2e - m_new) : 0.f;
          sum += a + b;
          pk[i] = pack_half2(a, b);
        }
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {  // four 16-byte chunks = 32 keys of this row
          const int chunk = c * 4 + cc;   // 0..15 over the 128 keys
          *reinterpret_cast<uint4*>(gen + (sP - base) + (chunk / 8) * (kRows * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4)) =
              make_uint4(pk[4 * cc], pk[4 * cc + 1], pk[4 * cc + 2], pk[4 * cc + 3]);
        }
      }
      l_run = l_run * corr + sum;
      m_run = m_new;
      fence_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);

      ok = mbar_wait(o_ready, j & 1);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_o + lane_sel + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[c * 32 + i] = acc[c * 32 + i] * corr + __uint_as_float(v[i]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_free);
    }
    if (!ok) atomicExch(status, 13);
    if (ok && (row & 63) < nrows) {
      const float inv = 1.0f / l_run;
      __half* dst = out + static_cast<long long>(t0 + (row & 63)) * o_stride + head * D;
#pragma unroll
      for (int c = 0; c < D / 8; ++c) {
        uint4 v;
        v.x = pack_half2(acc[c * 8] * inv, acc[c * 8 + 1] * inv);
        v.y = pack_half2(acc[c * 8 + 2] * inv, acc[c * 8 + 3] * inv);
        v.z = pack_half2(acc[c * 8 + 4] * inv, acc[c * 8 + 5] * inv);
        v.w = pack_half2(acc[c * 8 + 6] * inv, acc[c * 8 + 7] * inv);
        *reinterpret_cast<uint4*>(dst + c * 8) = v;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int D>
void launch_umma_prefill_d(const AttnShape& s, const float* q, const TokenMeta& m, const int2* tiles, int n_tiles,
                           const __half* kc, const __half* vc, __half* out, cudaStream_t st) {
  using S = PfSmem<D>;
  static bool configured = false;
  auto kernel = umma_prefill_kernel<D>;
  if (!configured) {
    RB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(S::kTotal)));
    configured = true;
  }
  // The layer's pool as rows of D halves; the row count only bounds coordinates (the kernel
  // never asks for a row the block table does not name).
  const long long rows = 1LL << 31;
  const CUtensorMap mk = make_map(kc, 2, rows, D, D, 16, 64, true);
  const CUtensorMap mv = make_map(vc, 2, rows, D, D, 16, 64, true);
  const float scale_log2e = kLog2e / sqrtf(static_cast<float>(D));
  dim3 grid(n_tiles, s.heads / 2);
  count_launch();
  kernel<<<grid, kPfThreads, S::kTotal, st>>>(mk, mv, q, m, tiles, out, s.heads, s.kv_heads, s.block_size, s.q_stride,
                                              s.o_stride, scale_log2e, status_word());
}

}  // namespace

bool umma_prefill_usable(const AttnShape& s, const float* q, const __half* kc, const __half* vc, const __half* out) {
  static const bool off = [] {
    const char* e = std::getenv("RB200_PREFILL");
    return e && std::string(e) == "mma_sync";
  }();
  if (off) return false;
  if (!(s.D == 64 || s.D == 128) || s.kv_heads <= 0 || s.heads % s.kv_heads != 0) return false;
  const int G = s.heads / s.kv_heads;
  return G % 2 == 0 && s.block_size % 16 == 0 && s.q_stride % 4 == 0 && s.o_stride % 8 == 0 &&
         (reinterpret_cast<uintptr_t>(q) & 15) == 0 && (reinterpret_cast<uintptr_t>(kc) & 15) == 0 &&
         (reinterpret_cast<uintptr_t>(vc) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
}

void launch_umma_prefill(const AttnShape& s, const float* q, const TokenMeta& m, const int2* tiles, int n_tiles,
                         const __half* kc, const __half* vc, __half* out, cudaStream_t st) {
  if (n_tiles == 0) return;
  if (s.D == 64) launch_umma_prefill_d<64>(s, q, m, tiles, n_tiles, kc, vc, out, st);
  else launch_umma_prefill_d<128>(s, q, m, tiles, n_tiles, kc, vc, out, st);
}

}  // namespace rb200
