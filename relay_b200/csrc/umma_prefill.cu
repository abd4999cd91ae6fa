// Causal flash attention for prompt chunks on tcgen05 tensor cores (replaces the WMMA
// flash_prefill_kernel of the reference, engine/src/cuda_kernels.cuh:51-178, for head sizes
// 64 and 128 with an even number of query heads per KV head and block sizes that are
// multiples of 16; other layouts stay on prefill_flash_kernel in attention.cu).
//
// One CTA = one prefill tile (up to 64 query positions, engine/src/cuda_backend.cu:533-545)
// of TWO query heads that share a KV head: 128 rows on the M axis of tcgen05.mma, so every
// K/V tile fetched is used by both heads. Per 128-key tile:
//   S = Q K^T    A = Q (fp16, shared memory, K-major, 128-byte swizzle), B = the K tile
//                (K-major), D = S in TMEM (128 lanes x 128 columns, fp32), double-buffered so
//                that the scores of tile j + 1 are computed while tile j is in softmax;
//   softmax      eight warps, two threads per row, one per 64-key half of the tile, each with
//                its own running (max, sum, O): tcgen05.ld the half row of S, scale, causal
//                mask, P = exp2(.) as fp16 into shared memory in the A-operand layout;
//   O_h = P_h V_h  one product per half: A = P_h, B = the V tile's 64 keys as they sit in
//                shared memory ([key][d] = MN-major), D = O_h in TMEM;
//   O = O * corr + O_h  in the softmax threads' registers (tcgen05.ld of O_h).
// The two halves of a row are merged once, at the end (log-sum-exp), through shared memory.
// Warp roles: warps 0 and 1 gather the K and the V tile (16-byte async copies that follow the
// block table, swizzle applied by hand: a tile's rows come from eight scattered 16-key pages,
// and one small TMA box per page was measured slower than the copies), warp 2 issues the
// MMAs and owns TMEM, warps 4-11 softmax / accumulate / epilogue.
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
constexpr int kPfThreads = 384;  // K loader, V loader, MMA issuer, one idle warp, 8 softmax warps
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
  static constexpr int kStages = D == 64 ? 3 : 2;
  static constexpr int kBarBytes = 256;
  static constexpr size_t kTotal = kQBytes + static_cast<size_t>(kStages) * 2 * kKBytes + kPBytes + kBarBytes + 1024;
};

// Barrier for the 256 softmax threads only (the producer and MMA warps do not take part).
__device__ __forceinline__ void softmax_bar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

template <int D>
__global__ void __launch_bounds__(kPfThreads, 1)
umma_prefill_kernel(const __half* __restrict__ kc, const __half* __restrict__ vc, const float* __restrict__ q, TokenMeta m, const int2* __restrict__ tiles,
                    __half* __restrict__ out, int heads, int kv_heads, int bs, int q_stride, int o_stride,
                    float scale_log2e, int* __restrict__ status) {
  using S = PfSmem<D>;
  constexpr int NS = S::kStages;
  // TMEM columns: S of even tiles 0..127, S of odd tiles 128..255, then the two halves' P V
  // products (keys 0-63 and 64-127 of a tile), D columns each.
  constexpr uint32_t kTmemCols = 512;
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  unsigned char* gen = smem_dyn + (base - smem_u32(smem_dyn));
  const uint32_t sQ = base;
  const uint32_t sK = sQ + S::kQBytes;                 // NS stages of [K tile][V tile]
  const uint32_t sP = sK + NS * 2 * S::kKBytes;
  const uint32_t bars = sP + S::kPBytes;
  const uint32_t kv_full = bars, kv_empty = bars + 24;                          // NS (<= 3) x 8 bytes each
  const uint32_t s_ready = bars + 48;                                           // one per S buffer
  const uint32_t p_ready = bars + 64, o_ready = bars + 80, o_free = bars + 96;  // one per half
  const uint32_t q_ready = bars + 112;
  const uint32_t tmem_slot = bars + 120;

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
    for (int s = 0; s < NS; ++s) {
      mbar_init(kv_full + 8 * s, 2);  // the K loader and the V loader
      mbar_init(kv_empty + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(s_ready + 8 * s, 1);
      mbar_init(p_ready + 8 * s, 4);
      mbar_init(o_ready + 8 * s, 1);
      mbar_init(o_free + 8 * s, 4);
    }
    mbar_init(q_ready, 8);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(gen + (tmem_slot - base));

  bool ok = true;
  if (warp < 2) {
    // ---- loaders: warp 0 gathers the K tile, warp 1 the V tile, 16 bytes per lane and copy.
    //      A tile's rows come from 8 pages (16 keys each) that the block table scatters over
    //      the pool; async copies with the swizzle applied by hand move them faster than
    //      one small TMA box per page would. A tile is published one tile late, after its
    //      copies have landed and been made visible to the tensor core's proxy, so two
    //      tiles' copies are in flight while the warp issues the next. ----
    constexpr int CH = D / 8;              // 16-byte chunks per row
    constexpr int RPI = 32 / CH;           // rows one warp instruction covers
    const __half* pool = warp == 0 ? kc : vc;
    const int c = lane % CH, rsub = lane / CH;
    auto publish = [&](int j) {
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(kv_full + 8 * (j % NS));
    };
    int published = -1;  // last tile handed to the MMA warp
    for (int j = 0; j < ntiles && ok; ++j) {
      const int s = j % NS;
      const uint32_t free_parity = ((j / NS) & 1) ^ 1;
      // Never sleep on a stage with a landed tile still unpublished: the consumer that frees
      // the stage may itself be waiting for that tile.
      if (published < j - 1 && !__all_sync(0xffffffffu, mbar_test(kv_empty + 8 * s, free_parity))) {
        cp_async_wait<0>();
        publish(j - 1);
        published = j - 1;
      }
      ok = mbar_wait(kv_empty + 8 * s, free_parity);
      if (!ok) break;
      const uint32_t dst0 = sK + s * 2 * S::kKBytes + (warp == 0 ? 0 : S::kKBytes) + (c / 8) * (kKeys * 128);
#pragma unroll 1
      for (int pg = 0; pg < kKeys / 16; ++pg) {
        const int key0 = j * kKeys + pg * 16;
        const bool page_ok = key0 < nk;
        long long page_base = 0;
        if (page_ok) {
          const int blk = table[key0 / bs], slot = key0 % bs;
          page_base = (static_cast<long long>(blk) * kv_heads + kvh) * bs * D + static_cast<long long>(slot) * D;
        }
#pragma unroll
        for (int ii = 0; ii < 16 / RPI; ++ii) {
          const int rl = ii * RPI + rsub, r = pg * 16 + rl;  // row in the page, row in the tile
          const int bytes = key0 + rl < nk ? 16 : 0;          // keys past the context: zeros
          cp_async16_zfill(dst0 + r * 128 + (((c & 7) ^ (r & 7)) << 4), pool + page_base + (bytes ? rl * D + c * 8 : 0), bytes);
        }
      }
      cp_async_commit();
      if (published < j - 1) {  // the usual case: tile j - 1 lands while tile j's copies are issued
        cp_async_wait<1>();
        publish(j - 1);
        published = j - 1;
      }
    }
    cp_async_wait<0>();
    if (ok && published < ntiles - 1) publish(ntiles - 1);
    if (!ok && lane == 0) atomicExch(status, 11);
  } else if (warp == 2) {
    // ---- MMA issuer ----
    if (elect_one()) {
      constexpr uint32_t idesc_qk = umma_idesc(kRows, kKeys);
      constexpr uint32_t idesc_pv = umma_idesc(kRows, D) | (1u << 16);  // B (V) is MN-major
      // S of tile j goes to buffer j % 2, so the scores of tile j + 1 are computed while the
      // softmax warps still work on tile j.
      auto issue_qk = [&](int j) {
        const uint32_t kt = sK + (j % NS) * 2 * S::kKBytes;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * (kRows * 128) + (k % 4) * 32;  // 64-wide atom, then 32 bytes per 16 dims
          umma_f16(tmem_base + (j & 1) * kKeys, smem_desc_sw128(sQ + off), smem_desc_sw128(kt + off), idesc_qk, k != 0);
        }
        umma_commit(s_ready + 8 * (j & 1));
      };
      ok = mbar_wait(q_ready, 0) && mbar_wait(kv_full, 0);
      if (ok) {
        tc_fence_after();
        issue_qk(0);
      }
      if (ok && ntiles > 1) {
        ok = mbar_wait(kv_full + 8 * (1 % NS), (1 / NS) & 1);
        if (ok) {
          tc_fence_after();
          issue_qk(1);
        }
      }
      for (int j = 0; j < ntiles && ok; ++j) {
        const uint32_t vt = sK + (j % NS) * 2 * S::kKBytes + S::kKBytes;
#pragma unroll 1
        for (int h = 0; h < 2 && ok; ++h) {  // keys 0-63, then 64-127: separate products, separate softmax states
          ok = mbar_wait(p_ready + 8 * h, j & 1);
          if (ok && j > 0) ok = mbar_wait(o_free + 8 * h, (j - 1) & 1);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16(tmem_base + 2 * kKeys + h * D, smem_desc_sw128(sP + h * (kRows * 128) + k * 32),
                     smem_desc_mn_sw128(vt + (h * 4 + k) * 2048, kKeys * 128), idesc_pv, k != 0);
          umma_commit(o_ready + 8 * h);
        }
        if (!ok) break;
        umma_commit(kv_empty + 8 * (j % NS));
        if (j + 2 < ntiles) {  // both halves have read S of tile j: its buffer takes tile j + 2
          ok = mbar_wait(kv_full + 8 * ((j + 2) % NS), ((j + 2) / NS) & 1);
          if (!ok) break;
          tc_fence_after();
          issue_qk(j + 2);
        }
      }
      if (!ok) atomicExch(status, 12);
    }
  } else if (warp >= 4) {
    // ---- softmax, accumulation, epilogue: two threads per row, one per 64-key half of a tile,
    //      each with its own running (max, sum, O); the halves are merged once at the end ----
    const int half = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int head = h0 + (row >> 6);
    const int rr = min(row & 63, nrows - 1);
    const int p = pos0 + rr;
    {  // Q row -> fp16 -> swizzled A operand (each half converts half of the row's chunks)
      const float* src = q + static_cast<long long>(t0 + rr) * q_stride + head * D;
#pragma unroll
      for (int cc = 0; cc < D / 16; ++cc) {
        const int c = half * (D / 16) + cc;
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
    const uint32_t tmem_o = tmem_base + 2 * kKeys + half * D + lane_sel;
    for (int j = 0; j < ntiles && ok; ++j) {
      ok = mbar_wait(s_ready + 8 * (j & 1), (j >> 1) & 1);
      if (!ok) break;
      tc_fence_after();
      const int key0 = j * kKeys + half * 64;
      uint32_t sv[64];
      tmem_ld32(tmem_base + (j & 1) * kKeys + lane_sel + half * 64, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
      tmem_ld32(tmem_base + (j & 1) * kKeys + lane_sel + half * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
      tmem_ld_wait();
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 64; ++i)
        if (key0 + i <= p) mx = fmaxf(mx, __uint_as_float(sv[i]));
      const float m_new = fmaxf(m_run, mx * scale_log2e);
      // nothing visible to this half yet: keep everything at zero (exp2(-inf - -inf) would be NaN)
      const float corr = m_new == -INFINITY ? 1.f : ex2(m_run - m_new);
      float sum = 0.f;
#pragma unroll
      for (int cc = 0; cc < 8; ++cc) {  // eight 16-byte chunks = this half's 64 keys
        uint32_t pk[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int e = cc * 8 + 2 * i;
          const float a = key0 + e <= p ? ex2(__uint_as_float(sv[e]) * scale_log2e - m_new) : 0.f;
          const float b = key0 + e + 1 <= p ? ex2(__uint_as_float(sv[e + 1]) * scale_log2e - m_new) : 0.f;
          sum += a + b;
          pk[i] = pack_half2(a, b);
        }
        *reinterpret_cast<uint4*>(gen + (sP - base) + half * (kRows * 128) + row * 128 + ((cc ^ (row & 7)) << 4)) =
            make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      l_run = l_run * corr + sum;
      m_run = m_new;
      fence_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready + 8 * half);

      ok = mbar_wait(o_ready + 8 * half, j & 1);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_o + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[c * 32 + i] = acc[c * 32 + i] * corr + __uint_as_float(v[i]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_free + 8 * half);
    }
    if (!ok) atomicExch(status, 13);
    // Merge the two halves of each row: the second half parks (m, l, O) in the idle K/V stages
    // as [value][row] (conflict-free), the first half combines and stores.
    float* park = reinterpret_cast<float*>(gen + (sK - base));
    if (half == 1) {
      park[row] = m_run;
      park[kRows + row] = l_run;
#pragma unroll
      for (int d = 0; d < D; ++d) park[(2 + d) * kRows + row] = acc[d];
    }
    softmax_bar();
    if (half == 0 && ok && (row & 63) < nrows) {
      const float m_b = park[row], l_b = park[kRows + row];
      const float M = fmaxf(m_run, m_b);  // the first half always sees key 0, so M is finite
      const float wa = ex2(m_run - M), wb = m_b == -INFINITY ? 0.f : ex2(m_b - M);
      const float inv = 1.0f / (wa * l_run + wb * l_b);
      __half* dst = out + static_cast<long long>(t0 + (row & 63)) * o_stride + head * D;
#pragma unroll
      for (int c = 0; c < D / 8; ++c) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = (wa * acc[c * 8 + i] + wb * park[(2 + c * 8 + i) * kRows + row]) * inv;
        uint4 v;
        v.x = pack_half2(o[0], o[1]);
        v.y = pack_half2(o[2], o[3]);
        v.z = pack_half2(o[4], o[5]);
        v.w = pack_half2(o[6], o[7]);
        *reinterpret_cast<uint4*>(dst + c * 8) = v;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
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
  const float scale_log2e = kLog2e / sqrtf(static_cast<float>(D));
  dim3 grid(n_tiles, s.heads / 2);
  count_launch();
  kernel<<<grid, kPfThreads, S::kTotal, st>>>(kc, vc, q, m, tiles, out, s.heads, s.kv_heads, s.block_size, s.q_stride,
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
