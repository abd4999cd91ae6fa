// Causal flash attention for prompt chunks on tcgen05 tensor cores (replaces the WMMA
// flash_prefill_kernel of the reference, engine/src/cuda_kernels.cuh:51-178, for head sizes
// 64 and 128 with an even number of query heads per KV head and block sizes that are
// multiples of 16; other layouts stay on prefill_flash_kernel in attention.cu).
//
// One CTA = one prefill tile (up to 64 query positions, engine/src/cuda_backend.cu:533-545)
// of TWO query heads that share a KV head: 128 rows on the M axis of tcgen05.mma, so every
// K/V tile fetched is used by both heads. Per 128-key tile:
//   S = Q K^T    A = Q (fp16, shared memory, K-major, 128-byte swizzle), B = the K tile
//                (K-major), D = S in TMEM (128 lanes x 128 columns, fp32). One buffer: the
//                softmax warps release it as soon as they hold the scores in registers, and
//                the product for tile j + 1 runs under the exponentials of tile j;
//   softmax      eight warps, two threads per row, one per 64-key half of the tile, each with
//                its own running (reference max, sum): tcgen05.ld the half row of S, scale,
//                causal mask (only on tiles that reach the diagonal), P = exp2(.) as fp16
//                written with tcgen05.st into one of two P buffers in TMEM;
//   O_h += P_h V_h  one product per half: A = P_h read from TMEM, B = the V tile's 64 keys as
//                they sit in shared memory ([key][d] = MN-major), D = O_h accumulating in TMEM.
// O never leaves TMEM inside the loop. The exponent's reference max only moves when a row's
// max has grown by more than 2^8 (any lane of the warp), and only then the warp waits for the
// previous product and rescales its O_h in TMEM; P stays below 2^8 and exact in the final
// quotient. So the softmax warps go from tile j straight to tile j + 1 while the tensor core
// does P V of tile j and Q K^T of tile j + 2, and no product waits for the other's operands.
// The two halves of a row are merged once, at the end (log-sum-exp), through shared memory.
// Warp roles: warps 0, 1 and 3 fetch the K and V tiles (one TMA box per 16-key page and 64-wide
// slice of the head, addressed through the block table), warp 2 issues the MMAs and owns
// TMEM, warps 4-11 softmax / epilogue.
//
// Every mbarrier wait is bounded in time; a wait that gives up records a code in the
// device's status word (tc::status_word) and the CTA still frees its TMEM and exits.
#include <cuda.h>

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
constexpr int kPfThreads = 384;  // two loader warps, MMA issuer, third loader warp, 8 softmax warps
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
  static constexpr int kStages = D == 64 ? 4 : 3;
  static constexpr int kBarBytes = 256;
  static constexpr size_t kTotal = kQBytes + static_cast<size_t>(kStages) * 2 * kKBytes + kBarBytes + 1024;
};

// Programmatic dependent launch (common.cuh): everything the kernel ahead may have written (Q, the
// K/V pages) is read only after pdl_wait(); the batch metadata (tiles, positions, block tables)
// was uploaded before the first kernel of the pass and is read before it.

// Barrier for the 256 softmax threads only (the producer and MMA warps do not take part).
__device__ __forceinline__ void softmax_bar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

template <int D>
__global__ void __launch_bounds__(kPfThreads, 1)
umma_prefill_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const __half* __restrict__ kc, const __half* __restrict__ vc, const float* __restrict__ q, TokenMeta m, const int2* __restrict__ tiles,
                    __half* __restrict__ out, int heads, int kv_heads, int bs, int q_stride, int o_stride,
                    float scale_log2e, int* __restrict__ status) {
  using S = PfSmem<D>;
  constexpr int NS = S::kStages;
  // how far (log2) a row's max may outgrow the exponent reference before O is rescaled
  constexpr float kGrow = 8.f;
  // TMEM columns: S 0..127 (single buffer: it is free again as soon as the softmax warps hold
  // it in registers), P of even tiles 128..191 and of odd tiles 192..255 (fp16 pairs: 32
  // columns per half), then the two halves' running O (keys 0-63 and 64-127 of every tile),
  // D columns each.
  constexpr uint32_t kTmemCols = 512;
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  unsigned char* gen = smem_dyn + (base - smem_u32(smem_dyn));
  const uint32_t sQ = base;
  const uint32_t sK = sQ + S::kQBytes;                 // NS stages of [K tile][V tile]
  const uint32_t bars = sK + NS * 2 * S::kKBytes;
  const uint32_t kv_full = bars, kv_empty = bars + 32;     // NS (<= 4) x 8 bytes each
  const uint32_t s_ready = bars + 64, s_free = bars + 72;  // S written by the MMA / read into registers by all 8 warps
  const uint32_t p_ready = bars + 80, pv_done = bars + 96;  // one per half
  const uint32_t q_ready = bars + 112;
  const uint32_t tmem_slot = bars + 120;

  pdl_trigger();
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
      mbar_init(kv_full + 8 * s, 1);  // the loader's expect-tx arrival (or its plain arrival after a gathered tile)
      mbar_init(kv_empty + 8 * s, 1);
    }
    mbar_init(s_ready, 1);
    mbar_init(s_free, 8);
    for (int s = 0; s < 2; ++s) {
      mbar_init(p_ready + 8 * s, 4);
      mbar_init(pv_done + 8 * s, 1);
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
  if (warp < 2 || warp == 3) {
    // ---- loaders: a tile's 128 keys come from 8 pages (16 keys each) that the block table
    //      scatters over the pool. One TMA box per page and 64-wide slice of the head (16 rows
    //      x 128 bytes, 128-byte swizzle), completing on the stage's mbarrier. Issuing a box
    //      costs the issuing warp some 90 cycles whatever its size, so the 16 (D = 64) or 32
    //      boxes of a tile are dealt round-robin to three warps, one box per lane.
    //      Block-table entries are read 32 pages (four tiles) at a time, one per lane, a
    //      group ahead of their use, so no copy waits for a table lookup. A last tile that
    //      reaches past the context is gathered by warp 0 with 16-byte async copies
    //      instead, which write zeros for the missing keys (the pool may hold anything
    //      there, and 0 x NaN would poison P V). ----
    constexpr int kAtoms = D / 64;
    constexpr int kBoxes = 2 * 8 * kAtoms;  // K then V; per operand: [64-wide slice][page]
    const int li = warp == 3 ? 2 : warp;    // loader index 0..2
    const int box = li + 3 * lane;          // this lane's box of every tile
    const bool has_box = box < kBoxes;
    const int box_pg = box & 7, box_atom = (box >> 3) % kAtoms, box_v = box / (8 * kAtoms);
    auto load_group = [&](int g) {  // first pool row ([block][kv head][slot]) of this lane's page
      const int key0 = (g * 4 + lane / 8) * kKeys + (lane % 8) * 16;
      if (key0 >= nk) return 0;
      return (table[key0 / bs] * kv_heads + kvh) * bs + key0 % bs;
    };
    int tab_cur = 0, tab_next = load_group(0);
    pdl_wait();
    for (int j = 0; j < ntiles && ok; ++j) {
      const int s = j % NS;
      if (j % 4 == 0) {
        tab_cur = tab_next;
        tab_next = load_group(j / 4 + 1);
      }
      ok = __all_sync(0xffffffffu, mbar_wait(kv_empty + 8 * s, ((j / NS) & 1) ^ 1));
      if (!ok) break;
      const uint32_t kdst = sK + s * 2 * S::kKBytes;
      if ((j + 1) * kKeys <= nk) {
        const int row = __shfl_sync(0xffffffffu, tab_cur, (j % 4) * 8 + box_pg);
        if (warp == 0 && lane == 0) mbar_expect_tx(kv_full + 8 * s, 2 * S::kKBytes);
        if (has_box)
          tma_load_2d(kdst + box_v * S::kKBytes + box_atom * (kKeys * 128) + box_pg * 2048, box_v ? &map_v : &map_k,
                      box_atom * 64, row, kv_full + 8 * s);
      } else if (warp == 0) {
        constexpr int CH = D / 8;     // 16-byte chunks per row
        constexpr int RPI = 32 / CH;  // rows one warp instruction covers
        const int c = lane % CH, rsub = lane / CH;
#pragma unroll 1
        for (int pg = 0; pg < 2 * (kKeys / 16); ++pg) {  // K pages, then V pages
          const long long src_row = __shfl_sync(0xffffffffu, tab_cur, (j % 4) * 8 + (pg & 7));
          const __half* src = (pg < 8 ? kc : vc) + src_row * D;
          const uint32_t dst = kdst + (pg < 8 ? 0 : S::kKBytes) + (pg & 7) * 2048 + (c / 8) * (kKeys * 128);
#pragma unroll
          for (int ii = 0; ii < 16 / RPI; ++ii) {
            const int rl = ii * RPI + rsub;
            const int bytes = j * kKeys + (pg & 7) * 16 + rl < nk ? 16 : 0;
            cp_async16_zfill(dst + rl * 128 + (((c & 7) ^ (rl & 7)) << 4), src + (bytes ? rl * D + c * 8 : 0), bytes);
          }
        }
        cp_async_commit();
        cp_async_wait<0>();
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(kv_full + 8 * s);
      }
    }
    if (!ok && lane == 0) atomicExch(status, 11);
  } else if (warp == 2) {
    // ---- MMA issuer ----
    if (elect_one()) {
      constexpr uint32_t idesc_qk = umma_idesc(kRows, kKeys);
      constexpr uint32_t idesc_pv = umma_idesc(kRows, D) | (1u << 16);  // B (V) is MN-major
      // Q K^T of tile j + 1 is issued as soon as the softmax warps have taken S of tile j into
      // registers, so it runs under their exponentials; P V of tile j follows when P arrives
      // and runs under the softmax of tile j + 1. Neither product waits for the other's data.
      auto issue_qk = [&](int j) {
        const uint32_t kt = sK + (j % NS) * 2 * S::kKBytes;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * (kRows * 128) + (k % 4) * 32;  // 64-wide atom, then 32 bytes per 16 dims
          umma_f16(tmem_base, smem_desc_sw128(sQ + off), smem_desc_sw128(kt + off), idesc_qk, k != 0);
        }
        umma_commit(s_ready);
      };
      ok = mbar_wait(q_ready, 0) && mbar_wait(kv_full, 0);
      if (ok) {
        tc_fence_after();
        issue_qk(0);
      }
      for (int j = 0; j < ntiles && ok; ++j) {
        if (j + 1 < ntiles) {
          ok = mbar_wait(s_free, j & 1) && mbar_wait(kv_full + 8 * ((j + 1) % NS), ((j + 1) / NS) & 1);
          if (!ok) break;
          tc_fence_after();
          issue_qk(j + 1);
        }
        const uint32_t vt = sK + (j % NS) * 2 * S::kKBytes + S::kKBytes;
#pragma unroll 1
        for (int h = 0; h < 2 && ok; ++h) {  // keys 0-63, then 64-127: separate products, separate softmax states
          ok = mbar_wait(p_ready + 8 * h, j & 1);
          if (!ok) break;
          tc_fence_after();
          const uint32_t pa = tmem_base + kKeys + (j & 1) * 64 + h * 32;  // P_h: 64 halves = 32 columns per row
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16_ta(tmem_base + 2 * kKeys + h * D, pa + 8 * k, smem_desc_mn_sw128(vt + (h * 4 + k) * 2048, kKeys * 128),
                        idesc_pv, (j > 0) || (k != 0));
          umma_commit(pv_done + 8 * h);
        }
        if (!ok) break;
        umma_commit(kv_empty + 8 * (j % NS));
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
    pdl_wait();
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
    float m_ref = -INFINITY, l_run = 0.f;  // m_ref: the max the exponents refer to (log2 domain)
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tmem_o = tmem_base + 2 * kKeys + half * D + lane_sel;
    for (int j = 0; j < ntiles && ok; ++j) {
      ok = __all_sync(0xffffffffu, mbar_wait(s_ready, j & 1));
      if (!ok) break;
      tc_fence_after();
      const int key0 = j * kKeys + half * 64;
      const uint32_t tmem_s = tmem_base + lane_sel + half * 64;
      const uint32_t tmem_p = tmem_base + kKeys + (j & 1) * 64 + half * 32 + lane_sel;
      uint32_t sv[64];
      tmem_ld32(tmem_s, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
      tmem_ld32(tmem_s + 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free);  // the scores are in registers: S may take the next tile
      const bool diag = j * kKeys + kKeys - 1 > pos0;  // some row of the tile does not see every key
      if (diag) {
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (key0 + i > p) sv[i] = __float_as_uint(-INFINITY);
      }
      // Exponentials against the current reference, with the row maximum gathered in the same
      // pass (four chains each, not one 64-deep): the maximum is only needed to notice that a
      // row outgrew the reference, and then the pass is repeated.
      uint32_t pk[32];
      float sum = 0.f, mx = 0.f;
      auto exp_pass = [&](float neg_m) {
        // packed fp32 pairs (fma.rn.f32x2 / add.f32x2) halve the instruction count of the scale and the sum
        float2 sum2[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        const float2 sc2 = make_float2(scale_log2e, scale_log2e), nm2 = make_float2(neg_m, neg_m);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float2 sp = make_float2(__uint_as_float(sv[2 * i]), __uint_as_float(sv[2 * i + 1]));
          const float2 x = __ffma2_rn(sp, sc2, nm2);
          const float2 e = make_float2(ex2(x.x), ex2(x.y));
          mx4[i & 3] = fmaxf(mx4[i & 3], fmaxf(sp.x, sp.y));
          sum2[i & 3] = __fadd2_rn(sum2[i & 3], e);
          pk[i] = pack_half2(e.x, e.y);
        }
        const float2 st = __fadd2_rn(__fadd2_rn(sum2[0], sum2[1]), __fadd2_rn(sum2[2], sum2[3]));
        sum = st.x + st.y;
        mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      };
      // rows that see nothing yet keep m_ref = -inf; all their scores are masked to -inf
      exp_pass(m_ref == -INFINITY ? 0.f : -m_ref);
      const float m_cand = mx * scale_log2e;
      if (__any_sync(0xffffffffu, m_cand > m_ref + kGrow)) {
        // a row outgrew the reference by 2^8 (always so on a row's first visible tile): move every
        // row's reference to its exact max, rescale what has been accumulated (nothing yet on
        // the first tile) and redo the exponentials
        const float m_new = fmaxf(m_ref, m_cand);
        const float corr = m_new == -INFINITY ? 1.f : ex2(m_ref - m_new);
        if (j > 0) {
          ok = __all_sync(0xffffffffu, mbar_wait(pv_done + 8 * half, (j - 1) & 1));
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t v[32];
            tmem_ld32(tmem_o + c * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
            tmem_st32(tmem_o + c * 32, v);
          }
        }
        l_run *= corr;
        m_ref = m_new;
        exp_pass(m_ref == -INFINITY ? 0.f : -m_ref);
      }
      l_run += sum;
      // Arrive for tile j only after this half's product of tile j - 1 has completed (normally
      // long ago). The MMA warp looks at the halves in turn; without this a half could arrive
      // for two tiles while the MMA warp waits for the other half, and a phase that completes
      // twice unobserved looks incomplete to a parity wait. It also keeps the four warps that
      // share p_ready (four arrivals per tile) within one tile of each other, and it means the
      // product of tile j - 2, the last reader of this tile's P buffer, is done.
      if (j > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(pv_done + 8 * half, (j - 1) & 1));
        if (!ok) break;
      }
      tmem_st32(tmem_p, pk);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready + 8 * half);
    }
    if (ok) {
      ok = __all_sync(0xffffffffu, mbar_wait(pv_done + 8 * half, (ntiles - 1) & 1));
      tc_fence_after();
    }
    if (!ok) atomicExch(status, 13);
    // Merge the two halves of each row: the second half parks (m, l, O) in the idle K/V stages
    // as [value][row] (conflict-free), the first half combines and stores.
    float* park = reinterpret_cast<float*>(gen + (sK - base));
    if (half == 1 && ok) {
      park[row] = m_ref;
      park[kRows + row] = l_run;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_o + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) park[(2 + c * 32 + i) * kRows + row] = __uint_as_float(v[i]);
      }
    }
    softmax_bar();
    if (half == 0 && ok) {
      const float m_b = park[row], l_b = park[kRows + row];
      const float M = fmaxf(m_ref, m_b);  // the first half always sees key 0, so M is finite
      const float wa = ex2(m_ref - M), wb = m_b == -INFINITY ? 0.f : ex2(m_b - M);
      const float inv = 1.0f / (wa * l_run + wb * l_b);
      const bool live = (row & 63) < nrows;
      __half* dst = out + static_cast<long long>(t0 + (row & 63)) * o_stride + head * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_o + c * 32, v);  // every lane takes part in the load; only live rows store
        tmem_ld_wait();
        if (live) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
              o[i] = (wa * __uint_as_float(v[g * 8 + i]) + wb * park[(2 + c * 32 + g * 8 + i) * kRows + row]) * inv;
            uint4 w;
            w.x = pack_half2(o[0], o[1]);
            w.y = pack_half2(o[2], o[3]);
            w.z = pack_half2(o[4], o[5]);
            w.w = pack_half2(o[6], o[7]);
            *reinterpret_cast<uint4*>(dst + c * 32 + g * 8) = w;
          }
        }
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
  static PerDeviceOnce once;
  auto kernel = umma_prefill_kernel<D>;
  if (once.first())
    RB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(S::kTotal)));
  // The layer's pool as rows of D halves, box = one 16-key page x 64 dims. With the pool's real
  // row count a page outside it reads as zeros; callers that do not know it get a bound that only
  // limits the coordinates (the kernel never asks for a row the block table does not name).
  const long long rows = s.pool_rows > 0 ? s.pool_rows : (1LL << 31);
  const CUtensorMap mk = make_map(kc, 2, rows, D, D, 16, 64, true);
  const CUtensorMap mv = make_map(vc, 2, rows, D, D, 16, 64, true);
  const float scale_log2e = kLog2e / sqrtf(static_cast<float>(D));
  dim3 grid(n_tiles, s.heads / 2);
  count_launch();
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kPfThreads);
  cfg.dynamicSmemBytes = S::kTotal;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // set-up may overlap the previous kernel's tail
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const int heads = s.heads, kv_heads = s.kv_heads, bs = s.block_size, q_stride = s.q_stride, o_stride = s.o_stride;
  int* status = status_word();
  RB_CUDA(cudaLaunchKernelEx(&cfg, kernel, mk, mv, kc, vc, q, m, tiles, out, heads, kv_heads, bs, q_stride, o_stride, scale_log2e,
                             status));
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
