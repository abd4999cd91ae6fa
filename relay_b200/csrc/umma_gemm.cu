// Tensor-core GEMM for more than 8 tokens on Blackwell's fifth-generation tensor cores:
//   y[T,N] = x[T,K] W[N,K]^T (+ beta*y),  W fp16 or int8 with a per-row scale.
// Replaces the reference's cublasGemmEx call (engine/src/cuda_backend.cu:724-730) and its
// dequantise-then-cuBLAS path for int8 (engine/src/cuda_kernels.cuh:432-436,
// engine/src/cuda_backend.cu:719-721).
//
// Shape of one CTA: 128 weight rows (the M axis of tcgen05.mma, one TMEM lane per row) by BN
// tokens (the N axis, one TMEM column per token), K in blocks of 64 halves = one 128-byte
// swizzle atom. Six warps with fixed roles (ten with int8 weights):
//   warp 0   TMA producer: one elected lane streams the weight tile and the activation tile
//            of each k block into a ring of shared-memory stages (cp.async.bulk.tensor,
//            128-byte swizzle, completion on an mbarrier);
//   warp 1   MMA issuer: one elected lane issues four tcgen05.mma (K = 16 each) per k block
//            on shared-memory descriptors, accumulating in TMEM, and releases each stage
//            with tcgen05.commit; it also owns the TMEM allocation;
//   warps 2-5  epilogue: read the accumulator with tcgen05.ld (each warp its own quarter of
//            the 128 lanes), apply the row scale and beta*y, store fp32 rows coalesced along
//            N.
// With int8 weights the fp16 copy of the matrix exists only in tensor memory. The producer lands
// the raw int8 tile (64-byte swizzle) in the shared-memory ring; eight converter warps (2-5 take
// the even k blocks, 6-9 the odd ones, one thread per weight row) widen 64 int8 to 64 halves
// and write them with tcgen05.st into a second ring of 32-column TMEM slots; the MMA issuer
// takes the A operand from that TMEM slot and the activation tile from shared memory. The two
// rings are released separately (raw stage by the converters, TMEM slot and activation tile
// by tcgen05.commit), so HBM loads run ahead of the conversion by the depth of the smem ring.
// Weight bytes are read from HBM once per token tile; activations come from L2.
//
// Matrices with few 128-row tiles (the attention output and down projections have 32) would
// leave most SMs idle, so K is split across a thread-block cluster: each CTA of the cluster
// accumulates its k range in its own TMEM, parks the partial tile in its shared memory, and
// after a cluster barrier every CTA adds one slice of the tile from all members' shared
// memory over DSMEM in a fixed order (deterministic, no atomics, no global scratch).
//
// Every mbarrier wait is bounded: on exhaustion the kernel records a code in `status`,
// stops issuing work, and still releases its TMEM before it returns.
#include <cuda.h>

#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "kernels.h"
#include "tcgen05.cuh"

namespace rb200 {

using namespace tc;

namespace {

constexpr int kTileM = 128;
constexpr int kBlockK = 64;        // halves per k block: one 128-byte swizzle atom
constexpr int kUmmaThreads = 192;      // producer, MMA, 4 epilogue warps
constexpr int kUmmaThreadsInt8 = 320;  // + 4 more warps that only widen int8 tiles

__device__ __forceinline__ void cvt_s8x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
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

// MT = 128-row M tiles per CTA (1 or 2). Two tiles share every activation tile a CTA loads and let
// a grid of up to 256-row tiles fit the SMs in one wave where 128-row tiles need two (the
// gate/up projection at 256 tokens: 144 CTAs of 200 rows, tensor pipe active 76 %).
// fp16 weights only. With a K split the two partial tiles are exchanged one after the other (one
// alone fills the shared memory of the idle operand stages).
template <int BN, bool INT8, int MT = 1>
struct UmmaSmem {
  // Elements of K per block. int8 weights with up to 128 tokens take 128 (two swizzle atoms of
  // activations per stage): there the pace is set by the hand-offs per block, not by the MMAs.
  static constexpr int kKB = (INT8 && BN <= 128) ? 2 * kBlockK : kBlockK;
  static constexpr int kAtoms = kKB / kBlockK;                          // 128-byte activation atoms per block
  static constexpr int kAccCols = MT * (BN < 32 ? 32 : BN);             // TMEM columns of the accumulators
  static constexpr int kABytes = INT8 ? 0 : MT * kTileM * kBlockK * 2;  // fp16 operand tiles (fp16 weights only)
  static constexpr int kBBytes = BN * kKB * 2;
  static constexpr int kRawBytes = INT8 ? kTileM * kKB : 0;             // int8 tile as TMA lands it
  static constexpr int kStageBytes = kABytes + kBBytes + kRawBytes;
  // Shared-memory stages: what is in flight from HBM. int8 stages are half the size of fp16
  // ones, so there are about twice as many (up to 16).
  static constexpr int kStages = INT8 ? (180 * 1024 / kStageBytes > 16 ? 16 : 180 * 1024 / kStageBytes)
                                      : (MT == 2 ? (BN >= 256 ? 3 : 4) : (BN >= 256 ? 4 : (BN >= 128 ? 5 : (BN >= 32 ? 6 : 8))));
  // int8: the widened A tile of a k block lives in TMEM (32 columns: 64 halves per row) in a
  // ring of its own, as deep as the allocation (a power of two) allows next to the accumulator.
  static constexpr int kTmemCols = INT8 ? (BN >= 256 ? 512 : 256) : kAccCols;
  static constexpr int kASlotCols = kKB / 2;  // fp16 pairs per row of a widened block
  static constexpr int kAStages = INT8 ? (kTmemCols - kAccCols) / kASlotCols : 0;
  static constexpr int kBarBytes = 1024;
  static constexpr size_t kTotal = static_cast<size_t>(kStages) * kStageBytes + kBarBytes + 1024;  // + alignment slack
};

template <int BN, bool INT8, int MT>
__global__ void __launch_bounds__(INT8 ? kUmmaThreadsInt8 : kUmmaThreads, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                 const float* __restrict__ scale, float* __restrict__ y, int T, int N, int K, int rows, float beta,
                 int* __restrict__ status) {
  static_assert(MT == 1 || !INT8, "two M tiles per CTA: fp16 weights only");
  using S = UmmaSmem<BN, INT8, MT>;
  constexpr int NS = S::kStages;
  pdl_trigger();
  constexpr uint32_t kTmemCols = S::kTmemCols;
  constexpr uint32_t kACol0 = S::kAccCols;  // int8: TMEM column of A stage 0 (32 columns per stage)
  extern __shared__ unsigned char smem_dyn[];
  // operand tiles need 1024-byte alignment for the 128-byte swizzle pattern
  const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  const uint32_t sA = base;
  const uint32_t sB = sA + NS * S::kABytes;
  const uint32_t sRaw = sB + NS * S::kBBytes;
  const uint32_t bars = sRaw + NS * S::kRawBytes;
  constexpr int NA = S::kAStages > 0 ? S::kAStages : 1;
  const uint32_t full_bar = bars;              // NS x 8 bytes: TMA landed
  const uint32_t empty_bar = bars + 8 * NS;    // NS x 8: MMA finished reading the stage's shared memory
  const uint32_t raw_free = bars + 16 * NS;    // NS x 8: int8 only, the raw tile has been widened
  const uint32_t conv_bar = bars + 24 * NS;    // NA x 8: int8 only, A stage written to TMEM
  const uint32_t a_free = conv_bar + 8 * NA;   // NA x 8: int8 only, MMA finished reading the A stage
  const uint32_t accum_bar = a_free + 8 * NA;  // accumulator complete
  const uint32_t tmem_slot = accum_bar + 8;
  unsigned char* gen_base = smem_dyn + (base - smem_u32(smem_dyn));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // `rows` (a multiple of 8, at most 128 * MT) weight rows per CTA: the host shrinks the tile so that
  // the grid fills the SMs evenly; the MMA still spans 128 lanes and the rest is ignored.
  const int m0 = blockIdx.x * rows, tok0 = blockIdx.y * BN;
  constexpr int KB = S::kKB;
  const uint32_t stage_tx = static_cast<uint32_t>(rows) * KB * (INT8 ? 1 : 2) + S::kBBytes;
  const int splits = gridDim.z, split = blockIdx.z;  // the cluster spans z: split == rank in the cluster
  const int nk_all = (K + KB - 1) / KB;  // a last half block (K is a multiple of 64) reads zeros past K
  const int kb_begin = static_cast<int>(static_cast<long long>(nk_all) * split / splits);
  const int nk = static_cast<int>(static_cast<long long>(nk_all) * (split + 1) / splits) - kb_begin;

  const int pre = min(nk, NS);  // stages the first thread fills before the block is set up
  if (warp == 0 && lane == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(full_bar + 8 * s, 1);
      mbar_init(empty_bar + 8 * s, 1);
      mbar_init(raw_free + 8 * s, 4);
    }
    for (int a = 0; a < NA; ++a) {
      mbar_init(conv_bar + 8 * a, 4);
      mbar_init(a_free + 8 * a, 1);
    }
    mbar_init(accum_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
    // The first tiles leave for HBM before anything else is set up (TMEM, the block barrier):
    // the barriers they complete on are this thread's own work above, and the ring starts empty.
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_x)) : "memory");
    for (int kb = 0; kb < pre; ++kb) {
      mbar_expect_tx(full_bar + 8 * kb, stage_tx);
      const int kx = (kb_begin + kb) * KB;
      if (INT8) tma_load_2d(sRaw + kb * S::kRawBytes, &map_w, kx, m0, full_bar + 8 * kb);
      else tma_load_2d(sA + kb * S::kABytes, &map_w, kx, m0, full_bar + 8 * kb);
    }
    pdl_wait();  // the activations come from the kernel ahead, which may still be running
    for (int kb = 0; kb < pre; ++kb)
#pragma unroll
      for (int at = 0; at < S::kAtoms; ++at)
        tma_load_2d(sB + kb * S::kBBytes + at * (BN * 128), &map_x, (kb_begin + kb) * KB + at * kBlockK, tok0, full_bar + 8 * kb);
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
  if (warp == 0) {
    // ---- TMA producer ----
    if (elect_one()) {
      pdl_wait();
      for (int kb = pre; kb < nk && ok; ++kb) {
        const int s = kb % NS;
        ok = mbar_wait(empty_bar + 8 * s, ((kb / NS) & 1) ^ 1);
        if (INT8 && ok) ok = mbar_wait(raw_free + 8 * s, ((kb / NS) & 1) ^ 1);
        if (!ok) break;
        mbar_expect_tx(full_bar + 8 * s, stage_tx);
        const int kx = (kb_begin + kb) * KB;
        if (INT8) tma_load_2d(sRaw + s * S::kRawBytes, &map_w, kx, m0, full_bar + 8 * s);
        else tma_load_2d(sA + s * S::kABytes, &map_w, kx, m0, full_bar + 8 * s);
#pragma unroll
        for (int at = 0; at < S::kAtoms; ++at)
          tma_load_2d(sB + s * S::kBBytes + at * (BN * 128), &map_x, kx + at * kBlockK, tok0, full_bar + 8 * s);
      }
      if (!ok) atomicExch(status, 1);
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc(kTileM, BN);
      for (int kb = 0; kb < nk && ok; ++kb) {
        const int s = kb % NS;
        ok = mbar_wait(full_bar + 8 * s, (kb / NS) & 1);
        if (INT8 && ok) ok = mbar_wait(conv_bar + 8 * (kb % NA), (kb / NA) & 1);
        if (!ok) break;
        tc_fence_after();
        const uint64_t db = smem_desc_sw128(sB + s * S::kBBytes);
        if constexpr (INT8) {
          const uint32_t ta = tmem_base + kACol0 + (kb % NA) * S::kASlotCols;  // 16 halves = 8 columns per step
#pragma unroll
          for (int k4 = 0; k4 < KB / 16; ++k4)  // activations: atom k4 / 4 (BN rows x 128 bytes each), 32 bytes per step inside it
            umma_f16_ta(tmem_base, ta + 8 * k4, db + (k4 / 4) * (BN * 128 >> 4) + 2 * (k4 % 4), idesc, (kb | k4) != 0);
          umma_commit(a_free + 8 * (kb % NA));
        } else {
          const uint64_t da = smem_desc_sw128(sA + s * S::kABytes);
#pragma unroll
          for (int k4 = 0; k4 < kBlockK / 16; ++k4) {  // 16 halves = 32 bytes = 2 descriptor units per step
            umma_f16(tmem_base, da + 2 * k4, db + 2 * k4, idesc, (kb | k4) != 0);
            if constexpr (MT == 2)  // rows 128.. of the tile (16 KB further on), the same activations
              umma_f16(tmem_base + BN, da + (kTileM * kBlockK * 2 >> 4) + 2 * k4, db + 2 * k4, idesc, (kb | k4) != 0);
          }
        }
        umma_commit(empty_bar + 8 * s);  // arrives once the MMAs above have read the stage
      }
      umma_commit(accum_bar);
      if (!ok) atomicExch(status, 2);
    }
  } else {
    // ---- int8 widening (main loop), then the epilogue ----
    if constexpr (INT8) {
      // Two groups of four warps take alternate k blocks, so two blocks are widened at a time.
      // Thread = one weight row (the TMEM lane it may write): the row's KB int8 from the swizzled
      // raw tile (64-byte rows: 64-byte swizzle, 128-byte rows: 128-byte swizzle) -> KB fp16 ->
      // the KB / 2 TMEM columns of an A stage.
      constexpr int CH = KB / 16;  // 16-byte pieces of a raw row
      const int crow = (warp & 3) * 32 + lane, group = (warp - 2) >> 2;
      const int sw = CH == 4 ? ((crow >> 1) & 3) : (crow & 7);
      const uint32_t tcol = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + kACol0;
      for (int kb = group; kb < nk && ok; kb += 2) {
        const int s = kb % NS, a = kb % NA;
        ok = mbar_wait(full_bar + 8 * s, (kb / NS) & 1);
        if (!ok) break;
        const uint4* raw = reinterpret_cast<const uint4*>(gen_base + (sRaw + s * S::kRawBytes - base)) + crow * CH;
        uint4 r[CH];
#pragma unroll
        for (int c = 0; c < CH; ++c) r[c] = raw[c ^ sw];
        __syncwarp();
        if (lane == 0) mbar_arrive(raw_free + 8 * s);  // the raw tile is in registers: its stage may be refilled
        uint32_t h[CH * 8];
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          cvt_s8x4(r[c].x, h[8 * c], h[8 * c + 1]);
          cvt_s8x4(r[c].y, h[8 * c + 2], h[8 * c + 3]);
          cvt_s8x4(r[c].z, h[8 * c + 4], h[8 * c + 5]);
          cvt_s8x4(r[c].w, h[8 * c + 6], h[8 * c + 7]);
        }
        ok = mbar_wait(a_free + 8 * a, ((kb / NA) & 1) ^ 1);  // the MMA that last read this A stage is done
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int q = 0; q < CH / 4; ++q)
          tmem_st32(tcol + a * S::kASlotCols + 32 * q, *reinterpret_cast<uint32_t(*)[32]>(&h[32 * q]));
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(conv_bar + 8 * a);  // one arrival per warp
      }
      if (!ok) atomicExch(status, 3);
    }
    pdl_wait();  // y (read with beta, written always) belongs to the kernels ahead until they complete
    bool done = warp < 6 ? mbar_wait(accum_bar, 0) : true;  // warps 6-9 (int8 only) take no part in the epilogue
    if (!done) atomicExch(status, 4);
    tc_fence_after();
    const int quarter = warp & 3;  // the TMEM lane quarter this warp may read
    const int row = quarter * 32 + lane;
    if (warp >= 6) {
      // nothing: only widening warps
    } else if (splits == 1) {
      if (done && ok) {
#pragma unroll 1
        for (int a = 0; a < MT; ++a) {  // the CTA's M tiles: TMEM columns a * BN .., weight rows a * 128 ..
          const int row_a = a * kTileM + row, n_a = m0 + row_a;
          const bool live_a = row_a < rows && n_a < N;
          const float sc_a = (INT8 && live_a) ? scale[n_a] : 1.0f;
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 32) {
            uint32_t v[32];
            tmem_ld32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + a * BN + c0, v);
            tmem_ld_wait();
            if (live_a) {
              float* d0 = y + static_cast<long long>(tok0 + c0) * N + n_a;
              const int nt = min(32, T - tok0 - c0);  // valid token columns of this chunk
              if (beta != 0.f) {
                float old[32];  // all loads first, so that they are in flight together
#pragma unroll
                for (int j = 0; j < 32; ++j) old[j] = j < nt ? d0[static_cast<long long>(j) * N] : 0.f;
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (j < nt) d0[static_cast<long long>(j) * N] = __uint_as_float(v[j]) * sc_a + beta * old[j];
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (j < nt) d0[static_cast<long long>(j) * N] = __uint_as_float(v[j]) * sc_a;
              }
            }
          }
        }
      }
    }
  }
#pragma unroll 1
  for (int a = 0; a < (splits > 1 ? MT : 0); ++a) {  // the CTA's M tiles, one exchange each
    if (warp >= 2 && warp < 6) {
      // Park this CTA's partial tile as red[token][row] in the (now idle) operand stages.
      const int quarter = warp & 3, row = quarter * 32 + lane;
      float* red = reinterpret_cast<float*>(gen_base);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + a * BN + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) red[(c0 + j) * kTileM + row] = __uint_as_float(v[j]);
      }
    }
    cluster_sync_all();  // every member's partial tile is in its shared memory
    if (warp >= 2 && warp < 6) {
      // This CTA finishes `per` token columns of the tile: a thread takes four consecutive weight
      // rows of one column (16-byte DSMEM loads; the rows are contiguous in red[token][row]), the
      // four warps take the columns round-robin, the members are added in rank order.
      const int tid = threadIdx.x - 64, r4 = (tid & 31) * 4, cg = tid >> 5;
      const int n4 = m0 + a * kTileM + r4;
      const int per = (BN + splits - 1) / splits;
      const int c_begin = split * per, c_end = min(min(BN, c_begin + per), T - tok0);
      bool live[4];
      float sc[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        live[k] = a * kTileM + r4 + k < rows && n4 + k < N;
        sc[k] = (INT8 && live[k]) ? scale[n4 + k] : 1.0f;
      }
      const bool vec = (N & 3) == 0 && live[3];  // the four outputs form one aligned float4 of y
      uint32_t peer[8];
#pragma unroll
      for (int r = 0; r < 8; ++r)  // fully unrolled so that peer[] stays in registers
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer[r]) : "r"(base + static_cast<uint32_t>(r4) * 4), "r"(r < splits ? r : 0));
      for (int c = c_begin + cg; c < c_end; c += 8) {
        float4 acc[2], old[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          old[u] = acc[u];
          const int cc = c + 4 * u;
          if (beta != 0.f && cc < c_end) {
            const float* src = y + static_cast<long long>(tok0 + cc) * N + n4;
            if (vec) old[u] = *reinterpret_cast<const float4*>(src);
            else {
              if (live[0]) old[u].x = src[0];
              if (live[1]) old[u].y = src[1];
              if (live[2]) old[u].z = src[2];
              if (live[3]) old[u].w = src[3];
            }
          }
        }
#pragma unroll
        for (int r = 0; r < 8; ++r) {  // members in rank order: the sum is the same on every run
          if (r >= splits) break;
          float4 part[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            part[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c + 4 * u < c_end)
              asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                           : "=f"(part[u].x), "=f"(part[u].y), "=f"(part[u].z), "=f"(part[u].w)
                           : "r"(peer[r] + static_cast<uint32_t>((c + 4 * u) * kTileM) * 4)
                           : "memory");
          }
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            acc[u].x += part[u].x;
            acc[u].y += part[u].y;
            acc[u].z += part[u].z;
            acc[u].w += part[u].w;
          }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int cc = c + 4 * u;
          if (cc >= c_end) continue;
          float* dst = y + static_cast<long long>(tok0 + cc) * N + n4;
          const float4 v = make_float4(acc[u].x * sc[0] + beta * old[u].x, acc[u].y * sc[1] + beta * old[u].y,
                                       acc[u].z * sc[2] + beta * old[u].z, acc[u].w * sc[3] + beta * old[u].w);
          if (vec) *reinterpret_cast<float4*>(dst) = v;
          else {
            if (live[0]) dst[0] = v.x;
            if (live[1]) dst[1] = v.y;
            if (live[2]) dst[2] = v.z;
            if (live[3]) dst[3] = v.w;
          }
        }
      }
    }
    cluster_sync_all();  // nobody leaves (or parks its next tile) while a peer may still read its shared memory
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- host side --------------------------------------------------------------------------

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(p);
    else
      cudaGetLastError();
  });
  if (!fn) fail(RB200_ERR_RUNTIME, "cuTensorMapEncodeTiled is not available from this driver");
  return fn;
}

}  // namespace

// A 2-D tensor map over a row-major [rows][ld] matrix of 1- or 2-byte elements, box = [box_rows][box_cols].
CUtensorMap tc::make_map(const void* ptr, int elem_bytes, long long rows, long long cols, long long ld, int box_rows,
                         int box_cols, bool swizzle128, bool swizzle64) {
  CUtensorMap m;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * elem_bytes};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode_fn()(&m, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                                 const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : (swizzle64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE),
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) fail(RB200_ERR_RUNTIME, "cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(r)));
  return m;
}

// A 3-D tensor map over 1-byte elements [d2][d1][d0] (d0 contiguous, byte strides ld1, ld2), 128-byte swizzle.
CUtensorMap tc::make_map_3d(const void* ptr, long long d0, long long d1, long long d2, long long ld1, long long ld2, int box0,
                            int box1, int box2) {
  CUtensorMap m;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(d0), static_cast<cuuint64_t>(d1), static_cast<cuuint64_t>(d2)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld1), static_cast<cuuint64_t>(ld2)};
  const cuuint32_t box[3] = {static_cast<cuuint32_t>(box0), static_cast<cuuint32_t>(box1), static_cast<cuuint32_t>(box2)};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) fail(RB200_ERR_RUNTIME, "cuTensorMapEncodeTiled (3-D) failed with code " + std::to_string(static_cast<int>(r)));
  return m;
}

int* tc::status_word() {
  // One word per device, allocated on first use and kept for the life of the process.
  static int* words[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  RB_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(mu);
  if (!words[dev]) {
    RB_CUDA(cudaMalloc(&words[dev], sizeof(int)));
    RB_CUDA(cudaMemset(words[dev], 0, sizeof(int)));
  }
  return words[dev];
}

namespace {

// One launch with the tile shape the planner chose.
template <int BN, bool INT8, int MT>
void launch_umma_cfg(const WeightView& W, const __half* x, int ldx, float* y, int T, float beta, cudaStream_t st, int rows,
                     int splits) {
  using S = UmmaSmem<BN, INT8, MT>;
  static PerDeviceOnce once;
  auto kernel = umma_gemm_kernel<BN, INT8, MT>;
  if (once.first())
    RB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(S::kTotal)));
  const CUtensorMap mw = INT8 ? make_map(W.i8, 1, W.N, W.K, W.ld, rows, S::kKB, S::kKB == 128, S::kKB == 64)
                              : make_map(W.f16, 2, W.N, W.K, W.ld, rows, kBlockK, true);
  const CUtensorMap mx = make_map(x, 2, T, W.K, ldx, BN, kBlockK, true);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(div_up(W.N, rows), div_up(T, BN), splits);
  cfg.blockDim = dim3(INT8 ? kUmmaThreadsInt8 : kUmmaThreads);
  cfg.dynamicSmemBytes = S::kTotal;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = splits;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // may start under the kernel ahead (common.cuh)
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  count_launch();
  int* status = status_word();
  const float* scale = W.scale;
  const int N = W.N, K = W.K;
  RB_CUDA(cudaLaunchKernelEx(&cfg, kernel, mw, mx, scale, y, T, N, K, rows, beta, status));
}

template <int BN, bool INT8>
void launch_umma_t(const WeightView& W, const __half* x, int ldx, float* y, int T, float beta, cudaStream_t st) {
  using S = UmmaSmem<BN, INT8, 1>;
  // Rows per CTA, M tiles per CTA and the K split (a cluster along z): the combination that needs
  // the fewest (waves x weight bytes per CTA), where a CTA's fixed cost (prologue, pipeline fill,
  // epilogue) counts like 48 KB of weights. A cluster needs its CTAs on SMs of one GPC at the same
  // time, so fewer clusters than SMs / size are resident together: the occupancy query says how many.
  const int ttiles = div_up(T, BN), nk = div_up(W.K, S::kKB);
  static const std::array<int, 9> capacity =
      cluster_capacity(umma_gemm_kernel<BN, INT8, 1>, INT8 ? kUmmaThreadsInt8 : kUmmaThreads, S::kTotal);
  const bool can_split = static_cast<size_t>(BN) * kTileM * 4 <= static_cast<size_t>(S::kStages) * S::kStageBytes;
  using S2 = UmmaSmem<BN, INT8, INT8 ? 1 : 2>;
  const bool can_split2 = static_cast<size_t>(BN) * kTileM * 4 <= static_cast<size_t>(S2::kStages) * S2::kStageBytes;
  constexpr bool kTwoTiles = !INT8 && BN >= 128;  // two M tiles per CTA: fp16, wide token tiles
  static const bool two_off = [] {
    const char* e = std::getenv("RB200_GEMM_MT");
    return e && std::atoi(e) == 1;
  }();
  const double elem = INT8 ? 1.0 : 2.0;
  int rows = kTileM, splits = 1, mt = 1;
  double best = 1e30;
  // Two M tiles only with at least 200 of their 256 rows in use: the second MMA tile costs the
  // same however few of its rows count (176-row tiles measured slower than 128-row ones).
  for (int m = 1; m <= ((kTwoTiles && !two_off) ? 2 : 1); ++m) {
    for (int r = kTileM * m; r >= (m == 1 ? 64 : 200); r -= 8) {
      // Two M tiles are planned without a K split only: with one (the kernel can do it, and the
      // forced-split tests run it) the projections with few row tiles measured slower at 256
      // tokens (QKV 31 us, attention output 28 us, down 48 us against 22.5, 17.7 and 36 us with
      // 128-row tiles in clusters of four): their time is pipeline fill and the partial-tile
      // exchange, which two exchanges and shorter k ranges make worse, not the L2 traffic of the
      // shared activation tile.
      for (int sp = 1; sp <= (m == 1 ? 8 : 1); ++sp) {
        if (sp > 1 && (!can_split || nk / sp < 4)) break;
        const long long clusters = static_cast<long long>(div_up(W.N, r)) * ttiles;
        const int cap = m == 1 ? capacity[sp] : sm_count();
        const double cost = static_cast<double>(div_up(clusters, static_cast<long long>(cap))) *
                            (static_cast<double>(r) * elem * W.K / sp + 48.0 * 1024 + (sp > 1 ? 8.0 * 1024 : 0.0));
        if (cost < best - 1e-9) {
          best = cost;
          rows = r;
          splits = sp;
          mt = m;
        }
      }
    }
  }
  static const int forced = [] {
    const char* e = std::getenv("RB200_GEMM_SPLITS");
    return e ? std::atoi(e) : 0;
  }();
  if (forced > 0 && can_split) {
    splits = std::min({forced, 8, std::max(1, nk)});
    if (mt == 2 && !can_split2) {
      rows = kTileM;
      mt = 1;
    }
  }
  static const bool debug = std::getenv("RB200_GEMM_DEBUG") != nullptr;
  if (debug)
    std::fprintf(stderr, "umma_gemm N=%d K=%d T=%d int8=%d: token tile %d, %d rows per CTA (%d M tiles), K split %d, grid %d x %d x %d; "
                 "resident clusters by size: %d %d %d %d %d %d %d %d\n",
                 W.N, W.K, T, INT8 ? 1 : 0, BN, rows, mt, splits, div_up(W.N, rows), ttiles, splits, capacity[1], capacity[2],
                 capacity[3], capacity[4], capacity[5], capacity[6], capacity[7], capacity[8]);
  if constexpr (kTwoTiles) {
    if (mt == 2) return launch_umma_cfg<BN, INT8, 2>(W, x, ldx, y, T, beta, st, rows, splits);
  }
  launch_umma_cfg<BN, INT8, 1>(W, x, ldx, y, T, beta, st, rows, splits);
}

template <bool INT8>
void launch_umma_i(const WeightView& W, const __half* x, int ldx, float* y, int T, float beta, cudaStream_t st) {
  if (T <= 16) launch_umma_t<16, INT8>(W, x, ldx, y, T, beta, st);
  else if (T <= 32) launch_umma_t<32, INT8>(W, x, ldx, y, T, beta, st);
  else if (T <= 64) launch_umma_t<64, INT8>(W, x, ldx, y, T, beta, st);
  else if (T <= 128 || (T > 256 && T <= 384 && false)) launch_umma_t<128, INT8>(W, x, ldx, y, T, beta, st);
  else launch_umma_t<256, INT8>(W, x, ldx, y, T, beta, st);
}

}  // namespace

bool umma_gemm_usable(const WeightView& W, const __half* x, int ldx) {
  // TMA wants 16-byte aligned bases and row strides
  const uintptr_t wp = reinterpret_cast<uintptr_t>(W.i8 ? static_cast<const void*>(W.i8) : static_cast<const void*>(W.f16));
  return (wp & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (static_cast<long long>(W.ld) * (W.i8 ? 1 : 2)) % 16 == 0 &&
         (static_cast<long long>(ldx) * 2) % 16 == 0 && W.K % kBlockK == 0;
}

void launch_umma_gemm(const WeightView& W, const __half* x, int ldx, float* y, int T, float beta, cudaStream_t st) {
  if (T == 0) return;
  if (W.i8) launch_umma_i<true>(W, x, ldx, y, T, beta, st);
  else launch_umma_i<false>(W, x, ldx, y, T, beta, st);
}

int umma_gemm_status() {
  int v = 0;
  RB_CUDA(cudaMemcpy(&v, status_word(), sizeof(int), cudaMemcpyDeviceToHost));
  return v;
}

const int* umma_status_word() { return status_word(); }

void umma_status_clear(cudaStream_t st) { RB_CUDA(cudaMemsetAsync(status_word(), 0, sizeof(int), st)); }

}  // namespace rb200
