// Attention over the paged KV cache, three kernels:
//
//  * decode_split_kernel + decode_merge_kernel — split-context flash decoding for chunks of
//    one token (replaces decode_attention_kernel / decode_combine_kernel of the reference,
//    engine/src/cuda_kernels.cuh:223-362). One CTA per (decode token, KV head, 512-key
//    slice). Each of its 4 warps is an independent worker on 16-key tiles: it streams the
//    tile's K and V rows from the page pool into its own swizzled shared-memory ring with
//    16-byte async copies (3 tiles in flight per warp, 2 CTAs per SM), scores all G query
//    heads of the KV head against the tile with one tensor-core pass (heads on the M axis of
//    m16n8k16, keys on N), keeps a running (max, sum, O) per head in registers, and the
//    warps' results are merged through shared memory into the slice's partial (m, l, O).
//    The work per byte is so low that the kernel is bound by HBM bandwidth: per context
//    token it reads 2 * kv_heads * D * 2 bytes exactly once.
//  * prefill_flash_kernel — causal flash attention for chunks of several tokens (replaces
//    flash_prefill_kernel, engine/src/cuda_kernels.cuh:51-178): 64 query rows of one head per
//    CTA, 64-key K/V tiles double-buffered in shared memory, S, P and O in registers.
//  * reference_attention_kernel — one CTA per (token, head), any head size (the role of the
//    reference's M0 attention_kernel, engine/src/cuda_backend.cu:202-243).
//
// Page addressing everywhere is KVLayout::offset (engine/include/relay/kv_cache.h:32-35):
// key j of a sequence lives at ((table[j / bs] * kv_heads + kvh) * bs + j % bs) * D.
#include <cstdlib>
#include <mutex>

#include "kernels.h"
#include "tcgen05.cuh"

namespace rb200 {

namespace {

constexpr int kDecWarps = 4;    // independent tile workers per decode CTA
constexpr int kDecStages = 3;   // 16-key tiles in flight per warp
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Halves from the start of one layer's pool to row `key` of KV head `kvh`.
// `table` is indexed by absolute block number of the sequence minus `first_block`.
__device__ __forceinline__ long long key_offset(const int* table, int first_block, int key, int bs, int bs_shift,
                                                int kv_heads, int kvh, int D) {
  int blk_i, slot;
  if (bs_shift >= 0) {
    blk_i = key >> bs_shift;
    slot = key & (bs - 1);
  } else {
    blk_i = key / bs;
    slot = key - blk_i * bs;
  }
  const long long blk = table[blk_i - first_block];
  return ((blk * kv_heads + kvh) * bs + slot) * static_cast<long long>(D);
}

// ---------------------------------------------------------------------------------------
// Split-context decode
// ---------------------------------------------------------------------------------------

// Shared by decode and prefill: scores of 16 query rows against 16 keys.
// s[0] covers keys 0-7 of the tile, s[1] keys 8-15; ktile is [16][D] halves, swizzled.
template <int D>
__device__ __forceinline__ void qk_16x16(float (&s)[2][4], const uint32_t (&qf)[D / 16][4], uint32_t ktile, int lane) {
  constexpr int CH = D / 8;
  const int row = (lane & 7) + ((lane >> 4) << 3);
  const int csel = (lane >> 3) & 1;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    uint32_t kb[4];
    ldmatrix_x4(kb, ktile + swz<CH>(row, 2 * kk + csel) * 16);
    mma_f16(s[0], qf[kk], kb[0], kb[1]);
    mma_f16(s[1], qf[kk], kb[2], kb[3]);
  }
}

// O(16 x D) += P(16 x 16 keys) V(16 keys x D); vtile is [16][D] halves, swizzled.
template <int D>
__device__ __forceinline__ void pv_16x16(float (&o)[D / 8][4], const uint32_t (&pa)[4], uint32_t vtile, int lane) {
  constexpr int CH = D / 8;
  const int row = (lane & 7) + (((lane >> 3) & 1) << 3);
  const int csel = lane >> 4;
#pragma unroll
  for (int j = 0; j < D / 16; ++j) {
    uint32_t vb[4];
    ldmatrix_x4_trans(vb, vtile + swz<CH>(row, 2 * j + csel) * 16);
    mma_f16(o[2 * j], pa, vb[0], vb[1]);
    mma_f16(o[2 * j + 1], pa, vb[2], vb[3]);
  }
}

template <int D>
constexpr size_t decode_smem_bytes() {
  return static_cast<size_t>(kDecWarps) * kDecStages * 2 * 16 * D * sizeof(__half);
}

// CONTIG: block_size is a multiple of 16, so a 16-key tile is one contiguous run of a page.
// WIDE: more than 8 query heads per KV head (rows 8..15 of the M tile are real heads).
template <int D, bool CONTIG, bool WIDE>
__global__ void __launch_bounds__(kDecWarps * 32, 2)
decode_split_kernel(const float* __restrict__ q, TokenMeta m, const int* __restrict__ decode_tokens,
                    const __half* __restrict__ kc, const __half* __restrict__ vc, float* __restrict__ part_o,
                    float* __restrict__ part_ml, __half* __restrict__ out, int heads, int kv_heads, int bs,
                    int bs_shift, int q_stride, int o_stride, float scale_log2e, int max_parts, int slice,
                    int cluster_merge) {
  constexpr int CH = D / 8;               // 16-byte chunks per K/V row
  constexpr int TILE_HALVES = 16 * D;     // one 16-key tile of K (or V)
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ int s_table[kDecodeSlice];   // block ids covering the slice: slice / block_size <= 512 entries
  __shared__ float s_m[kDecWarps][16], s_l[kDecWarps][16];
  __shared__ float cm_m[16], cm_l[16];    // cluster merge: this slice's (max, sum) per head

  pdl_trigger();
  // The token's context length and the block ids of the slice are batch metadata, complete before
  // the pass started: they are fetched (a chain of four dependent loads) while the kernel ahead,
  // which writes q and this step's K/V, still runs.
  const int di = blockIdx.x, kvh = blockIdx.y, part = blockIdx.z;
  const int tok = decode_tokens[di];
  const int ctx = m.pos[tok] + 1;
  const int k0 = part * slice;
  // A slice past the context has nothing to do. Launched as a cluster over the slices (the merge
  // then happens here, over distributed shared memory) its CTA still has to meet the others at the
  // cluster barriers, so it runs through with no keys: max -inf, sum 0.
  const bool empty = k0 >= ctx;
  if (empty && !cluster_merge) return;
  const int k1 = empty ? k0 : min(ctx, k0 + slice);
  const int ntiles = (k1 - k0 + 15) >> 4;
  const int G = heads / kv_heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;

  // Block ids of the slice, fetched as 16-byte vectors where the table allows it.
  const int* table = m.tables + m.table_off[m.seq[tok]];
  const int first_block = bs_shift >= 0 ? (k0 >> bs_shift) : k0 / bs;
  const int last_block = bs_shift >= 0 ? ((k1 - 1) >> bs_shift) : (k1 - 1) / bs;
  const int nblk = empty ? 0 : last_block - first_block + 1;
  {
    const int* src = table + first_block;
    if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
      for (int i = threadIdx.x * 4; i < nblk; i += blockDim.x * 4) {
        if (i + 4 <= nblk) {
          *reinterpret_cast<int4*>(&s_table[i]) = *reinterpret_cast<const int4*>(src + i);
        } else {
          for (int e = i; e < nblk; ++e) s_table[e] = src[e];
        }
      }
    } else {
      for (int i = threadIdx.x; i < nblk; i += blockDim.x) s_table[i] = src[i];
    }
  }
  pdl_wait();

  // The G query heads of this KV head as A fragments (rows = heads, columns = d), fp16.
  uint32_t qf[D / 16][4];
  {
    const float* q0 = q + static_cast<long long>(tok) * q_stride + (kvh * G) * D;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      const int d0 = kk * 16 + 2 * t4;
      float2 a = make_float2(0.f, 0.f), b = a, c = a, e = a;
      if (g < G) {
        a = *reinterpret_cast<const float2*>(q0 + g * D + d0);
        c = *reinterpret_cast<const float2*>(q0 + g * D + d0 + 8);
      }
      if (WIDE && g + 8 < G) {
        b = *reinterpret_cast<const float2*>(q0 + (g + 8) * D + d0);
        e = *reinterpret_cast<const float2*>(q0 + (g + 8) * D + d0 + 8);
      }
      qf[kk][0] = pack_half2(a.x, a.y);
      qf[kk][1] = pack_half2(b.x, b.y);
      qf[kk][2] = pack_half2(c.x, c.y);
      qf[kk][3] = pack_half2(e.x, e.y);
    }
  }
  __syncthreads();  // s_table is ready

  __half* ring = reinterpret_cast<__half*>(smem_raw) + static_cast<size_t>(warp) * kDecStages * 2 * TILE_HALVES;
  const uint32_t ring_u32 = smem_u32(ring);

  // Async copy of tile `tile` (keys k0 + 16*tile ...) into stage `stage` of this warp's ring.
  auto load_tile = [&](int tile, int stage) {
    const uint32_t kdst = ring_u32 + static_cast<uint32_t>(stage) * 2 * TILE_HALVES * 2;
    const uint32_t vdst = kdst + TILE_HALVES * 2;
    const int key0 = k0 + tile * 16;
    const int nvalid = min(16, k1 - key0);
    if constexpr (CONTIG) {
      const long long base = key_offset(s_table, first_block, key0, bs, bs_shift, kv_heads, kvh, D);
      const __half* ksrc = kc + base;
      const __half* vsrc = vc + base;
#pragma unroll
      for (int idx = lane; idx < 16 * CH; idx += 32) {
        const int row = idx / CH, c = idx % CH;
        const int bytes = row < nvalid ? 16 : 0;
        const uint32_t off = static_cast<uint32_t>(swz<CH>(row, c)) * 16;
        cp_async16_zfill(kdst + off, ksrc + idx * 8, bytes);
        cp_async16_zfill(vdst + off, vsrc + idx * 8, bytes);
      }
    } else {
#pragma unroll
      for (int idx = lane; idx < 16 * CH; idx += 32) {
        const int row = idx / CH, c = idx % CH;
        const bool ok = row < nvalid;
        const long long base = ok ? key_offset(s_table, first_block, key0 + row, bs, bs_shift, kv_heads, kvh, D) : 0;
        const int bytes = ok ? 16 : 0;
        const uint32_t off = static_cast<uint32_t>(swz<CH>(row, c)) * 16;
        cp_async16_zfill(kdst + off, kc + base + c * 8, bytes);
        cp_async16_zfill(vdst + off, vc + base + c * 8, bytes);
      }
    }
  };

  // Tiles warp, warp + 4, ... of the slice belong to this warp.
  const int my_tiles = ntiles > warp ? (ntiles - warp + kDecWarps - 1) / kDecWarps : 0;
#pragma unroll
  for (int s = 0; s < kDecStages - 1; ++s) {
    if (s < my_tiles) load_tile(warp + s * kDecWarps, s);
    cp_async_commit();
  }

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;  // rows g and g + 8, log2 domain

  for (int j = 0; j < my_tiles; ++j) {
    cp_async_wait<kDecStages - 2>();
    __syncwarp();
    if (j + kDecStages - 1 < my_tiles) load_tile(warp + (j + kDecStages - 1) * kDecWarps, (j + kDecStages - 1) % kDecStages);
    cp_async_commit();

    const int stage = j % kDecStages;
    const uint32_t ktile = ring_u32 + static_cast<uint32_t>(stage) * 2 * TILE_HALVES * 2;
    const uint32_t vtile = ktile + TILE_HALVES * 2;
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    qk_16x16<D>(s, qf, ktile, lane);

    // scale into the log2 domain and mask the keys past the context
    const int key0 = k0 + (warp + j * kDecWarps) * 16 + 2 * t4;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int ka = key0 + nt * 8;
      s[nt][0] = ka < k1 ? s[nt][0] * scale_log2e : -INFINITY;
      s[nt][1] = ka + 1 < k1 ? s[nt][1] * scale_log2e : -INFINITY;
      s[nt][2] = ka < k1 ? s[nt][2] * scale_log2e : -INFINITY;
      s[nt][3] = ka + 1 < k1 ? s[nt][3] * scale_log2e : -INFINITY;
    }
    float mx0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    const float mn0 = fmaxf(m0, mx0);
    const float c0 = fast_exp2(m0 - mn0);
    m0 = mn0;
    const float p00 = fast_exp2(s[0][0] - mn0), p01 = fast_exp2(s[0][1] - mn0);
    const float p10 = fast_exp2(s[1][0] - mn0), p11 = fast_exp2(s[1][1] - mn0);
    l0 = l0 * c0 + ((p00 + p01) + (p10 + p11));
    uint32_t pa[4];
    pa[0] = pack_half2(p00, p01);
    pa[2] = pack_half2(p10, p11);
    float c1 = 1.f;
    if constexpr (WIDE) {
      float mx1 = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn1 = fmaxf(m1, mx1);
      c1 = fast_exp2(m1 - mn1);
      m1 = mn1;
      const float r00 = fast_exp2(s[0][2] - mn1), r01 = fast_exp2(s[0][3] - mn1);
      const float r10 = fast_exp2(s[1][2] - mn1), r11 = fast_exp2(s[1][3] - mn1);
      l1 = l1 * c1 + ((r00 + r01) + (r10 + r11));
      pa[1] = pack_half2(r00, r01);
      pa[3] = pack_half2(r10, r11);
    } else {
      pa[1] = 0u;
      pa[3] = 0u;
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= c0;
      o[i][1] *= c0;
      if constexpr (WIDE) {
        o[i][2] *= c1;
        o[i][3] *= c1;
      }
    }
    pv_16x16<D>(o, pa, vtile, lane);
  }
  cp_async_wait<0>();
  __syncwarp();

  // Merge the warps' (m, l, O) through shared memory (each warp reuses its own ring).
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  if constexpr (WIDE) {
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  }
  float* os = reinterpret_cast<float*>(ring);  // [16][D] floats = 64*D bytes <= ring size 192*D
  if (t4 == 0) {
    s_m[warp][g] = m0;
    s_l[warp][g] = l0;
    s_m[warp][g + 8] = WIDE ? m1 : -INFINITY;
    s_l[warp][g + 8] = WIDE ? l1 : 0.f;
  }
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    *reinterpret_cast<float2*>(os + g * D + i * 8 + 2 * t4) = make_float2(o[i][0], o[i][1]);
    if constexpr (WIDE) *reinterpret_cast<float2*>(os + (g + 8) * D + i * 8 + 2 * t4) = make_float2(o[i][2], o[i][3]);
  }
  __syncthreads();

  const float* os_all = reinterpret_cast<const float*>(smem_raw);
  constexpr int WARP_FLOATS = kDecStages * 2 * TILE_HALVES / 2;  // ring size of one warp in floats
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int r = idx / D, d = idx - r * D;
    float M = s_m[0][r];
#pragma unroll
    for (int w = 1; w < kDecWarps; ++w) M = fmaxf(M, s_m[w][r]);
    float acc = 0.f, L = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float mw = s_m[w][r];
      if (mw != -INFINITY) {
        const float e = fast_exp2(mw - M);
        acc += e * os_all[w * WARP_FLOATS + r * D + d];
        L += e * s_l[w][r];
      }
    }
    const int head = kvh * G + r;
    if (max_parts == 1) {
      out[static_cast<long long>(tok) * o_stride + head * D + d] = __float2half_rn(acc / L);
    } else if (cluster_merge) {
      // parked behind warp 0's own partial, in a part of its ring nothing reads any more
      reinterpret_cast<float*>(smem_raw)[16 * D + idx] = acc;
      if (d == 0) {
        cm_m[r] = M;
        cm_l[r] = L;
      }
    } else {
      const long long slot = (static_cast<long long>(di) * heads + head) * max_parts + part;
      part_o[slot * D + d] = acc;
      if (d == 0) {
        part_ml[slot * 2] = M * kLn2;  // natural-log units, as the merge formula is stated
        part_ml[slot * 2 + 1] = L;
      }
    }
  }
  if (cluster_merge) {
    // out = sum_p 2^(m_p - M) O_p / sum_p 2^(m_p - M) l_p over the cluster's slices
    // (engine/src/cuda_kernels.cuh:341-362, in the log2 domain the slices already use): the CTA of
    // slice p finishes the heads r with r % slices == p, reading every member's (m, l, O) over
    // distributed shared memory in rank order, so the result is the same on every run and neither
    // partial results nor a second kernel touch global memory.
    tc::cluster_sync_all();
    const uint32_t o_addr = smem_u32(reinterpret_cast<float*>(smem_raw) + 16 * D);
    for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
      const int r = idx / D, d = idx - r * D;
      if (r % max_parts != part) continue;
      float M = -INFINITY;
      for (int p = 0; p < max_parts; ++p) M = fmaxf(M, tc::ld_dsmem_f32(smem_u32(&cm_m[r]), p));
      float acc = 0.f, L = 0.f;
      for (int p = 0; p < max_parts; ++p) {
        const float mp = tc::ld_dsmem_f32(smem_u32(&cm_m[r]), p);
        if (mp != -INFINITY) {
          const float e = fast_exp2(mp - M);
          acc += e * tc::ld_dsmem_f32(o_addr + static_cast<uint32_t>(idx) * 4, p);
          L += e * tc::ld_dsmem_f32(smem_u32(&cm_l[r]), p);
        }
      }
      out[static_cast<long long>(tok) * o_stride + (kvh * G + r) * D + d] = __float2half_rn(acc / L);
    }
    tc::cluster_sync_all();  // nobody leaves while a peer may still read its shared memory
  }
}

// out = sum_p e^(m_p - M) O_p / sum_p e^(m_p - M) l_p over the slices the token's context
// reaches (engine/src/cuda_kernels.cuh:341-362). One warp per (decode token, head): lanes
// first work across the slices (max and sum by warp reduction), then across the head
// dimension, four values per lane, with each slice's weight broadcast by shuffle.
__global__ void decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    const int* __restrict__ decode_tokens, const int* __restrict__ pos,
                                    __half* __restrict__ out, int heads, int D, int o_stride, int max_parts,
                                    int n_pairs, int slice) {
  pdl_trigger();
  const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int pair_c = min(pair, n_pairs - 1);
  const int di = pair_c / heads, h = pair_c - di * heads;
  const int tok = decode_tokens[di];                 // batch metadata: read while the split kernel still runs
  const int parts = (pos[tok] + slice) / slice;      // ceil((pos + 1) / slice)
  pdl_wait();
  if (pair >= n_pairs) return;
  const long long base = static_cast<long long>(pair) * max_parts;
  float M = -INFINITY;
  for (int p0 = 0; p0 < parts; p0 += 32)
    M = fmaxf(M, p0 + lane < parts ? part_ml[(base + p0 + lane) * 2] : -INFINITY);
  M = warp_max(M);
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  float L = 0.f;
  for (int p0 = 0; p0 < parts; p0 += 32) {
    float w = 0.f, wl = 0.f;
    if (p0 + lane < parts) {
      const float2 ml = *reinterpret_cast<const float2*>(part_ml + (base + p0 + lane) * 2);
      w = __expf(ml.x - M);
      wl = w * ml.y;
    }
    L += wl;
    const int np = min(32, parts - p0);
    for (int d0 = lane * 4; d0 < D; d0 += 128) {  // D <= 128: a single trip
      for (int p = 0; p < np; ++p) {
        const float wp = __shfl_sync(0xffffffffu, w, p);
        const float4 o = *reinterpret_cast<const float4*>(part_o + (base + p0 + p) * D + d0);
        acc[0] += wp * o.x;
        acc[1] += wp * o.y;
        acc[2] += wp * o.z;
        acc[3] += wp * o.w;
      }
    }
    if (lane * 4 >= D)  // lanes past the head dimension still take part in the shuffles
      for (int p = 0; p < np; ++p) (void)__shfl_sync(0xffffffffu, w, p);
  }
  L = warp_sum(L);
  const float inv = 1.0f / L;
  if (lane * 4 < D) {
    __half2* o = reinterpret_cast<__half2*>(out + static_cast<long long>(tok) * o_stride + h * D + lane * 4);
    o[0] = __floats2half2_rn(acc[0] * inv, acc[1] * inv);
    o[1] = __floats2half2_rn(acc[2] * inv, acc[3] * inv);
  }
}

// ---------------------------------------------------------------------------------------
// Flash prefill
// ---------------------------------------------------------------------------------------

constexpr int kPreKeys = 64;  // keys per shared-memory stage

template <int D>
constexpr size_t prefill_smem_bytes() {
  return static_cast<size_t>(2) * 2 * kPreKeys * D * sizeof(__half);
}

template <int D>
__global__ void __launch_bounds__(128)
prefill_flash_kernel(const float* __restrict__ q, TokenMeta m, const int2* __restrict__ tiles,
                     const __half* __restrict__ kc, const __half* __restrict__ vc, __half* __restrict__ out, int heads,
                     int kv_heads, int bs, int bs_shift, int q_stride, int o_stride, float scale_log2e) {
  constexpr int CH = D / 8;
  constexpr int STAGE_HALVES = 2 * kPreKeys * D;  // K tile then V tile
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const uint32_t smem0 = smem_u32(smem_raw);

  const int2 tile = tiles[blockIdx.x];
  const int t0 = tile.x, nrows = tile.y;
  const int head = blockIdx.y, kvh = head / (heads / kv_heads);
  const int pos0 = m.pos[t0];
  const int nk = pos0 + nrows;  // keys the last row sees
  const int* table = m.tables + m.table_off[m.seq[t0]];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;

  // This warp's 16 query rows (rows past the tile's end repeat the last one; never written).
  const int r0 = min(warp * 16 + g, nrows - 1), r1 = min(warp * 16 + g + 8, nrows - 1);
  const int pr0 = pos0 + r0, pr1 = pos0 + r1;
  const int warp_last_pos = pos0 + min(warp * 16 + 15, nrows - 1);
  const bool warp_active = warp * 16 < nrows;
  uint32_t qf[D / 16][4];
  {
    const float* qa = q + static_cast<long long>(t0 + r0) * q_stride + head * D;
    const float* qb = q + static_cast<long long>(t0 + r1) * q_stride + head * D;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      const int d0 = kk * 16 + 2 * t4;
      const float2 a = *reinterpret_cast<const float2*>(qa + d0), b = *reinterpret_cast<const float2*>(qb + d0);
      const float2 c = *reinterpret_cast<const float2*>(qa + d0 + 8), e = *reinterpret_cast<const float2*>(qb + d0 + 8);
      qf[kk][0] = pack_half2(a.x, a.y);
      qf[kk][1] = pack_half2(b.x, b.y);
      qf[kk][2] = pack_half2(c.x, c.y);
      qf[kk][3] = pack_half2(e.x, e.y);
    }
  }

  auto load_stage = [&](int kt, int stage) {
    const uint32_t kdst = smem0 + static_cast<uint32_t>(stage) * STAGE_HALVES * 2;
    const uint32_t vdst = kdst + kPreKeys * D * 2;
    const int key0 = kt * kPreKeys;
    for (int idx = threadIdx.x; idx < kPreKeys * CH; idx += blockDim.x) {
      const int row = idx / CH, c = idx % CH;
      const bool ok = key0 + row < nk;
      const long long base = ok ? key_offset(table, 0, key0 + row, bs, bs_shift, kv_heads, kvh, D) : 0;
      const int bytes = ok ? 16 : 0;
      const uint32_t off = static_cast<uint32_t>(swz<CH>(row, c)) * 16;
      cp_async16_zfill(kdst + off, kc + base + c * 8, bytes);
      cp_async16_zfill(vdst + off, vc + base + c * 8, bytes);
    }
  };

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  const int nkt = (nk + kPreKeys - 1) / kPreKeys;
  load_stage(0, 0);
  cp_async_commit();
  for (int kt = 0; kt < nkt; ++kt) {
    if (kt + 1 < nkt) load_stage(kt + 1, (kt + 1) & 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const int key0 = kt * kPreKeys;
    if (warp_active && key0 <= warp_last_pos) {
      const uint32_t ktile = smem0 + static_cast<uint32_t>(kt & 1) * STAGE_HALVES * 2;
      const uint32_t vtile = ktile + kPreKeys * D * 2;
      float s[kPreKeys / 8][4];
#pragma unroll
      for (int i = 0; i < kPreKeys / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
      for (int kp = 0; kp < kPreKeys / 16; ++kp) {
        float s2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        qk_16x16<D>(s2, qf, ktile + kp * 16 * D * 2, lane);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[2 * kp][e] = s2[0][e];
          s[2 * kp + 1][e] = s2[1][e];
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < kPreKeys / 8; ++nt) {
        const int ka = key0 + nt * 8 + 2 * t4;
        s[nt][0] = ka <= pr0 ? s[nt][0] * scale_log2e : -INFINITY;
        s[nt][1] = ka + 1 <= pr0 ? s[nt][1] * scale_log2e : -INFINITY;
        s[nt][2] = ka <= pr1 ? s[nt][2] * scale_log2e : -INFINITY;
        s[nt][3] = ka + 1 <= pr1 ? s[nt][3] * scale_log2e : -INFINITY;
        mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
        mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      const float c0 = fast_exp2(m0 - mn0), c1 = fast_exp2(m1 - mn1);
      m0 = mn0;
      m1 = mn1;
      float sum0 = 0.f, sum1 = 0.f;
      uint32_t pa[kPreKeys / 16][4];
#pragma unroll
      for (int kp = 0; kp < kPreKeys / 16; ++kp) {
        const float a0 = fast_exp2(s[2 * kp][0] - mn0), a1 = fast_exp2(s[2 * kp][1] - mn0);
        const float b0 = fast_exp2(s[2 * kp][2] - mn1), b1 = fast_exp2(s[2 * kp][3] - mn1);
        const float a2 = fast_exp2(s[2 * kp + 1][0] - mn0), a3 = fast_exp2(s[2 * kp + 1][1] - mn0);
        const float b2 = fast_exp2(s[2 * kp + 1][2] - mn1), b3 = fast_exp2(s[2 * kp + 1][3] - mn1);
        sum0 += (a0 + a1) + (a2 + a3);
        sum1 += (b0 + b1) + (b2 + b3);
        pa[kp][0] = pack_half2(a0, a1);
        pa[kp][1] = pack_half2(b0, b1);
        pa[kp][2] = pack_half2(a2, a3);
        pa[kp][3] = pack_half2(b2, b3);
      }
      l0 = l0 * c0 + sum0;
      l1 = l1 * c1 + sum1;
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        o[i][0] *= c0;
        o[i][1] *= c0;
        o[i][2] *= c1;
        o[i][3] *= c1;
      }
#pragma unroll
      for (int kp = 0; kp < kPreKeys / 16; ++kp) pv_16x16<D>(o, pa[kp], vtile + kp * 16 * D * 2, lane);
    }
    __syncthreads();
  }

  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = 1.0f / l0, i1 = 1.0f / l1;
  const bool w0 = warp * 16 + g < nrows, w1 = warp * 16 + g + 8 < nrows;
  __half* oa = out + static_cast<long long>(t0 + r0) * o_stride + head * D + 2 * t4;
  __half* ob = out + static_cast<long long>(t0 + r1) * o_stride + head * D + 2 * t4;
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    if (w0) *reinterpret_cast<__half2*>(oa + i * 8) = __floats2half2_rn(o[i][0] * i0, o[i][1] * i0);
    if (w1) *reinterpret_cast<__half2*>(ob + i * 8) = __floats2half2_rn(o[i][2] * i1, o[i][3] * i1);
  }
}

// ---------------------------------------------------------------------------------------
// Simple attention: one CTA per (token, head), 128 keys per step, any D <= 256
// ---------------------------------------------------------------------------------------

__global__ void __launch_bounds__(128)
reference_attention_kernel(const float* __restrict__ q, TokenMeta m, const __half* __restrict__ kc,
                           const __half* __restrict__ vc, __half* __restrict__ out, int heads, int kv_heads, int D,
                           int bs, int q_stride, int o_stride, float scale) {
  __shared__ float sq[256];
  __shared__ float sp[128];
  __shared__ long long soff[128];
  __shared__ float red[4];
  const int t = blockIdx.x, h = blockIdx.y, kvh = h / (heads / kv_heads);
  const float* qsrc = q + static_cast<long long>(t) * q_stride + h * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) sq[d] = qsrc[d];
  __syncthreads();
  const int ctx = m.pos[t] + 1;
  const int* table = m.tables + m.table_off[m.seq[t]];
  float run_m = -INFINITY, run_l = 0.f, acc0 = 0.f, acc1 = 0.f;  // thread owns dims tid and tid + 128
  for (int j0 = 0; j0 < ctx; j0 += 128) {
    const int j = j0 + threadIdx.x;
    float s = -INFINITY;
    if (j < ctx) {
      const long long off = key_offset(table, 0, j, bs, -1, kv_heads, kvh, D);
      soff[threadIdx.x] = off;
      float a = 0.f;
      for (int d = 0; d < D; ++d) a += sq[d] * __half2float(kc[off + d]);
      s = a * scale;
    }
    float mx = warp_max(s);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    const float new_m = fmaxf(run_m, mx);
    const float corr = __expf(run_m - new_m);
    const float p = j < ctx ? __expf(s - new_m) : 0.f;
    sp[threadIdx.x] = p;
    float ps = warp_sum(p);
    __syncthreads();  // red consumed, sp and soff written
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ps;
    __syncthreads();
    run_l = run_l * corr + ((red[0] + red[1]) + (red[2] + red[3]));
    run_m = new_m;
    acc0 *= corr;
    acc1 *= corr;
    const int nj = min(128, ctx - j0);
    for (int jj = 0; jj < nj; ++jj) {
      const float pj = sp[jj];
      const long long off = soff[jj];
      if (threadIdx.x < D) acc0 += pj * __half2float(vc[off + threadIdx.x]);
      if (threadIdx.x + 128 < D) acc1 += pj * __half2float(vc[off + threadIdx.x + 128]);
    }
    __syncthreads();
  }
  __half* o = out + static_cast<long long>(t) * o_stride + h * D;
  if (threadIdx.x < D) o[threadIdx.x] = __float2half_rn(acc0 / run_l);
  if (threadIdx.x + 128 < D) o[threadIdx.x + 128] = __float2half_rn(acc1 / run_l);
}

int shift_of(int bs) {
  if (bs <= 0 || (bs & (bs - 1)) != 0) return -1;
  int s = 0;
  while ((1 << s) < bs) ++s;
  return s;
}

template <class K>
void raise_smem(K kernel, size_t bytes) {
  // The attribute belongs to the (kernel, device) pair; it is only ever raised.
  RB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)));
}

template <int D, bool CONTIG, bool WIDE>
void launch_decode_t(const AttnShape& s, const float* q, const TokenMeta& m, const int* decode_tokens, int n_decode,
                     int parts, int slice, const __half* kc, const __half* vc, float* part_o, float* part_ml, __half* out,
                     cudaStream_t st, bool cluster_merge) {
  static PerDeviceOnce once;
  auto kernel = decode_split_kernel<D, CONTIG, WIDE>;
  if (once.first()) raise_smem(kernel, decode_smem_bytes<D>());
  RB_REQUIRE(!cluster_merge || parts <= 8, "decode attention: a cluster holds at most 8 slices");
  const float scale_log2e = kLog2e / sqrtf(static_cast<float>(D));
  dim3 grid(n_decode, s.kv_heads, parts);
  count_launch();
  if (!cluster_merge) {
    launch_pdl(kernel, grid, dim3(kDecWarps * 32), decode_smem_bytes<D>(), st, q, m, decode_tokens, kc, vc, part_o, part_ml, out,
               s.heads, s.kv_heads, s.block_size, shift_of(s.block_size), s.q_stride, s.o_stride, scale_log2e, parts, slice, 0);
    return;
  }
  // the slices of one (token, KV head) as one thread-block cluster
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kDecWarps * 32);
  cfg.dynamicSmemBytes = decode_smem_bytes<D>();
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = parts;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  const int heads = s.heads, kv_heads = s.kv_heads, bs = s.block_size, bs_shift = shift_of(s.block_size), q_stride = s.q_stride,
            o_stride = s.o_stride, one = 1;
  RB_CUDA(cudaLaunchKernelEx(&cfg, kernel, q, m, decode_tokens, kc, vc, part_o, part_ml, out, heads, kv_heads, bs, bs_shift, q_stride,
                             o_stride, scale_log2e, parts, slice, one));
}

template <int D>
void launch_decode_d(const AttnShape& s, const float* q, const TokenMeta& m, const int* decode_tokens, int n_decode,
                     int parts, int slice, const __half* kc, const __half* vc, float* part_o, float* part_ml, __half* out,
                     cudaStream_t st, bool cm) {
  const bool contig = s.block_size % 16 == 0, wide = s.heads / s.kv_heads > 8;
  if (contig && !wide) launch_decode_t<D, true, false>(s, q, m, decode_tokens, n_decode, parts, slice, kc, vc, part_o, part_ml, out, st, cm);
  else if (contig) launch_decode_t<D, true, true>(s, q, m, decode_tokens, n_decode, parts, slice, kc, vc, part_o, part_ml, out, st, cm);
  else if (!wide) launch_decode_t<D, false, false>(s, q, m, decode_tokens, n_decode, parts, slice, kc, vc, part_o, part_ml, out, st, cm);
  else launch_decode_t<D, false, true>(s, q, m, decode_tokens, n_decode, parts, slice, kc, vc, part_o, part_ml, out, st, cm);
}

template <int D>
void launch_prefill_d(const AttnShape& s, const float* q, const TokenMeta& m, const int2* tiles, int n_tiles,
                      const __half* kc, const __half* vc, __half* out, cudaStream_t st) {
  static PerDeviceOnce once;
  auto kernel = prefill_flash_kernel<D>;
  if (once.first()) raise_smem(kernel, prefill_smem_bytes<D>());
  const float scale_log2e = kLog2e / sqrtf(static_cast<float>(D));
  dim3 grid(n_tiles, s.heads);
  count_launch();
  kernel<<<grid, 128, prefill_smem_bytes<D>(), st>>>(q, m, tiles, kc, vc, out, s.heads, s.kv_heads, s.block_size,
                                                     shift_of(s.block_size), s.q_stride, s.o_stride, scale_log2e);
}

}  // namespace

bool fast_attention_supported(const AttnShape& s) {
  const int D = s.D;
  if (!(D == 16 || D == 32 || D == 64 || D == 128)) return false;
  if (s.kv_heads <= 0 || s.heads % s.kv_heads != 0) return false;
  const int G = s.heads / s.kv_heads;
  return G >= 1 && G <= 16 && s.q_stride % 2 == 0 && s.o_stride % 2 == 0 && s.kv_heads <= 65535;
}

size_t decode_scratch_bytes(const AttnShape& s, int n_decode, int max_ctx) {
  const size_t parts = static_cast<size_t>(div_up(std::max(max_ctx, 1), kDecodeSlice));
  return static_cast<size_t>(n_decode) * s.heads * parts * (s.D + 2) * sizeof(float);
}

// A batch with enough (token, KV head) pairs to put a CTA on most SMs (more than half the
// resident slots: 17 sequences of the benchmark model) gets ONE slice per pair, as long as a
// slice's block ids fit the kernel's table (512 entries: 8192 keys at block size 16): no partial
// results, no merge. Splitting such contexts further to even out the waves of CTAs costs more
// than it gains (int8 steps at 20 / 24 / 32 sequences: 4.15 / 4.45 / 5.24 ms against 4.49 / 4.73 /
// 5.42 with slices cut for eight waves; 32 sequences with contexts of 1024 - 4096: 58.3 against
// 62.3 us per launch). Fewer pairs are cut into 512-key slices and then treated as below.
// RB200_DECODE_WAVES=n: slices cut for n waves of CTAs, whatever the batch.
DecodePlan plan_decode(const AttnShape& s, int n_decode, int max_ctx) {
  const long long pairs_kv = std::max<long long>(1, static_cast<long long>(n_decode) * s.kv_heads);
  static const int forced_waves = [] {
    const char* e = std::getenv("RB200_DECODE_WAVES");
    return e && std::atoi(e) > 0 ? std::atoi(e) : 0;
  }();
  const bool many = pairs_kv > 2LL * sm_count() * 7 / 16;  // more than half the slots the one-wave rule below counts
  const long long want_ctas = static_cast<long long>(forced_waves ? forced_waves : 8) * sm_count();
  const int want_parts = (many && !forced_waves) ? 1 : static_cast<int>(std::max<long long>(1, div_up(want_ctas, pairs_kv)));
  int slice = round_up(std::max(1, div_up(std::max(max_ctx, 1), want_parts)), kDecodeSlice);
  slice = static_cast<int>(std::min<long long>(slice, static_cast<long long>(kDecodeSlice) * s.block_size));
  slice = std::max(kDecodeSlice, slice / kDecodeSlice * kDecodeSlice);
  int parts = div_up(std::max(max_ctx, 1), slice);
  slice = round_up(div_up(std::max(max_ctx, 1), parts), kDecodeSlice);  // the same number of slices, of even length
  // A batch of a few sequences whose 512-key slices need more than one CTA per SM, but whose
  // (token, KV head) pairs are few: at most four longer slices per pair, so that the whole grid
  // is one wave (two CTAs per SM by shared memory; an eighth of the slots is left free, because a
  // grid that needs every slot queues behind the tail of the kernel ahead) and still at least 128
  // CTAs. Every CTA is then on an SM from the start, none is longer than the others (a slice
  // bounds its keys), and the slices of a pair merge on chip below. Measured, int8 steps through
  // rb200_decode_step, against 512-key slices and the merge kernel: 5 sequences 2.74 against
  // 2.92 ms, 8 sequences 3.01 against 3.14, 12 sequences (192 CTAs of 2048 keys) 3.42 against
  // 3.64, 16 sequences 3.74 against 4.03; 4 sequences the same (2.67 / 2.65). Left alone:
  // 3 sequences (96 CTAs would be too few: 2.62 against 2.53) and plans that fill the slots
  // (12 sequences as 288 CTAs of 1536 keys: 4.02). RB200_DECODE_ONE_WAVE=0 turns it off.
  static const bool one_wave = [] {
    const char* e = std::getenv("RB200_DECODE_ONE_WAVE");
    return !(e && e[0] == '0');
  }();
  const long long slots = 2LL * sm_count() * 7 / 8;
  if (one_wave && pairs_kv * parts > sm_count() && slots / pairs_kv >= 2) {
    const int fit = static_cast<int>(std::min<long long>(4, slots / pairs_kv));
    const int slice2 = round_up(div_up(std::max(max_ctx, 1), fit), kDecodeSlice);
    const int parts2 = div_up(std::max(max_ctx, 1), slice2);
    if (parts2 < parts && parts2 >= 2 && pairs_kv * parts2 >= 128 && slice2 <= kDecodeSlice * s.block_size) {
      slice = slice2;
      parts = parts2;
    }
  }
  DecodePlan p;
  p.slice = slice;
  p.parts = parts;
  // Up to 8 slices (the portable cluster size) can be merged inside the kernel, over distributed
  // shared memory. That pays only while the whole grid is resident at once: a
  // cluster keeps all its slots until its last slice is done and must be placed inside one GPC,
  // which costs more than the merge kernel once CTAs queue (32 sequences with contexts of
  // 1024 - 4096: 72.6 us against 62.4; an 8-sequence step 3.57 ms against 3.38; a 1-sequence
  // step 2.52 against 2.56). RB200_DECODE_CLUSTER=0 turns it off, =1 uses it whenever slices <= 8.
  static const int cluster_mode = [] {
    const char* e = std::getenv("RB200_DECODE_CLUSTER");
    return e ? (e[0] == '0' ? 0 : 2) : 1;
  }();
  // resident at once: one CTA per SM, or up to two with clusters of at most four
  const bool resident = pairs_kv * parts <= sm_count() || (one_wave && parts <= 4 && pairs_kv * parts <= slots);
  p.cluster_merge = parts > 1 && parts <= 8 && (cluster_mode == 2 || (cluster_mode == 1 && resident));
  // (Slices of 256 keys in clusters of up to 16, which put twice the CTAs on a single sequence's
  // keys, were measured too: 2.49 against 2.45 ms per 1-sequence step, no gain, and left out.)
  // one slice writes the output directly, a cluster merges on chip: no partial results, no merge kernel
  p.scratch_bytes = (parts > 1 && !p.cluster_merge) ? static_cast<size_t>(n_decode) * s.heads * parts * (s.D + 2) * sizeof(float) : 0;
  return p;
}

void launch_decode_attention(const AttnShape& s, const float* q, const TokenMeta& m, const int* decode_tokens,
                             int n_decode, int max_ctx, const __half* kc, const __half* vc, float* scratch,
                             __half* out, cudaStream_t st) {
  if (n_decode == 0) return;
  const DecodePlan plan = plan_decode(s, n_decode, max_ctx);
  const int parts = plan.parts, slice = plan.slice;
  RB_REQUIRE(parts <= 65535, "decode attention: context too long for one launch");
  float* part_o = scratch;
  float* part_ml = scratch + static_cast<size_t>(n_decode) * s.heads * parts * s.D;
  switch (s.D) {
    case 16: launch_decode_d<16>(s, q, m, decode_tokens, n_decode, parts, slice, kc, vc, part_o, part_ml, out, st, plan.cluster_merge); break;
    case 32: launch_decode_d<32>(s, q, m, decode_tokens, n_decode, parts, slice, kc, vc, part_o, part_ml, out, st, plan.cluster_merge); break;
    case 64: launch_decode_d<64>(s, q, m, decode_tokens, n_decode, parts, slice, kc, vc, part_o, part_ml, out, st, plan.cluster_merge); break;
    case 128: launch_decode_d<128>(s, q, m, decode_tokens, n_decode, parts, slice, kc, vc, part_o, part_ml, out, st, plan.cluster_merge); break;
    default: fail(RB200_ERR_INVALID_ARGUMENT, "decode attention: head_dim must be 16, 32, 64 or 128");
  }
  if (parts > 1 && !plan.cluster_merge) {
    const int pairs = n_decode * s.heads;
    count_launch();
    launch_pdl(decode_merge_kernel, dim3(div_up(pairs, 4)), dim3(128), 0, st, part_o, part_ml, decode_tokens, m.pos, out,
               s.heads, s.D, s.o_stride, parts, pairs, slice);
  }
}

void launch_prefill_attention(const AttnShape& s, const float* q, const TokenMeta& m, const int2* tiles, int n_tiles,
                              const __half* kc, const __half* vc, __half* out, cudaStream_t st) {
  if (n_tiles == 0) return;
  if (umma_prefill_usable(s, q, kc, vc, out)) return launch_umma_prefill(s, q, m, tiles, n_tiles, kc, vc, out, st);
  switch (s.D) {
    case 16: launch_prefill_d<16>(s, q, m, tiles, n_tiles, kc, vc, out, st); break;
    case 32: launch_prefill_d<32>(s, q, m, tiles, n_tiles, kc, vc, out, st); break;
    case 64: launch_prefill_d<64>(s, q, m, tiles, n_tiles, kc, vc, out, st); break;
    case 128: launch_prefill_d<128>(s, q, m, tiles, n_tiles, kc, vc, out, st); break;
    default: fail(RB200_ERR_INVALID_ARGUMENT, "prefill attention: head_dim must be 16, 32, 64 or 128");
  }
}

void launch_reference_attention(const AttnShape& s, const float* q, const TokenMeta& m, int T, const __half* kc,
                                const __half* vc, __half* out, cudaStream_t st) {
  if (T == 0) return;
  RB_REQUIRE(s.D <= 256, "attention: head_dim above 256 is not supported");
  const float scale = 1.0f / sqrtf(static_cast<float>(s.D));
  count_launch();
  reference_attention_kernel<<<dim3(T, s.heads), 128, 0, st>>>(q, m, kc, vc, out, s.heads, s.kv_heads, s.D, s.block_size,
                                                              s.q_stride, s.o_stride, scale);
}

}  // namespace rb200

// ---- decode attention for callers that cannot allocate -----------------------------------
//
// The split-context kernel parks one partial result per (token, head, slice) in global
// memory before the merge. rb200_decode_attention takes that scratch from its caller; the
// entry point below keeps it in a fixed array that is part of the loaded library image, so a
// caller needs no device allocation of its own at the moment it wants attention. Every GPU
// that loads the library holds these bytes until the process exits, hence the small cap.
namespace rb200 {
namespace {

static __device__ __align__(256) unsigned char g_static_decode_scratch[RB200_STATIC_DECODE_SCRATCH_BYTES];

// Device address of the array on the current device. In host code the array's name only
// stands for the symbol; the address a kernel can use comes from cudaGetSymbolAddress, asked
// once per device with that device current.
float* static_decode_scratch() {
  static void* addr[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  RB_CUDA(cudaGetDevice(&dev));
  RB_REQUIRE(dev >= 0 && dev < 64, "decode attention: device index out of range");
  std::lock_guard<std::mutex> lock(mu);
  if (!addr[dev]) {
    void* p = nullptr;
    RB_CUDA(cudaGetSymbolAddress(&p, g_static_decode_scratch));
    addr[dev] = p;
  }
  return static_cast<float*>(addr[dev]);
}

}  // namespace
}  // namespace rb200

// ---- C boundary -----------------------------------------------------------------------

using namespace rb200;

static AttnShape shape_of(const rb200_attn_shape* s) {
  return AttnShape{s->heads, s->kv_heads, s->head_dim, s->block_size, s->q_stride, s->o_stride};
}
static TokenMeta meta_of(const rb200_token_meta* m) { return TokenMeta{m->pos, m->seq, m->table_off, m->tables}; }

static void check_shape(const AttnShape& s) {
  RB_REQUIRE(s.heads > 0 && s.kv_heads > 0 && s.heads % s.kv_heads == 0 && s.D > 0 && s.block_size > 0,
             "attention: bad head layout");
  RB_REQUIRE(s.q_stride >= s.heads * s.D && s.o_stride >= s.heads * s.D, "attention: row strides too small");
}

extern "C" {

size_t rb200_decode_scratch_bytes(const rb200_attn_shape* s, int n_decode, int max_ctx) {
  return decode_scratch_bytes(shape_of(s), n_decode, max_ctx);
}

size_t rb200_decode_plan(const rb200_attn_shape* s, int n_decode, int max_ctx, int32_t* slice_out, int32_t* parts_out) {
  const DecodePlan p = plan_decode(shape_of(s), n_decode, max_ctx);
  if (slice_out) *slice_out = p.slice;
  if (parts_out) *parts_out = p.parts;
  return p.scratch_bytes;
}

int rb200_decode_attention(const rb200_attn_shape* s, const float* q, const rb200_token_meta* m,
                           const int32_t* decode_tokens, int n_decode, int max_ctx, const void* k_pool,
                           const void* v_pool, void* scratch, size_t scratch_bytes, void* out, void* stream) {
  return guarded([&] {
    const AttnShape sh = shape_of(s);
    check_shape(sh);
    RB_REQUIRE(fast_attention_supported(sh), "decode attention: head_dim must be 16/32/64/128 and heads/kv_heads <= 16");
    RB_REQUIRE(n_decode >= 0 && max_ctx >= 1, "decode attention: bad batch");
    RB_REQUIRE(scratch_bytes >= plan_decode(sh, n_decode, max_ctx).scratch_bytes, "decode attention: scratch too small");
    launch_decode_attention(sh, q, meta_of(m), decode_tokens, n_decode, max_ctx, static_cast<const __half*>(k_pool),
                            static_cast<const __half*>(v_pool), static_cast<float*>(scratch), static_cast<__half*>(out),
                            as_stream(stream));
    RB_CUDA(cudaGetLastError());
    return 0;
  });
}

int rb200_decode_attention_static(const rb200_attn_shape* s, const float* q, const rb200_token_meta* m,
                                  const int32_t* decode_tokens, int n_decode, int max_ctx, const void* k_pool,
                                  const void* v_pool, void* out, void* stream) {
  return guarded([&] {
    const AttnShape sh = shape_of(s);
    check_shape(sh);
    RB_REQUIRE(fast_attention_supported(sh), "decode attention: head_dim must be 16/32/64/128 and heads/kv_heads <= 16");
    RB_REQUIRE(n_decode >= 0 && max_ctx >= 1, "decode attention: bad batch");
    // What this launch will really park: the slices the planner cuts, not the 512-key upper bound
    // of rb200_decode_scratch_bytes (a batch that fills the GPU with one slice per pair parks nothing).
    const size_t need = plan_decode(sh, n_decode, max_ctx).scratch_bytes;
    if (need > static_cast<size_t>(RB200_STATIC_DECODE_SCRATCH_BYTES))
      fail(RB200_ERR_INVALID_ARGUMENT, "decode attention (static scratch): this batch needs " + std::to_string(need) +
                                           " bytes of partial results, the built-in buffer holds " +
                                           std::to_string(static_cast<size_t>(RB200_STATIC_DECODE_SCRATCH_BYTES)) +
                                           "; use rb200_decode_attention with caller-owned scratch");
    // The first call on a device looks the buffer's address up (no allocation). Nothing in the
    // buffer has to start at zero: every slice's partial is written before the merge reads it.
    float* scratch = static_decode_scratch();
    launch_decode_attention(sh, q, meta_of(m), decode_tokens, n_decode, max_ctx, static_cast<const __half*>(k_pool),
                            static_cast<const __half*>(v_pool), scratch, static_cast<__half*>(out), as_stream(stream));
    RB_CUDA(cudaGetLastError());
    return 0;
  });
}

int rb200_prefill_attention(const rb200_attn_shape* s, const float* q, const rb200_token_meta* m, const int32_t* tiles,
                            int n_tiles, const void* k_pool, const void* v_pool, void* out, void* stream) {
  return guarded([&] {
    const AttnShape sh = shape_of(s);
    check_shape(sh);
    RB_REQUIRE(fast_attention_supported(sh), "prefill attention: head_dim must be 16/32/64/128");
    launch_prefill_attention(sh, q, meta_of(m), reinterpret_cast<const int2*>(tiles), n_tiles,
                             static_cast<const __half*>(k_pool), static_cast<const __half*>(v_pool),
                             static_cast<__half*>(out), as_stream(stream));
    RB_CUDA(cudaGetLastError());
    return 0;
  });
}

int rb200_reference_attention(const rb200_attn_shape* s, const float* q, const rb200_token_meta* m, int n_tokens,
                              const void* k_pool, const void* v_pool, void* out, void* stream) {
  return guarded([&] {
    const AttnShape sh = shape_of(s);
    check_shape(sh);
    launch_reference_attention(sh, q, meta_of(m), n_tokens, static_cast<const __half*>(k_pool),
                               static_cast<const __half*>(v_pool), static_cast<__half*>(out), as_stream(stream));
    RB_CUDA(cudaGetLastError());
    return 0;
  });
}

}  // extern "C"
