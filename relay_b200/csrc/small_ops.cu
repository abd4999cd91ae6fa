// The memory-bound kernels around the GEMMs and attention: embedding gather, RMSNorm,
// bias + RoPE + paged-KV append, SiLU*up, fp32->fp16 / int8 weight conversion, KV page
// gather/scatter and the greedy-token reduction. Each replaces one small kernel of the
// reference's CUDA backend (engine/src/cuda_backend.cu:110-270); all are vectorised and
// bound by HBM traffic or launch latency.
#include "i8_digits.cuh"
#include "kernels.h"
#include "tcgen05.cuh"

namespace rb200 {

namespace {

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = lane < nw ? red[lane] : 0.0f;
  r = warp_sum(r);
  __syncthreads();
  return r;
}

__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = lane < nw ? red[lane] : 0.0f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r = fmaxf(r, __shfl_xor_sync(0xffffffffu, r, o));
  __syncthreads();
  return r;
}

// x[t, :] = float(table[tokens[t], :])  (engine/src/cuda_backend.cu:150-154)
__global__ void embed_kernel(const int* __restrict__ tokens, const __half* __restrict__ table, float* __restrict__ x,
                             int H, int ld_table) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const __half* row = table + static_cast<long long>(tokens[t]) * ld_table;
  float* dst = x + static_cast<long long>(t) * H;
  if ((H & 7) == 0) {
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
      uint4 raw = *reinterpret_cast<const uint4*>(row + i);
      const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
      float2 a = __half22float2(h2[0]), b = __half22float2(h2[1]), c = __half22float2(h2[2]), d = __half22float2(h2[3]);
      *reinterpret_cast<float4*>(dst + i) = make_float4(a.x, a.y, b.x, b.y);
      *reinterpret_cast<float4*>(dst + i + 4) = make_float4(c.x, c.y, d.x, d.y);
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = __half2float(row[i]);
  }
}

// out[r, :] = w * (x[row(r), :] * 1/sqrt(mean(x^2) + eps)) as fp16; columns H..ld_out-1 zero.
// (engine/src/cuda_backend.cu:157-167; the CPU backend's form is engine/src/cpu_backend.cpp:47-52.)
// With `digits` (H and ld_out multiples of 4): the fp16 row is also written as the int8 digits
// the integer tensor-core linear reads (digits[d][r][0..ld_out), tscale[r]; i8_digits.cuh), so
// that the GEMM behind this kernel needs no pass over the activations of its own.
__global__ void rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w,
                               __half* __restrict__ out, int H, int ld_out, float eps, int8_t* __restrict__ digits,
                               float* __restrict__ tscale) {
  pdl_trigger();
  __shared__ float red[32];
  const int r = blockIdx.x;
  const float* xr = x + static_cast<long long>(rows ? rows[r] : r) * H;
  __half* o = out + static_cast<long long>(r) * ld_out;
  float ss = 0.0f;
  const bool vec = (H & 3) == 0;
  // Rows of up to 8 values per thread (every width the path's models have) stay in registers
  // between the two passes, and the norm weights are fetched before the dependency wait (they and
  // the row list do not come from the kernel ahead): one round trip to memory behind the wait
  // instead of three.
  const bool cached = vec && H <= static_cast<int>(blockDim.x) * 8;
  float4 xc[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
  float4 wc[2] = {xc[0], xc[0]};
  if (cached) {
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int i = (k * blockDim.x + threadIdx.x) * 4;
      if (i < H) wc[k] = *reinterpret_cast<const float4*>(w + i);
    }
  }
  pdl_wait();
  if (cached) {
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int i = (k * blockDim.x + threadIdx.x) * 4;
      if (i < H) xc[k] = *reinterpret_cast<const float4*>(xr + i);
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) ss += xc[k].x * xc[k].x + xc[k].y * xc[k].y + xc[k].z * xc[k].z + xc[k].w * xc[k].w;
  } else if (vec) {
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      float4 v = *reinterpret_cast<const float4*>(xr + i);
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) ss += xr[i] * xr[i];
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / static_cast<float>(H) + eps);
  float mx = 0.0f;  // largest magnitude of the rounded row
  if (vec) {
    for (int i = threadIdx.x * 4, k = 0; i < H; i += blockDim.x * 4, ++k) {
      float4 v, g;
      if (cached) {
        v = k == 0 ? xc[0] : xc[1];
        g = k == 0 ? wc[0] : wc[1];
      } else {
        v = *reinterpret_cast<const float4*>(xr + i);
        g = *reinterpret_cast<const float4*>(w + i);
      }
      uint2 p;
      p.x = pack_half2(g.x * (v.x * inv), g.y * (v.y * inv));
      p.y = pack_half2(g.z * (v.z * inv), g.w * (v.w * inv));
      *reinterpret_cast<uint2*>(o + i) = p;
      const __half2 m = __hmax2(__habs2(*reinterpret_cast<__half2*>(&p.x)), __habs2(*reinterpret_cast<__half2*>(&p.y)));
      mx = fmaxf(mx, fmaxf(__low2float(m), __high2float(m)));
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = __float2half_rn(w[i] * (xr[i] * inv));
  }
  for (int i = H + threadIdx.x; i < ld_out; i += blockDim.x) o[i] = __float2half_rn(0.0f);
  if (digits != nullptr) {  // the whole grid or none of it
    mx = block_max(mx, red);
    float up, down;
    i8d::digit_scales(mx, up, down);
    if (threadIdx.x == 0) tscale[r] = down;
    const long long plane = static_cast<long long>(gridDim.x) * ld_out;
    int8_t* d = digits + static_cast<long long>(r) * ld_out;
    for (int i = threadIdx.x * 4; i < ld_out; i += blockDim.x * 4) {
      // i < H: the four halves this thread stored above
      const uint2 p = i < H ? *reinterpret_cast<const uint2*>(o + i) : make_uint2(0u, 0u);
      uint32_t dw[i8d::kDigits];
      i8d::digits4(p, up, dw);
#pragma unroll
      for (int g = 0; g < i8d::kDigits; ++g) *reinterpret_cast<uint32_t*>(d + g * plane + i) = dw[g];
    }
  }
}

// Bias, RoPE on the q and k heads in place (pairs (i, i + D/2), angle = pos * inv_freq[i]),
// then k and v rounded to fp16 into the token's slot of the paged pools
// (engine/src/cuda_backend.cu:171-198; page addressing engine/include/relay/kv_cache.h:32-35).
// The D/2 (cos, sin) pairs of the token are computed once and shared by all heads.
__global__ void qkv_post_kernel(float* __restrict__ qkv, const float* __restrict__ bias,
                                const float* __restrict__ inv_freq, TokenMeta m, __half* __restrict__ kc,
                                __half* __restrict__ vc, int heads, int kv_heads, int D, int block_size) {
  pdl_trigger();
  extern __shared__ float cs[];  // [D/2] cos, [D/2] sin
  // gridDim.y blocks share a token (heads and kv_heads are multiples of it): each takes its share
  // of the q heads and of the k/v heads.
  const int t = blockIdx.x, part = blockIdx.y, parts = gridDim.y;
  const int Q = heads * D, KV = kv_heads * D, QKV = Q + 2 * KV, half = D / 2;
  float* row = qkv + static_cast<long long>(t) * QKV;
  // The rotation angles and the token's page depend on the batch metadata only: both are ready
  // by the time the projection ahead of this kernel has finished.
  const int p = m.pos[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s, c;
    sincosf(static_cast<float>(p) * inv_freq[i], &s, &c);
    cs[i] = c;
    cs[half + i] = s;
  }
  const int block = m.tables[m.table_off[m.seq[t]] + p / block_size], slot = p % block_size;
  __syncthreads();
  pdl_wait();
  // rotation: this part's q heads, then this part's k heads (stored below by the same block)
  const int qh = heads / parts, kh = kv_heads / parts;
  const int items = (qh + kh) * half;
  for (int idx = threadIdx.x; idx < items; idx += blockDim.x) {
    const int hl = idx / half, i = idx - hl * half;
    const int h = hl < qh ? part * qh + hl : heads + part * kh + (hl - qh);  // head index in the qkv row
    float* v = row + h * D;
    const float c = cs[i], s = cs[half + i];
    float a = v[i], b = v[i + half];
    if (bias) {
      a += bias[h * D + i];
      b += bias[h * D + i + half];
    }
    v[i] = a * c - b * s;
    v[i + half] = b * c + a * s;
  }
  __syncthreads();
  // k (rotated above by this very block) and v (plus its bias) -> fp16 pages
  const int kv0 = part * kh * D, kv1 = kv0 + kh * D;
  for (int idx = kv0 + threadIdx.x * 2; idx < kv1; idx += blockDim.x * 2) {
    const int h = idx / D, d = idx - h * D;
    const long long off = (static_cast<long long>(block) * kv_heads + h) * block_size * D +
                          static_cast<long long>(slot) * D + d;
    const float2 k2 = *reinterpret_cast<const float2*>(row + Q + idx);
    float2 v2 = *reinterpret_cast<const float2*>(row + Q + KV + idx);
    if (bias) {  // written back as well: the row then is what the reference's kernel leaves in place
      v2.x += bias[Q + KV + idx];
      v2.y += bias[Q + KV + idx + 1];
      *reinterpret_cast<float2*>(row + Q + KV + idx) = v2;
    }
    *reinterpret_cast<__half2*>(kc + off) = __floats2half2_rn(k2.x, k2.y);
    *reinterpret_cast<__half2*>(vc + off) = __floats2half2_rn(v2.x, v2.y);
  }
}

// act[t, i] = g / (1 + exp(-g)) * u  with g = gu[t, i], u = gu[t, I + i]
// (engine/src/cuda_backend.cu:245-253; CPU form engine/src/cpu_backend.cpp:189-194).
__global__ void silu_mul_kernel(const float* __restrict__ gu, __half* __restrict__ act, int I, int ld_act) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.y;
  const float* g = gu + static_cast<long long>(t) * 2 * I;
  const float* u = g + I;
  __half* a = act + static_cast<long long>(t) * ld_act;
  const int i0 = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i0 >= ld_act) return;
  if ((I & 3) == 0 && i0 + 4 <= I) {
    const float4 gv = *reinterpret_cast<const float4*>(g + i0);
    const float4 uv = *reinterpret_cast<const float4*>(u + i0);
    uint2 p;
    p.x = pack_half2(gv.x / (1.0f + expf(-gv.x)) * uv.x, gv.y / (1.0f + expf(-gv.y)) * uv.y);
    p.y = pack_half2(gv.z / (1.0f + expf(-gv.z)) * uv.z, gv.w / (1.0f + expf(-gv.w)) * uv.w);
    *reinterpret_cast<uint2*>(a + i0) = p;
  } else {
    for (int i = i0; i < i0 + 4 && i < ld_act; ++i)
      a[i] = __float2half_rn(i < I ? g[i] / (1.0f + expf(-g[i])) * u[i] : 0.0f);
  }
}

// The same for the few-token steps whose down projection reads its input as int8 digits
// (i8_digits.cuh): a cluster of kSiluCluster CTAs per token, each taking an equal share of the row.
// A CTA writes its share of the fp16 row as above (same expression, same rounding) and finds its
// largest magnitude; the shares' maxima are exchanged through distributed shared memory, and every
// CTA then writes the digit planes of its share against the row's scale (rank 0 writes the scale),
// so that projection needs no digit pass of its own. I and ld_act are multiples of 4, ld_act of
// 4 * kSiluCluster.
constexpr int kSiluCluster = 8;

__global__ void silu_mul_row_kernel(const float* __restrict__ gu, __half* __restrict__ act, int I, int ld_act,
                                    int8_t* __restrict__ digits, float* __restrict__ tscale) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[32];
  __shared__ float share_max;
  const int t = blockIdx.y, rank = blockIdx.x;  // the cluster spans x
  const int per = ld_act / kSiluCluster, lo = rank * per, hi = lo + per;
  const float* g = gu + static_cast<long long>(t) * 2 * I;
  const float* u = g + I;
  __half* a = act + static_cast<long long>(t) * ld_act;
  float mx = 0.0f;
  for (int i = lo + threadIdx.x * 4; i < hi; i += blockDim.x * 4) {
    uint2 p = make_uint2(0u, 0u);
    if (i < I) {
      const float4 gv = *reinterpret_cast<const float4*>(g + i);
      const float4 uv = *reinterpret_cast<const float4*>(u + i);
      p.x = pack_half2(gv.x / (1.0f + expf(-gv.x)) * uv.x, gv.y / (1.0f + expf(-gv.y)) * uv.y);
      p.y = pack_half2(gv.z / (1.0f + expf(-gv.z)) * uv.z, gv.w / (1.0f + expf(-gv.w)) * uv.w);
    }
    *reinterpret_cast<uint2*>(a + i) = p;
    const __half2 m = __hmax2(__habs2(*reinterpret_cast<__half2*>(&p.x)), __habs2(*reinterpret_cast<__half2*>(&p.y)));
    mx = fmaxf(mx, fmaxf(__low2float(m), __high2float(m)));
  }
  mx = block_max(mx, red);
  if (threadIdx.x == 0) share_max = mx;
  tc::cluster_sync_all();  // every share's maximum is in its CTA's shared memory
  float row_max = 0.0f;
#pragma unroll
  for (int r = 0; r < kSiluCluster; ++r) row_max = fmaxf(row_max, tc::ld_dsmem_f32(smem_u32(&share_max), r));
  tc::cluster_sync_all();  // nobody leaves while a peer may still read its shared memory
  float up, down;
  i8d::digit_scales(row_max, up, down);
  if (rank == 0 && threadIdx.x == 0) tscale[t] = down;
  const long long plane = static_cast<long long>(gridDim.y) * ld_act;
  int8_t* d = digits + static_cast<long long>(t) * ld_act;
  for (int i = lo + threadIdx.x * 4; i < hi; i += blockDim.x * 4) {
    const uint2 p = *reinterpret_cast<const uint2*>(a + i);  // the four halves this thread stored above
    uint32_t dw[i8d::kDigits];
    i8d::digits4(p, up, dw);
#pragma unroll
    for (int k = 0; k < i8d::kDigits; ++k) *reinterpret_cast<uint32_t*>(d + k * plane + i) = dw[k];
  }
}

// fp32 -> fp16 round-to-nearest-even, the bits of the host's f32_to_f16
// (engine/src/cuda_backend.cu:110-116, engine/src/safetensors.cpp:65-88).
__global__ void f32_to_f16_kernel(const float* __restrict__ in, __half* __restrict__ out, size_t n) {
  pdl_trigger();
  pdl_wait();
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    out[i] = __float2half_rn(in[i]);
}

// Rows [row0, row0 + rows) of an [N][K] fp32 matrix into fp16 rows of ld halves, zero padded.
__global__ void convert_rows_f16_kernel(const float* __restrict__ in, __half* __restrict__ out, int K, int ld) {
  const long long r = blockIdx.x;
  const float* src = in + r * K;
  __half* dst = out + r * ld;
  for (int k = threadIdx.x; k < ld; k += blockDim.x) dst[k] = __float2half_rn(k < K ? src[k] : 0.0f);
}

// Per-row symmetric int8: scale = max|w| / 127 (1 for a zero row), q = rint(w / scale)
// (engine/src/cuda_backend.cu:282-304), rows padded with zeros to ld bytes.
__global__ void quantize_rows_int8_kernel(const float* __restrict__ in, int8_t* __restrict__ out,
                                          float* __restrict__ scale, int K, int ld) {
  __shared__ float red[32];
  const long long r = blockIdx.x;
  const float* src = in + r * K;
  float mx = 0.0f;
  for (int k = threadIdx.x; k < K; k += blockDim.x) mx = fmaxf(mx, fabsf(src[k]));
  mx = warp_max(mx);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = (threadIdx.x & 31) < ((blockDim.x + 31) >> 5) ? red[threadIdx.x & 31] : 0.0f;
  mx = warp_max(mx);
  const float sc = mx > 0.0f ? mx / 127.0f : 1.0f;
  if (threadIdx.x == 0) scale[r] = sc;
  int8_t* dst = out + r * ld;
  for (int k = threadIdx.x; k < ld; k += blockDim.x)
    dst[k] = k < K ? static_cast<int8_t>(__float2int_rn(src[k] / sc)) : static_cast<int8_t>(0);
}

// Blocks of one layer's K and V into / out of a contiguous [K of each block][V of each
// block] staging buffer, 16 bytes per thread step (engine/src/cuda_backend.cu:257-270).
__global__ void kv_gather_kernel(const uint4* __restrict__ k, const uint4* __restrict__ v,
                                 const int* __restrict__ blocks, int n, long long block_vec, uint4* __restrict__ out) {
  const int i = blockIdx.x, which = blockIdx.y;
  const uint4* src = (which ? v : k) + static_cast<long long>(blocks[i]) * block_vec;
  uint4* dst = out + (static_cast<long long>(which) * n + i) * block_vec;
  for (long long e = blockIdx.z * blockDim.x + threadIdx.x; e < block_vec; e += static_cast<long long>(gridDim.z) * blockDim.x)
    dst[e] = src[e];
}

__global__ void kv_scatter_kernel(uint4* __restrict__ k, uint4* __restrict__ v, const int* __restrict__ blocks, int n,
                                  long long block_vec, const uint4* __restrict__ in) {
  const int i = blockIdx.x, which = blockIdx.y;
  uint4* dst = (which ? v : k) + static_cast<long long>(blocks[i]) * block_vec;
  const uint4* src = in + (static_cast<long long>(which) * n + i) * block_vec;
  for (long long e = blockIdx.z * blockDim.x + threadIdx.x; e < block_vec; e += static_cast<long long>(gridDim.z) * blockDim.x)
    dst[e] = src[e];
}

// Greedy token of each logits row; ties go to the lowest id (engine/src/sampler.cpp:17-22).
__global__ void argmax_rows_kernel(const float* __restrict__ logits, int V, int* __restrict__ token_out,
                                   float* __restrict__ logit_out) {
  pdl_trigger();
  pdl_wait();
  __shared__ float sv[32];
  __shared__ int si[32];
  const float* row = logits + static_cast<long long>(blockIdx.x) * V;
  float best;
  int bi;
  strided_argmax(row, V, threadIdx.x, blockDim.x, best, bi);
  auto merge = [&](float ov, int oi) {
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) merge(__shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) {
    sv[warp] = best;
    si[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    best = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) merge(__shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
    if (lane == 0) {
      token_out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
      if (logit_out) logit_out[blockIdx.x] = best;
    }
  }
}

}  // namespace

void launch_embed(const int* tokens, const __half* table, float* x, int T, int H, int ld_table, cudaStream_t st) {
  if (T == 0) return;
  count_launch();
  launch_pdl(embed_kernel, dim3(T), dim3(128), 0, st, tokens, table, x, H, ld_table);
}

void launch_rmsnorm(const float* x, const int* rows, const float* w, __half* out, int R, int H, int ld_out, float eps,
                    cudaStream_t st, I8Digits dg) {
  if (R == 0) return;
  const int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : 128);
  count_launch();
  RB_REQUIRE(dg.digits == nullptr || (H % 4 == 0 && ld_out % 4 == 0 && dg.tscale != nullptr), "rmsnorm: digits need rows of whole 4-element groups");
  launch_pdl(rmsnorm_kernel, dim3(R), dim3(threads), 0, st, x, rows, w, out, H, ld_out, eps, dg.digits, dg.tscale);
}

void launch_qkv_post(float* qkv, const float* bias, const float* inv_freq, const TokenMeta& m, int T, __half* kc,
                     __half* vc, int heads, int kv_heads, int D, int block_size, cudaStream_t st) {
  if (T == 0) return;
  count_launch();
  // Several blocks per token when the heads divide evenly (a block stores the k values it rotated itself).
  int parts = 1;
  for (int c : {4, 2})
    if (kv_heads % c == 0 && (heads % c == 0) && T * c <= 8192) {
      parts = c;
      break;
    }
  launch_pdl(qkv_post_kernel, dim3(T, parts), dim3(256), D * sizeof(float), st, qkv, bias, inv_freq, m, kc, vc, heads, kv_heads, D,
             block_size);
}

void launch_silu_mul(const float* gu, __half* act, int T, int I, int ld_act, cudaStream_t st, I8Digits dg) {
  if (T == 0) return;
  count_launch();
  RB_REQUIRE(dg.digits == nullptr || ((I & 3) == 0 && ld_act % (4 * kSiluCluster) == 0 && dg.tscale != nullptr),
             "silu_mul: digits need I a multiple of 4 and rows of whole 32-element groups");
  if (dg.digits != nullptr) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(kSiluCluster, T);
    cfg.blockDim = dim3(512);
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kSiluCluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    int8_t* digits = dg.digits;
    float* tscale = dg.tscale;
    RB_CUDA(cudaLaunchKernelEx(&cfg, silu_mul_row_kernel, gu, act, I, ld_act, digits, tscale));
    return;
  }
  dim3 grid(div_up(ld_act, 4 * 256), T);
  launch_pdl(silu_mul_kernel, grid, dim3(256), 0, st, gu, act, I, ld_act);
}

void launch_f32_to_f16(const float* in, __half* out, size_t n, cudaStream_t st) {
  if (n == 0) return;
  const unsigned grid = static_cast<unsigned>(std::min<size_t>((n + 255) / 256, 8192));
  count_launch();
  launch_pdl(f32_to_f16_kernel, dim3(grid), dim3(256), 0, st, in, out, n);
}

void launch_convert_rows_f16(const float* in, __half* out, int rows, int K, int ld, cudaStream_t st) {
  if (rows == 0) return;
  count_launch();
  convert_rows_f16_kernel<<<rows, 256, 0, st>>>(in, out, K, ld);
}

void launch_quantize_rows_int8(const float* in, int8_t* out, float* scale, int rows, int K, int ld, cudaStream_t st) {
  if (rows == 0) return;
  count_launch();
  quantize_rows_int8_kernel<<<rows, 256, 0, st>>>(in, out, scale, K, ld);
}

void launch_kv_gather(const void* k, const void* v, const int* blocks, int n, size_t block_bytes, void* staging,
                      cudaStream_t st) {
  if (n == 0) return;
  const long long vec = static_cast<long long>(block_bytes / 16);
  dim3 grid(n, 2, static_cast<unsigned>(std::max<long long>(1, std::min<long long>(8, vec / 256))));
  count_launch();
  kv_gather_kernel<<<grid, 256, 0, st>>>(static_cast<const uint4*>(k), static_cast<const uint4*>(v), blocks, n, vec,
                                         static_cast<uint4*>(staging));
}

void launch_kv_scatter(void* k, void* v, const int* blocks, int n, size_t block_bytes, const void* staging,
                       cudaStream_t st) {
  if (n == 0) return;
  const long long vec = static_cast<long long>(block_bytes / 16);
  dim3 grid(n, 2, static_cast<unsigned>(std::max<long long>(1, std::min<long long>(8, vec / 256))));
  count_launch();
  kv_scatter_kernel<<<grid, 256, 0, st>>>(static_cast<uint4*>(k), static_cast<uint4*>(v), blocks, n, vec,
                                          static_cast<const uint4*>(staging));
}

void launch_argmax_rows(const float* logits, int R, int V, int* token_out, float* logit_out, cudaStream_t st) {
  if (R == 0) return;
  count_launch();
  launch_pdl(argmax_rows_kernel, dim3(R), dim3(V >= 8192 ? 1024 : 256), 0, st, logits, V, token_out, logit_out);
}

}  // namespace rb200

// ---- C boundary -----------------------------------------------------------------------

using namespace rb200;

static TokenMeta meta_of(const rb200_token_meta* m) { return TokenMeta{m->pos, m->seq, m->table_off, m->tables}; }

extern "C" {

int rb200_embed(const int32_t* tokens, const void* table, float* x, int T, int H, int ld_table, void* stream) {
  return guarded([&] {
    RB_REQUIRE(T >= 0 && H > 0 && ld_table >= H, "embed: bad shape");
    launch_embed(tokens, static_cast<const __half*>(table), x, T, H, ld_table, as_stream(stream));
    RB_CUDA(cudaGetLastError());
    return 0;
  });
}

int rb200_rmsnorm(const float* x, const int32_t* rows, const float* w, void* out, int R, int H, int ld_out, float eps,
                  void* stream) {
  return guarded([&] {
    RB_REQUIRE(R >= 0 && H > 0 && ld_out >= H, "rmsnorm: bad shape");
    launch_rmsnorm(x, rows, w, static_cast<__half*>(out), R, H, ld_out, eps, as_stream(stream));
    RB_CUDA(cudaGetLastError());
    return 0;
  });
}

int rb200_qkv_post(float* qkv, const float* bias, const float* inv_freq, const rb200_token_meta* m, int T, void* k_pool,
                   void* v_pool, int heads, int kv_heads, int head_dim, int block_size, void* stream) {
  return guarded([&] {
    RB_REQUIRE(T >= 0 && heads > 0 && kv_heads > 0 && head_dim > 0 && head_dim % 2 == 0 && block_size > 0,
               "qkv_post: bad shape");
    launch_qkv_post(qkv, bias, inv_freq, meta_of(m), T, static_cast<__half*>(k_pool), static_cast<__half*>(v_pool),
                    heads, kv_heads, head_dim, block_size, as_stream(stream));
    RB_CUDA(cudaGetLastError());
    return 0;
  });
}

int rb200_silu_mul(const float* gu, void* act, int T, int I, int ld_act, void* stream) {
  return guarded([&] {
    RB_REQUIRE(T >= 0 && I > 0 && ld_act >= I, "silu_mul: bad shape");
    launch_silu_mul(gu, static_cast<__half*>(act), T, I, ld_act, as_stream(stream));
    RB_CUDA(cudaGetLastError());
    return 0;
  });
}

int rb200_f32_to_f16(const float* in, void* out, size_t n, void* stream) {
  return guarded([&] {
    launch_f32_to_f16(in, static_cast<__half*>(out), n, as_stream(stream));
    RB_CUDA(cudaGetLastError());
    return 0;
  });
}

int rb200_kv_gather(const void* k_pool, const void* v_pool, const int32_t* blocks, int n, size_t block_bytes,
                    void* staging, void* stream) {
  return guarded([&] {
    RB_REQUIRE(block_bytes % 16 == 0, "a KV block must be a multiple of 16 bytes");
    launch_kv_gather(k_pool, v_pool, blocks, n, block_bytes, staging, as_stream(stream));
    RB_CUDA(cudaGetLastError());
    return 0;
  });
}

int rb200_kv_scatter(void* k_pool, void* v_pool, const int32_t* blocks, int n, size_t block_bytes, const void* staging,
                     void* stream) {
  return guarded([&] {
    RB_REQUIRE(block_bytes % 16 == 0, "a KV block must be a multiple of 16 bytes");
    launch_kv_scatter(k_pool, v_pool, blocks, n, block_bytes, staging, as_stream(stream));
    RB_CUDA(cudaGetLastError());
    return 0;
  });
}

int rb200_argmax_rows(const float* logits, int R, int V, int32_t* token_out, float* logit_out, void* stream) {
  return guarded([&] {
    RB_REQUIRE(R >= 0 && V > 0, "argmax_rows: bad shape");
    launch_argmax_rows(logits, R, V, token_out, logit_out, as_stream(stream));
    RB_CUDA(cudaGetLastError());
    return 0;
  });
}

}  // extern "C"
