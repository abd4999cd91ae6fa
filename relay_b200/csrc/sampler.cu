// The sampler on the device: the next token of each logits row, and its log-probability,
// without the [rows][vocab] float32 logits ever crossing to the host.
//
// It follows relay's host sampler (engine/src/sampler.cpp) decision for decision:
//   * temperature <= 0: the greedy token, lowest id on ties (sampler.cpp:17-22);
//   * temperature > 0 without truncation (top_k 0 or >= vocab, top_p >= 1; what RL sampling
//     uses): the inverse CDF in id order of e_i = expf((l_i - max) / T), float32 terms summed
//     in float64, the random number a pure function of (seed, index) (sampler.cpp:9-15, 33-61);
//   * the log-probability Engine reports with the token (engine/src/engine.cpp:270-282):
//     (l_tok - max) / T - log(sum) from the same sum when sampling, log softmax at T = 1 in
//     float64 when greedy (sampler.cpp:24-31).
// Rows that ask for top-k or nucleus truncation need the vocabulary in sorted order
// (sampler.cpp:77-104); those are refused here and stay on the caller's host path.
//
// One CTA of 1024 threads per row. The float64 sums are taken in a different order than the
// host's sequential loop (per-lane partial sums, then a warp and a block reduction), which moves
// the total by a few units of 1e-16 relative: the token only differs when the scaled random
// number lands that close to a boundary of the CDF.
#include "kernels.h"

namespace rb200 {

namespace {

constexpr int kSampleThreads = 1024;
constexpr int kSampleWarps = kSampleThreads / 32;

// relay::uniform01 (engine/src/sampler.cpp:9-15): splitmix64 of (seed, index), 53 bits.
__device__ __forceinline__ double uniform01(unsigned long long seed, unsigned long long index) {
  unsigned long long z = seed + 0x9E3779B97F4A7C15ULL * (index + 1);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  z ^= z >> 31;
  return static_cast<double>(z >> 11) * (1.0 / 9007199254740992.0);
}

__device__ __forceinline__ double warp_sum_f64(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void __launch_bounds__(kSampleThreads)
sample_rows_kernel(const float* __restrict__ logits, int V, const rb200_sampling_params* __restrict__ params,
                   int* __restrict__ token_out, double* __restrict__ logprob_out) {
  pdl_trigger();
  pdl_wait();
  __shared__ float s_max[kSampleWarps];
  __shared__ int s_arg[kSampleWarps];
  __shared__ double s_sum[kSampleWarps + 1];
  __shared__ int s_token;
  const float* row = logits + static_cast<long long>(blockIdx.x) * V;
  const rb200_sampling_params p = params[blockIdx.x];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool greedy = !(p.temperature > 0.0f);

  // ---- the row's maximum and its lowest id ----
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += kSampleThreads) {
    const float v = row[i];
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
  auto merge = [&](float ov, int oi) {
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) merge(__shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
  if (lane == 0) {
    s_max[warp] = best;
    s_arg[warp] = bi;
  }
  __syncthreads();
  best = s_max[0];
  bi = s_arg[0];
#pragma unroll 1
  for (int w = 1; w < kSampleWarps; ++w) merge(s_max[w], s_arg[w]);
  const float mx = best;  // every thread holds the same (max, lowest id of the max)
  if (bi == 0x7fffffff) bi = 0;  // a row without any finite comparison (all NaN): the host's loop keeps id 0

  if (greedy) {
    if (logprob_out != nullptr) {
      // log_prob(logits, vocab, temperature <= 0 -> 1.0, token): float64 throughout
      double part = 0.0;
      const double dmx = static_cast<double>(mx);
      for (int i = threadIdx.x; i < V; i += kSampleThreads) part += exp(static_cast<double>(row[i]) - dmx);
      part = warp_sum_f64(part);
      if (lane == 0) s_sum[warp] = part;
      __syncthreads();
      if (threadIdx.x == 0) {
        double total = 0.0;
        for (int w = 0; w < kSampleWarps; ++w) total += s_sum[w];
        logprob_out[blockIdx.x] = (static_cast<double>(row[bi]) - dmx) - log(total);
      }
    }
    if (threadIdx.x == 0) token_out[blockIdx.x] = bi;
    return;
  }

  // ---- inverse CDF in id order ----
  // Warp w owns ids [w * seg, (w + 1) * seg), seg a multiple of 32; lane l of the warp reads ids
  // seg0 + 32 j + l (coalesced), so (j, l) in that order is id order.
  const float inv_t = 1.0f / p.temperature;
  const int seg = (V + kSampleWarps * 32 - 1) / (kSampleWarps * 32) * 32;
  const int seg0 = warp * seg, seg1 = min(V, seg0 + seg);
  double part = 0.0;
  for (int i = seg0 + lane; i < seg1; i += 32) part += static_cast<double>(expf((row[i] - mx) * inv_t));
  part = warp_sum_f64(part);
  if (lane == 0) s_sum[warp] = part;
  if (threadIdx.x == 0) s_token = -1;
  __syncthreads();
  // exclusive prefix of the warp sums, the same sequence of additions in every thread
  double before = 0.0, total = 0.0;
#pragma unroll 1
  for (int w = 0; w < kSampleWarps; ++w) {
    if (w == warp) before = total;
    total += s_sum[w];
  }
  const double r = uniform01(p.seed, p.index) * total;
  const double after = (warp == kSampleWarps - 1) ? INFINITY : before + s_sum[warp];
  // exactly one warp has before <= r < after (the last one takes everything from its start on)
  if (before <= r && r < after) {
    double carry = before;
    int found = -1, last_mass = -1;
    for (int j0 = seg0; j0 < seg1 && found < 0; j0 += 32) {
      const int i = j0 + lane;
      const float e = i < seg1 ? expf((row[i] - mx) * inv_t) : 0.0f;
      double incl = static_cast<double>(e);
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const double up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      const unsigned hit = __ballot_sync(0xffffffffu, i < seg1 && carry + incl > r);
      const unsigned mass = __ballot_sync(0xffffffffu, e > 0.0f);
      if (mass) last_mass = j0 + 31 - __clz(mass);
      if (hit) found = j0 + __ffs(hit) - 1;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    // Rounding left r at or above the last partial sum: the last token with any mass
    // (engine/src/sampler.cpp:52-53), which is in this segment or, failing that, the greedy one.
    if (found < 0) found = last_mass >= 0 ? last_mass : bi;
    if (lane == 0) s_token = found;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int tok = s_token >= 0 ? s_token : bi;
    token_out[blockIdx.x] = tok;
    if (logprob_out != nullptr)
      logprob_out[blockIdx.x] =
          (static_cast<double>(row[tok]) - static_cast<double>(mx)) * static_cast<double>(inv_t) - log(total);
  }
}

}  // namespace

bool sampling_on_device(const rb200_sampling_params& p, int V) {
  if (!(p.temperature > 0.0f)) return true;  // greedy
  return (p.top_k <= 0 || p.top_k >= V) && p.top_p >= 1.0f;
}

void launch_sample_rows(const float* logits, int R, int V, const rb200_sampling_params* params, int* token_out,
                        double* logprob_out, cudaStream_t st) {
  if (R == 0) return;
  count_launch();
  launch_pdl(sample_rows_kernel, dim3(R), dim3(kSampleThreads), 0, st, logits, V, params, token_out, logprob_out);
}

}  // namespace rb200

using namespace rb200;

extern "C" int rb200_sample_rows(const float* logits, int R, int V, const rb200_sampling_params* params, int32_t* token_out,
                                 double* logprob_out, void* stream) {
  return guarded([&] {
    RB_REQUIRE(R >= 0 && V > 0 && logits && params && token_out, "sample_rows: bad arguments");
    launch_sample_rows(logits, R, V, params, token_out, logprob_out, as_stream(stream));
    RB_CUDA(cudaGetLastError());
    return 0;
  });
}
