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
//   * temperature > 0 with top-k and / or nucleus truncation: the candidates in order of
//     decreasing logit, ties by id (sampler.cpp:77-104), by a kernel of its own further down.
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
  // rows with top-k / nucleus truncation belong to sample_truncated_rows_kernel
  if (!greedy && !((p.top_k <= 0 || p.top_k >= V) && p.top_p >= 1.0f)) return;

  // ---- the row's maximum and its lowest id ----
  float best;
  int bi;
  strided_argmax(row, V, threadIdx.x, kSampleThreads, best, bi);
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


// ---- rows with top-k / nucleus truncation (engine/src/sampler.cpp:77-104) --------------------
//
// The host sorts the whole vocabulary by (logit descending, id ascending), keeps the k best,
// turns them into probabilities in that order, cuts the nucleus, and walks the kept ones in
// that order. Here the sorted order is produced a band at a time: kBand candidates (ranks
// [b kBand, (b + 1) kBand)) are found by a bisection on the key value (how many logits are at
// least this large), with equal logits told apart by id, gathered into shared memory and
// sorted there; one thread then adds and walks the band's probabilities one after the other,
// exactly as the host's loops do. Truncated sampling almost always ends inside the first band
// (top_k <= kBand, or a nucleus among the kBand most likely tokens); otherwise the next
// bands follow. Sums that span several bands, and the all-vocabulary sum a nucleus without top-k
// needs, are added in another order than the host's, which moves them by parts in 1e-16.

constexpr int kBand = 2048;

// Larger float <=> larger key, equal floats <=> equal keys (-0 and +0 compare equal on the host,
// so they share a key and fall back to the id order).
__device__ __forceinline__ uint32_t order_key(float x) {
  const uint32_t b = x == 0.0f ? 0u : __float_as_uint(x);
  return (b >> 31) ? ~b : (b ^ 0x80000000u);
}

struct TruncShared {
  uint32_t key[kBand];
  int id[kBand];
  double prob[kBand];
  int cnt[kSampleWarps];
  int cnt2[kSampleWarps];
  double dsum[kSampleWarps];
  float fmax[kSampleWarps];
  int fill;       // members gathered so far
  int flag;       // loop control written by thread 0
  int token;
  double carry, carry2;  // running sums that thread 0 carries from band to band
};

// A boundary of the sorted order: the prefix "key > tau, plus the first t ties at tau by id".
struct Cut {
  uint32_t tau;
  int t;
  bool none;  // the empty prefix
};

struct RowView {
  const float* row;
  int V, seg0, seg1, lane, warp;
};

// Number of logits whose key satisfies pred; every thread gets the result.
template <class Pred>
__device__ int block_count(const RowView& r, TruncShared& sh, Pred pred) {
  int c = 0;
  for (int i = r.seg0 + r.lane; i < r.seg1; i += 32) c += pred(order_key(r.row[i])) ? 1 : 0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  __syncthreads();  // the previous use of sh.cnt is over
  if (r.lane == 0) sh.cnt[r.warp] = c;
  __syncthreads();
  int total = 0;
#pragma unroll 1
  for (int w = 0; w < kSampleWarps; ++w) total += sh.cnt[w];
  return total;
}

// The cut behind the c best logits (1 <= c <= V).
__device__ Cut find_cut(const RowView& r, TruncShared& sh, int c) {
  unsigned long long lo = 0, hi = 0xFFFFFFFFull;  // the largest tau with count(key >= tau) >= c
  while (lo < hi) {
    const uint32_t mid = static_cast<uint32_t>((lo + hi + 1) >> 1);
    if (block_count(r, sh, [mid](uint32_t k) { return k >= mid; }) >= c) lo = mid;
    else hi = mid - 1;
  }
  Cut cut;
  cut.tau = static_cast<uint32_t>(lo);
  cut.none = false;
  const uint32_t tau = cut.tau;
  cut.t = c - block_count(r, sh, [tau](uint32_t k) { return k > tau; });
  return cut;
}

// Gathers the logits between two cuts (in `hi`'s prefix, not in `lo`'s) into sh.key / sh.id, sorts
// them by (key descending, id ascending), fills sh.prob, and returns how many there are.
__device__ int load_band(const RowView& r, TruncShared& sh, const Cut& lo, const Cut& hi, float temperature, double mx) {
  // ties before this warp's segment, for each cut's tau
  int ties_hi = 0, ties_lo = 0;
  for (int i = r.seg0 + r.lane; i < r.seg1; i += 32) {
    const uint32_t k = order_key(r.row[i]);
    ties_hi += k == hi.tau ? 1 : 0;
    ties_lo += (!lo.none && k == lo.tau) ? 1 : 0;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ties_hi += __shfl_xor_sync(0xffffffffu, ties_hi, o);
    ties_lo += __shfl_xor_sync(0xffffffffu, ties_lo, o);
  }
  __syncthreads();
  if (r.lane == 0) {
    sh.cnt[r.warp] = ties_hi;
    sh.cnt2[r.warp] = ties_lo;
  }
  if (threadIdx.x == 0) sh.fill = 0;
  __syncthreads();
  int base_hi = 0, base_lo = 0;
#pragma unroll 1
  for (int w = 0; w < r.warp; ++w) {
    base_hi += sh.cnt[w];
    base_lo += sh.cnt2[w];
  }
  const uint32_t lt = (1u << r.lane) - 1u;
  for (int i0 = r.seg0; i0 < r.seg1; i0 += 32) {
    const int i = i0 + r.lane;
    const bool in = i < r.seg1;
    const uint32_t k = in ? order_key(r.row[i]) : 0u;
    const bool tie_hi = in && k == hi.tau, tie_lo = in && !lo.none && k == lo.tau;
    const uint32_t bal_hi = __ballot_sync(0xffffffffu, tie_hi), bal_lo = __ballot_sync(0xffffffffu, tie_lo);
    const bool in_hi = in && (k > hi.tau || (tie_hi && base_hi + __popc(bal_hi & lt) < hi.t));
    const bool in_lo = in && !lo.none && (k > lo.tau || (tie_lo && base_lo + __popc(bal_lo & lt) < lo.t));
    base_hi += __popc(bal_hi);
    base_lo += __popc(bal_lo);
    if (in_hi && !in_lo) {
      const int at = atomicAdd(&sh.fill, 1);
      if (at < kBand) {
        sh.key[at] = k;
        sh.id[at] = i;
      }
    }
  }
  __syncthreads();
  const int n = min(sh.fill, kBand);
  for (int i = threadIdx.x; i < kBand; i += kSampleThreads)
    if (i >= n) {
      sh.key[i] = 0u;  // below every real key's place: (smallest key, largest id) sorts last
      sh.id[i] = 0x7fffffff;
    }
  __syncthreads();
  // bitonic sort, "a before b" = key larger, or equal key and id smaller
  for (int size = 2; size <= kBand; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = threadIdx.x; t < kBand / 2; t += kSampleThreads) {
        const int a = 2 * t - (t & (stride - 1)), b = a + stride;
        const bool up = (a & size) == 0;  // this run is sorted "before first"
        const uint32_t ka = sh.key[a], kb = sh.key[b];
        const int ia = sh.id[a], ib = sh.id[b];
        const bool a_first = ka > kb || (ka == kb && ia < ib);
        if (a_first != up) {
          sh.key[a] = kb;
          sh.key[b] = ka;
          sh.id[a] = ib;
          sh.id[b] = ia;
        }
      }
      __syncthreads();
    }
  }
  // exp(logit / T - max / T): the quotient in float32, the rest in float64 (engine/src/sampler.cpp:86-87)
  for (int i = threadIdx.x; i < n; i += kSampleThreads) sh.prob[i] = exp(static_cast<double>(r.row[sh.id[i]] / temperature) - mx);
  __syncthreads();
  return n;
}

__global__ void __launch_bounds__(kSampleThreads)
sample_truncated_rows_kernel(const float* __restrict__ logits, int V, const rb200_sampling_params* __restrict__ params,
                             int* __restrict__ token_out, double* __restrict__ logprob_out) {
  pdl_trigger();
  pdl_wait();
  const rb200_sampling_params p = params[blockIdx.x];
  const bool truncated = p.temperature > 0.0f && !((p.top_k <= 0 || p.top_k >= V) && p.top_p >= 1.0f);
  if (!truncated) return;  // sample_rows_kernel takes this row
  __shared__ TruncShared sh;
  RowView r;
  r.row = logits + static_cast<long long>(blockIdx.x) * V;
  r.V = V;
  r.lane = threadIdx.x & 31;
  r.warp = threadIdx.x >> 5;
  const int seg = (V + kSampleWarps * 32 - 1) / (kSampleWarps * 32) * 32;
  r.seg0 = min(V, r.warp * seg);
  r.seg1 = min(V, r.seg0 + seg);
  const float T = p.temperature;
  const int k = (p.top_k > 0 && p.top_k < V) ? p.top_k : V;

  // the largest logit (the first candidate) and the float64 exponent offset
  float best = -INFINITY;
  for (int i = r.seg0 + r.lane; i < r.seg1; i += 32) best = fmaxf(best, r.row[i]);
  best = warp_max(best);
  if (r.lane == 0) sh.fmax[r.warp] = best;
  __syncthreads();
  best = sh.fmax[0];
#pragma unroll 1
  for (int w = 1; w < kSampleWarps; ++w) best = fmaxf(best, sh.fmax[w]);
  const double mx = static_cast<double>(best / T);

  // one band is kept in shared memory between the phases when the whole walk stays inside it
  const int n_bands_k = (k + kBand - 1) / kBand;
  Cut lo_cut, hi_cut;
  int band_in_smem = -1, band_n = 0;
  auto band = [&](int b, int limit) {  // ranks [b kBand, min((b + 1) kBand, limit))
    if (b == band_in_smem) return band_n;
    if (b == 0) lo_cut.none = true;
    else if (band_in_smem == b - 1) lo_cut = hi_cut;
    else lo_cut = find_cut(r, sh, b * kBand);
    hi_cut = find_cut(r, sh, min((b + 1) * kBand, limit));
    band_n = load_band(r, sh, lo_cut, hi_cut, T, mx);
    band_in_smem = b;
    return band_n;
  };

  // ---- the sum of the candidates' probabilities ----
  double total = 0.0;
  if (k == V) {
    double part = 0.0;
    for (int i = r.seg0 + r.lane; i < r.seg1; i += 32) part += exp(static_cast<double>(r.row[i] / T) - mx);
    part = warp_sum_f64(part);
    __syncthreads();
    if (r.lane == 0) sh.dsum[r.warp] = part;
    __syncthreads();
#pragma unroll 1
    for (int w = 0; w < kSampleWarps; ++w) total += sh.dsum[w];
  } else {
    for (int b = 0; b < n_bands_k; ++b) {
      const int n = band(b, k);
      if (threadIdx.x == 0) {
        double acc = b == 0 ? 0.0 : sh.carry;
        for (int i = 0; i < n; ++i) acc += sh.prob[i];  // in sorted order, like the host's loop
        sh.carry = acc;
      }
      __syncthreads();
    }
    total = sh.carry;
    __syncthreads();
  }

  // ---- the nucleus: the shortest prefix whose probability reaches top_p ----
  int keep = k;
  double kept = total;
  if (p.top_p < 1.0f) {
    const double top_p = static_cast<double>(p.top_p);
    if (threadIdx.x == 0) {
      sh.carry = 0.0;   // cum: the host's running sum of prob / total
      sh.carry2 = 0.0;  // the kept candidates' probability so far
    }
    __syncthreads();
    for (int b = 0; b < n_bands_k; ++b) {
      const int n = band(b, k);
      if (threadIdx.x == 0) {
        double cum = sh.carry, run = sh.carry2;
        int hit = -1;
        for (int i = 0; i < n; ++i) {
          cum += sh.prob[i] / total;
          run += sh.prob[i];
          if (cum >= top_p) {
            hit = i;
            break;
          }
        }
        sh.carry = cum;
        sh.carry2 = run;
        sh.flag = hit;
      }
      __syncthreads();
      const int hit = sh.flag;
      kept = sh.carry2;  // if no prefix reaches top_p (rounding), every candidate stays and this is their sum
      __syncthreads();
      if (hit >= 0) {
        keep = b * kBand + hit + 1;
        break;
      }
    }
  }

  // ---- the walk ----
  const int n_bands_keep = (keep + kBand - 1) / kBand;
  int token = -1;
  if (threadIdx.x == 0) sh.carry = uniform01(p.seed, p.index) * kept;
  __syncthreads();
  for (int b = 0; b < n_bands_keep && token < 0; ++b) {
    const int n = min(band(b, k), keep - b * kBand);
    if (threadIdx.x == 0) {
      double rr = sh.carry;
      int tok = -1;
      for (int i = 0; i < n; ++i) {
        rr -= sh.prob[i];
        if (rr < 0) {
          tok = sh.id[i];
          break;
        }
      }
      if (tok < 0 && b + 1 == n_bands_keep) tok = sh.id[n - 1];  // the last kept candidate (engine/src/sampler.cpp:104)
      sh.carry = rr;
      sh.token = tok;
    }
    __syncthreads();
    token = sh.token;
    __syncthreads();
  }
  if (threadIdx.x == 0) token_out[blockIdx.x] = token;

  // ---- log softmax(logits / T)[token] over the whole vocabulary, float64 (engine/src/sampler.cpp:24-31) ----
  if (logprob_out != nullptr) {
    const double t = static_cast<double>(T), dmx = static_cast<double>(best);
    double part = 0.0;
    for (int i = r.seg0 + r.lane; i < r.seg1; i += 32) part += exp((static_cast<double>(r.row[i]) - dmx) / t);
    part = warp_sum_f64(part);
    __syncthreads();
    if (r.lane == 0) sh.dsum[r.warp] = part;
    __syncthreads();
    if (threadIdx.x == 0) {
      double sum = 0.0;
      for (int w = 0; w < kSampleWarps; ++w) sum += sh.dsum[w];
      logprob_out[blockIdx.x] = (static_cast<double>(r.row[token]) - dmx) / t - log(sum);
    }
  }
}

}  // namespace

bool sampling_truncated(const rb200_sampling_params& p, int V) {
  return p.temperature > 0.0f && !((p.top_k <= 0 || p.top_k >= V) && p.top_p >= 1.0f);
}

void launch_sample_rows(const float* logits, int R, int V, const rb200_sampling_params* params, int* token_out,
                        double* logprob_out, cudaStream_t st, bool any_truncated) {
  if (R == 0) return;
  count_launch();
  launch_pdl(sample_rows_kernel, dim3(R), dim3(kSampleThreads), 0, st, logits, V, params, token_out, logprob_out);
  if (any_truncated) {  // its CTAs return at once on rows the kernel above has taken, and the other way round
    count_launch();
    launch_pdl(sample_truncated_rows_kernel, dim3(R), dim3(kSampleThreads), 0, st, logits, V, params, token_out, logprob_out);
  }
}

}  // namespace rb200

using namespace rb200;

extern "C" int rb200_sample_rows(const float* logits, int R, int V, const rb200_sampling_params* params, int32_t* token_out,
                                 double* logprob_out, void* stream) {
  return guarded([&] {
    RB_REQUIRE(R >= 0 && V > 0 && logits && params && token_out, "sample_rows: bad arguments");
    launch_sample_rows(logits, R, V, params, token_out, logprob_out, as_stream(stream), true);
    RB_CUDA(cudaGetLastError());
    return 0;
  });
}
