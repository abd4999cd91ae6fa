// Shared by every translation unit of librelay_b200: the per-thread error slot behind
// rb200_last_error(), CUDA call checking, and the sm_100a device primitives the attention
// and GEMM kernels are built from (16-byte async copies into swizzled shared memory,
// ldmatrix, the m16n8k16 fp16 tensor-core instruction, packed conversions).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>

#include "relay_b200.h"

namespace rb200 {

// ---- errors -------------------------------------------------------------------------

struct Error : std::runtime_error {
  int kind;
  Error(int k, const std::string& what) : std::runtime_error(what), kind(k) {}
};

void set_last_error(int kind, const std::string& what);

// Runs f, turning exceptions into -1 + rb200_last_error() (the reference's C API
// convention, engine/src/c_api.cpp:31-46).
template <class F>
int guarded(F&& f) {
  try {
    return f();
  } catch (const Error& e) {
    set_last_error(e.kind, e.what());
  } catch (const std::exception& e) {
    set_last_error(RB200_ERR_RUNTIME, e.what());
  }
  return -1;
}

[[noreturn]] inline void fail(int kind, const std::string& what) { throw Error(kind, what); }

#define RB_CUDA(x)                                                                                   \
  do {                                                                                               \
    cudaError_t err_ = (x);                                                                          \
    if (err_ != cudaSuccess)                                                                         \
      ::rb200::fail(RB200_ERR_RUNTIME, std::string("CUDA error: ") + cudaGetErrorString(err_) + " at " + \
                                           __FILE__ + ":" + std::to_string(__LINE__));              \
  } while (0)

#define RB_REQUIRE(cond, msg)                                          \
  do {                                                                 \
    if (!(cond)) ::rb200::fail(RB200_ERR_INVALID_ARGUMENT, (msg));     \
  } while (0)

inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

inline int div_up(long long a, long long b) { return static_cast<int>((a + b - 1) / b); }
inline int round_up(int a, int b) { return (a + b - 1) / b * b; }

// Kernels launched by this library in this process (each launch_* wrapper counts its own).
std::atomic<uint64_t>& launch_counter();
inline void count_launch(int n = 1) { launch_counter().fetch_add(static_cast<uint64_t>(n), std::memory_order_relaxed); }

// Number of SMs of the current device (148 on B200), cached per device.
int sm_count();

// A kernel attribute (cudaFuncSetAttribute) belongs to the device that is current when it is
// set, so a process that drives several GPUs has to set it once on each. One of these, as a
// function-local static next to the launch, remembers the devices already done; first() is
// true once per device (two threads racing on it both set the attribute, which is harmless:
// the call is idempotent and only ever raises the limit).
struct PerDeviceOnce {
  static constexpr int kMaxDevices = 64;
  std::atomic<bool> done[kMaxDevices] = {};
  bool first() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
      cudaGetLastError();
      return true;  // unknown device: set the attribute every time
    }
    return !done[dev].exchange(true, std::memory_order_acq_rel);
  }
};

// ---- device primitives ----------------------------------------------------------------

#ifdef __CUDACC__

// Programmatic dependent launch. Every kernel of the forward pass starts with pdl_trigger()
// (the next kernel in the stream may be scheduled once all CTAs of this one have started) and
// pdl_wait() (nothing this kernel reads or writes in global memory is touched before the
// kernel ahead of it has completed and its writes are visible), and is launched through
// launch_pdl(): its launch latency and block scheduling then overlap the tail of its
// predecessor. Both instructions do nothing in a kernel launched the ordinary way.
//
// What a kernel may read BEFORE pdl_wait(): the weights, and the batch metadata (positions,
// sequence ids, block tables, row lists). The metadata reaches the device by a copy that precedes
// the first kernel of a pass, or is updated by session_advance_kernel / session_finish_kernel, and
// session_advance_kernel does not call pdl_trigger(): the kernel behind it, and with it every
// later kernel of the step, starts only once the update is complete. Activations and K/V pages
// are written by kernels of the same pass and are read after the wait only.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  RB_CUDA(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte global -> shared asynchronous copy (LDGSTS), L2-only caching: KV pages and
// weights are streamed once, so they should not displace L1.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}
// The same, copying `bytes` (0 or 16) and zero-filling the rest.
__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}

// D(16x8, fp32) += A(16x16, fp16, row) * B(16x8, fp16, col).
__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Index (in 16-byte chunks) of chunk `chunk` of row `row` in a [rows][CH chunks] shared
// tile, XOR-swizzled so that the 8 rows an ldmatrix phase touches at one chunk column fall
// into 8 different 16-byte bank groups. CH = row bytes / 16: 2, 4 or >= 8 (a multiple of 8).
template <int CH>
__device__ __forceinline__ int swz(int row, int chunk) {
  if constexpr (CH >= 8) return row * CH + (chunk ^ (row & 7));
  else if constexpr (CH == 4) return row * CH + (chunk ^ ((row >> 1) & 3));
  else if constexpr (CH == 2) return row * CH + (chunk ^ ((row >> 2) & 1));
  else return row * CH + chunk;
}

// (largest value, lowest index holding it) over this thread's share of row[0..V): elements
// t, t + n, t + 2n, ... for thread t of n. Eight loads are issued before any of them is compared,
// so the loop runs at memory throughput rather than one round trip per element.
__device__ __forceinline__ void strided_argmax(const float* __restrict__ row, int V, int t, int n, float& best, int& bi) {
  best = -INFINITY;
  bi = 0x7fffffff;
  constexpr int U = 8;
  for (int i0 = t; i0 < V; i0 += U * n) {
    float v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) v[u] = i0 + u * n < V ? row[i0 + u * n] : -INFINITY;
#pragma unroll
    for (int u = 0; u < U; ++u)  // ascending index: a later equal value never replaces an earlier one
      if (v[u] > best) {
        best = v[u];
        bi = i0 + u * n;
      }
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

#endif  // __CUDACC__

}  // namespace rb200
