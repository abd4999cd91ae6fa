// The prefill -> decode KV hop over NVLink: one layer's blocks are gathered into a
// contiguous [K of each block][V of each block] buffer and handed to ncclSend; the
// receiver's ncclRecv lands in its staging buffer and a scatter kernel writes the pages
// into its own block ids. This replaces, for GPU-to-GPU transfers inside one box, the
// host-staged payload path of the reference's transfer engine (sender
// engine/src/kv_transfer.cpp:107-128 -> read_kv_layer -> socket; receiver :289-297 ->
// write_kv_layer); the framing, ordering and abort messages stay on the host connection,
// which also fixes the order in which the two sides post their send and receive.
//
// NCCL is loaded at run time (dlopen) so that the library has no link-time dependency on
// it and a process that already loaded NCCL (for example through torch) shares that copy.
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <thread>

#include "backend.h"

namespace rb200 {

namespace {

struct NcclApi {
  void* lib = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
  ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

NcclApi& api() {
  static NcclApi a;
  static std::once_flag once;
  std::call_once(once, [] {
    for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
      a.lib = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
      if (a.lib) break;
    }
    if (!a.lib) return;
    auto sym = [&](const char* n) { return dlsym(a.lib, n); };
    a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(sym("ncclGetUniqueId"));
    a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(sym("ncclCommInitRank"));
    a.CommInitRankConfig = reinterpret_cast<decltype(a.CommInitRankConfig)>(sym("ncclCommInitRankConfig"));
    a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(sym("ncclCommDestroy"));
    a.CommAbort = reinterpret_cast<decltype(a.CommAbort)>(sym("ncclCommAbort"));
    a.CommGetAsyncError = reinterpret_cast<decltype(a.CommGetAsyncError)>(sym("ncclCommGetAsyncError"));
    a.Send = reinterpret_cast<decltype(a.Send)>(sym("ncclSend"));
    a.Recv = reinterpret_cast<decltype(a.Recv)>(sym("ncclRecv"));
    a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(sym("ncclGetErrorString"));
  });
  if (!a.lib || !a.GetUniqueId || !a.CommInitRank || !a.Send || !a.Recv || !a.CommDestroy || !a.CommAbort)
    fail(RB200_ERR_RUNTIME, "NCCL is not available (libnccl.so.2 could not be loaded)");
  return a;
}

void nccl_check(ncclResult_t r, const char* what) {
  if (r != ncclSuccess && r != ncclInProgress) {
    const NcclApi& a = api();
    fail(RB200_ERR_RUNTIME, std::string("NCCL error in ") + what + ": " + (a.GetErrorString ? a.GetErrorString(r) : "?"));
  }
}

}  // namespace

static ncclComm_t comm_of(const NcclState& s) { return static_cast<ncclComm_t>(s.comm); }

constexpr int kInitTimeoutMs = 120000;  // communicator set-up
constexpr int kCallTimeoutMs = 60000;   // a send / receive call that has to connect the two ranks first

// The communicator is non-blocking: a call may return ncclInProgress while NCCL still works on
// it in the background (rendezvous, the first connection between two ranks). The next call on the
// communicator has to wait for that; this polls with a host deadline and aborts the communicator
// when it runs out, so no call of this file can block for ever on a peer that never shows up.
static void wait_ready(ncclComm_t comm, ncclResult_t r, int timeout_ms, const char* what) {
  const NcclApi& a = api();
  const auto start = std::chrono::steady_clock::now();
  const auto deadline = start + std::chrono::milliseconds(timeout_ms);
  while (r == ncclInProgress) {
    if (!a.CommGetAsyncError) return;  // a library too old to poll: it is blocking anyway
    if (a.CommGetAsyncError(comm, &r) != ncclSuccess) break;
    if (r != ncclInProgress) break;
    const auto now = std::chrono::steady_clock::now();
    if (now > deadline) {
      a.CommAbort(comm);
      fail(RB200_ERR_RUNTIME, std::string(what) + ": timed out; communicator aborted");
    }
    // an enqueue completes within microseconds: spin for the first millisecond, then back off
    if (now - start > std::chrono::milliseconds(1)) std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
  if (r != ncclSuccess) {
    a.CommAbort(comm);
    fail(RB200_ERR_RUNTIME, std::string("NCCL error in ") + what + ": " + (a.GetErrorString ? a.GetErrorString(r) : "?"));
  }
}

constexpr int kDefaultSyncTimeoutMs = 60000;  // kv_hop_sync(timeout_ms <= 0)
constexpr int kFinalizeTimeoutMs = 10000;     // finalize / destructor

void Backend::nccl_init(const void* id, int nranks, int rank) {
  set_device();
  RB_REQUIRE(nranks >= 2 && rank >= 0 && rank < nranks, "nccl_init: bad rank");
  RB_REQUIRE(!nccl_, "nccl_init: already initialised");
  NcclApi& a = api();
  ncclUniqueId uid;
  static_assert(sizeof(uid) == RB200_NCCL_ID_BYTES, "NCCL unique id size");
  std::memcpy(&uid, id, sizeof(uid));
  auto st = std::make_unique<NcclState>();
  ncclComm_t comm = nullptr;
  // RB200_NCCL_BLOCKING=1: a blocking communicator (each send / receive call then costs less host
  // time, but set-up and the first connection to a peer wait without a deadline).
  static const bool blocking = [] {
    const char* e = std::getenv("RB200_NCCL_BLOCKING");
    return e && e[0] == '1';
  }();
  if (!blocking && a.CommInitRankConfig && a.CommGetAsyncError) {
    ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
    cfg.blocking = 0;
    const ncclResult_t r = a.CommInitRankConfig(&comm, nranks, uid, rank, &cfg);
    if (r != ncclSuccess && r != ncclInProgress) nccl_check(r, "ncclCommInitRankConfig");
    RB_REQUIRE(comm != nullptr, "nccl_init: no communicator");
    wait_ready(comm, ncclInProgress, kInitTimeoutMs, "ncclCommInitRankConfig");
  } else {
    nccl_check(a.CommInitRank(&comm, nranks, uid, rank), "ncclCommInitRank");
  }
  st->comm = comm;
  st->nranks = nranks;
  st->rank = rank;
  nccl_ = std::move(st);
}

void Backend::nccl_finalize() {
  if (!nccl_) return;
  set_device();
  // A send or receive the peer never matched would keep the copy stream busy for ever: wait with
  // the deadline of kv_hop_sync, which aborts the communicator when it runs out.
  kv_hop_sync(kFinalizeTimeoutMs);
  if (!nccl_) return;  // aborted
  ncclComm_t comm = comm_of(*nccl_);
  nccl_.reset();
  const ncclResult_t r = api().CommDestroy(comm);
  if (r != ncclSuccess && r != ncclInProgress) nccl_check(r, "ncclCommDestroy");
}

void Backend::nccl_finalize_noexcept() noexcept {
  try {
    nccl_finalize();
  } catch (...) {
    nccl_.reset();
  }
}

void Backend::send_kv_layer(int peer, int layer, const int32_t* blocks, int n) {
  set_device();
  RB_REQUIRE(nccl_ != nullptr, "send_kv_layer: call nccl_init first");
  RB_REQUIRE(peer >= 0 && peer < nccl_->nranks && peer != nccl_->rank, "send_kv_layer: bad peer");
  check_layer(layer);
  check_blocks(blocks, n);
  if (n == 0) return;
  std::lock_guard<std::mutex> lock(copy_mu_);
  const size_t bb = kv_block_bytes();
  ensure_kv_staging(n);
  const int* ids = static_cast<const int*>(staging_ids(blocks, n));
  // The gather must see this layer's appends of the latest forward pass: order the copy
  // stream behind the layer's event on the device instead of blocking the host.
  RB_CUDA(cudaStreamWaitEvent(copy_stream_, layer_done_[layer], 0));
  const size_t off = static_cast<size_t>(layer) * layer_elems();
  launch_kv_gather(kc_.as<__half>() + off, vc_.as<__half>() + off, ids, n, bb, kv_staging_.p, copy_stream_);
  RB_CUDA(cudaGetLastError());
  try {
    wait_ready(comm_of(*nccl_), api().Send(kv_staging_.p, 2 * static_cast<size_t>(n) * bb, ncclInt8, peer, comm_of(*nccl_), copy_stream_),
               kCallTimeoutMs, "ncclSend");
  } catch (...) {
    nccl_.reset();  // wait_ready aborted the communicator
    throw;
  }
}

void Backend::recv_kv_layer(int peer, int layer, const int32_t* blocks, int n) {
  set_device();
  RB_REQUIRE(nccl_ != nullptr, "recv_kv_layer: call nccl_init first");
  RB_REQUIRE(peer >= 0 && peer < nccl_->nranks && peer != nccl_->rank, "recv_kv_layer: bad peer");
  check_layer(layer);
  check_blocks(blocks, n);
  if (n == 0) return;
  std::lock_guard<std::mutex> lock(copy_mu_);
  const size_t bb = kv_block_bytes();
  ensure_kv_staging(n);
  const int* ids = static_cast<const int*>(staging_ids(blocks, n));
  try {
    wait_ready(comm_of(*nccl_), api().Recv(kv_staging_.p, 2 * static_cast<size_t>(n) * bb, ncclInt8, peer, comm_of(*nccl_), copy_stream_),
               kCallTimeoutMs, "ncclRecv");
  } catch (...) {
    nccl_.reset();
    throw;
  }
  const size_t off = static_cast<size_t>(layer) * layer_elems();
  launch_kv_scatter(kc_.as<__half>() + off, vc_.as<__half>() + off, ids, n, bb, kv_staging_.p, copy_stream_);
  RB_CUDA(cudaGetLastError());
}

void Backend::kv_hop_sync(int timeout_ms) {
  set_device();
  if (timeout_ms <= 0) timeout_ms = kDefaultSyncTimeoutMs;  // never wait without a limit
  const auto started = std::chrono::steady_clock::now();
  const auto deadline = started + std::chrono::milliseconds(timeout_ms);
  for (;;) {
    const cudaError_t q = cudaStreamQuery(copy_stream_);
    if (q == cudaSuccess) {
      std::lock_guard<std::mutex> lock(copy_mu_);
      if (links_idle()) return;
    } else if (q != cudaErrorNotReady) {
      RB_CUDA(q);
    }
    if (nccl_ && api().CommGetAsyncError) {
      ncclResult_t async = ncclSuccess;
      api().CommGetAsyncError(comm_of(*nccl_), &async);
      if (async != ncclSuccess && async != ncclInProgress) {
        api().CommAbort(comm_of(*nccl_));
        nccl_.reset();
        fail(RB200_ERR_RUNTIME, "NCCL reported an asynchronous error; communicator aborted");
      }
    }
    if (std::chrono::steady_clock::now() > deadline) {
      if (nccl_ && cudaStreamQuery(copy_stream_) == cudaErrorNotReady) {
        api().CommAbort(comm_of(*nccl_));
        nccl_.reset();
      }
      {
        std::lock_guard<std::mutex> lock(copy_mu_);
        links_release();
      }
      cudaGetLastError();
      fail(RB200_ERR_RUNTIME, "kv_hop_sync: timed out; communicator aborted");
    }
    // a hop of a prompt or two ends within a millisecond or two: poll without sleeping that long
    if (std::chrono::steady_clock::now() - started > std::chrono::milliseconds(2)) std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}

}  // namespace rb200

extern "C" int rb200_nccl_unique_id(void* id) {
  return rb200::guarded([&] {
    RB_REQUIRE(id != nullptr, "nccl_unique_id: null argument");
    ncclUniqueId uid;
    rb200::nccl_check(rb200::api().GetUniqueId(&uid), "ncclGetUniqueId");
    std::memcpy(id, &uid, sizeof(uid));
    return 0;
  });
}
