// K/V links: the prefill -> decode hop between two GPUs of one box without a library kernel in
// the way. It carries the same payload as the NCCL hop of kv_hop.cu and the Layer frames of
// relay's transfer engine (engine/include/relay/kv_transfer.h:14-18: all K blocks of a layer,
// then all V blocks, request-relative order; sender engine/src/kv_transfer.cpp:107-128,
// receiver :269-301), but moves it with one kernel of plain peer stores (or, optionally, the
// copy engines) and orders it with two counters, so that no per-operation library latency is paid.
//
// Each end of a link owns one device region: a ring of `n_slots` landing slots and, per slot,
// two 32-bit counters. The ends exchange CUDA IPC handles of their regions out of band (the host
// connection that already carries relay's Hello frame) and map each other's region.
//
//   sender, message k (slot s = k % n_slots):
//                        wait until its own ack[s] says the message that last used s was scattered;
//                        gather the pages straight into the PEER's slot (one kernel whose 16-byte
//                        stores cross NVLink: the pages are read once and nothing is staged);
//                        store k + 1 into the peer's arrived[s] (one-thread kernel);
//   receiver, message k: stream-wait until its own arrived[s] reaches k + 1;
//                        scatter its slot into the pages of its own block ids;
//                        store k + 1 into the peer's ack[s].
// Consecutive messages alternate between two streams on each end; the per-slot counters keep
// that safe whatever stream a message is on. RB200_KV_LINK=ce gathers into the sender's own slot
// and lets a copy engine move the slot instead (no SM busy during the transfer): a copy-engine
// peer copy has a fixed cost of about 20 us on this hardware (back-to-back copies of 8 / 32 /
// 256 MB run at 270 / 515 / 734 GB/s) that neither more streams (four measured no faster than
// two) nor the gather of the next message hide, so that path measured 360 GB/s layer by layer
// and 500 GB/s with 134 MB messages against 408 and 673 GB/s for the peer stores, at the same
// cost to a prefill running beside it (0.4 ms per 2048-token prompt either way).
//
// The waits are stream memory operations (cuStreamWaitValue32) on the waiting GPU's own memory:
// no kernel spins, and a wait the peer never satisfies is released from the host when
// rb200_kv_hop_sync's deadline runs out (the link is then marked broken). Only plain stores from
// this library's own kernels and copy-engine copies touch the peer's memory; no TMA and no
// library kernel ever sees a peer pointer. Messages pair up by order on the link, which
// the host connection's ordered frames already guarantee.
#include <cuda.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "backend.h"

namespace rb200 {

namespace {

constexpr uint32_t kLinkMagic = 0x4b4c3230u;  // "02LK"
constexpr int kMaxSlots = 64;
constexpr size_t kControlBytes = 512;         // arrived[64] @0, ack[64] @256; the ring starts behind
constexpr int kMaxIds = 480;                  // block ids handed to a kernel by value (1.9 KB of parameters)

struct LinkHandle {  // what crosses the host connection: RB200_KV_LINK_HANDLE_BYTES
  uint32_t magic;
  int32_t n_slots;
  uint64_t slot_bytes;
  cudaIpcMemHandle_t mem;
  unsigned char pad[RB200_KV_LINK_HANDLE_BYTES - 16 - sizeof(cudaIpcMemHandle_t)];
};
static_assert(sizeof(LinkHandle) == RB200_KV_LINK_HANDLE_BYTES, "link handle size");

struct IdList {
  int n;
  int ids[kMaxIds];
};

// Pages of one or more consecutive layers into / out of a contiguous slot, per layer
// [K of each block][V of each block]; the block ids ride in the kernel's parameters, so no upload
// precedes the launch. k and v point at the first layer of the message; grid = (blocks, 2,
// layers x parts), `parts` CTAs sharing one block.
// A CTA's share of one block: four 16-byte loads in flight per thread before the first store.
__device__ __forceinline__ void copy_share(const uint4* __restrict__ src, uint4* __restrict__ dst, long long n, int part, int parts) {
  const long long stride = static_cast<long long>(parts) * blockDim.x;
  long long e = static_cast<long long>(part) * blockDim.x + threadIdx.x;
  for (; e + 3 * stride < n; e += 4 * stride) {
    const uint4 a = src[e], b = src[e + stride], c = src[e + 2 * stride], d = src[e + 3 * stride];
    dst[e] = a;
    dst[e + stride] = b;
    dst[e + 2 * stride] = c;
    dst[e + 3 * stride] = d;
  }
  for (; e < n; e += stride) dst[e] = src[e];
}

__global__ void link_gather_kernel(const uint4* __restrict__ k, const uint4* __restrict__ v, const __grid_constant__ IdList ids,
                                   long long block_vec, long long layer_vec, int parts, uint4* __restrict__ out) {
  const int i = blockIdx.x, which = blockIdx.y, lz = blockIdx.z / parts, part = blockIdx.z % parts;
  const uint4* src = (which ? v : k) + lz * layer_vec + static_cast<long long>(ids.ids[i]) * block_vec;
  uint4* dst = out + ((static_cast<long long>(lz) * 2 + which) * ids.n + i) * block_vec;
  copy_share(src, dst, block_vec, part, parts);
}

__global__ void link_scatter_kernel(uint4* __restrict__ k, uint4* __restrict__ v, const __grid_constant__ IdList ids,
                                    long long block_vec, long long layer_vec, int parts, const uint4* __restrict__ in) {
  const int i = blockIdx.x, which = blockIdx.y, lz = blockIdx.z / parts, part = blockIdx.z % parts;
  uint4* dst = (which ? v : k) + lz * layer_vec + static_cast<long long>(ids.ids[i]) * block_vec;
  const uint4* src = in + ((static_cast<long long>(lz) * 2 + which) * ids.n + i) * block_vec;
  copy_share(src, dst, block_vec, part, parts);
}

// One store of `value` to a counter in the peer's region, behind everything this stream has
// written there (the copy ahead of it has completed in stream order; the fence orders this
// thread's store behind it system-wide).
__global__ void link_signal_kernel(uint32_t* counter, uint32_t value) {
  __threadfence_system();
  *reinterpret_cast<volatile uint32_t*>(counter) = value;
  __threadfence_system();
}

using WaitValueFn = CUresult (*)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);

WaitValueFn wait_value_fn() {
  static WaitValueFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuStreamWaitValue32", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<WaitValueFn>(p);
    else
      cudaGetLastError();
  });
  if (!fn) fail(RB200_ERR_RUNTIME, "cuStreamWaitValue32 is not available from this driver");
  return fn;
}

void stream_wait_geq(cudaStream_t st, uint32_t* addr, uint32_t value) {
  const CUresult r = wait_value_fn()(st, reinterpret_cast<CUdeviceptr>(addr), value, CU_STREAM_WAIT_VALUE_GEQ);
  if (r != CUDA_SUCCESS) fail(RB200_ERR_RUNTIME, "cuStreamWaitValue32 failed with code " + std::to_string(static_cast<int>(r)));
}

uint32_t* arrived_of(void* region, const KvLink& l, uint32_t k) {
  return static_cast<uint32_t*>(region) + k % static_cast<uint32_t>(l.n_slots);
}
uint32_t* ack_of(void* region, const KvLink& l, uint32_t k) {
  return reinterpret_cast<uint32_t*>(static_cast<char*>(region) + 256) + k % static_cast<uint32_t>(l.n_slots);
}
char* slot_of(void* region, const KvLink& l, uint32_t k) {
  return static_cast<char*>(region) + kControlBytes + static_cast<size_t>(k % static_cast<uint32_t>(l.n_slots)) * l.slot_bytes;
}

// How `n_layers` layers of `n` blocks each travel: whole layers per message while a layer fits a
// slot (as many as the slot holds), else one layer as several messages of blocks. Both ends cut
// the same way, because they were created with the same ring.
struct LinkMsg {
  int layer, layers, b0, m;
};

std::vector<LinkMsg> link_messages(size_t slot_bytes, size_t block_bytes, int layer0, int n_layers, int n) {
  std::vector<LinkMsg> out;
  const size_t layer_bytes = 2 * static_cast<size_t>(n) * block_bytes;
  if (n <= kMaxIds && layer_bytes <= slot_bytes) {
    const int per = static_cast<int>(std::min<size_t>(slot_bytes / layer_bytes, 4096));
    for (int a = 0; a < n_layers; a += per) out.push_back({layer0 + a, std::min(per, n_layers - a), 0, n});
    return out;
  }
  const int per_msg = static_cast<int>(std::min<size_t>(kMaxIds, slot_bytes / (2 * block_bytes)));
  for (int a = 0; a < n_layers; ++a)
    for (int b0 = 0; b0 < n; b0 += per_msg) out.push_back({layer0 + a, 1, b0, std::min(per_msg, n - b0)});
  return out;
}

// CTAs sharing one block: each thread moves four 16-byte pieces where the message is large
// enough to fill the SMs that way, fewer where it is not.
int link_parts(long long block_vec, int n_blocks) {
  int parts = static_cast<int>(std::max<long long>(1, std::min<long long>(8, block_vec / 1024)));
  while (parts < 8 && static_cast<long long>(parts) * 2 * 256 <= block_vec && 2LL * n_blocks * parts < 2 * sm_count()) parts *= 2;
  return parts;
}

bool sm_copy() {  // false with RB200_KV_LINK=ce: gather into this end's slot, then a copy-engine peer copy
  static const bool on = [] {
    const char* e = std::getenv("RB200_KV_LINK");
    return !(e && std::string(e) == "ce");
  }();
  return on;
}

}  // namespace

cudaError_t KvLink::busy(bool gathers_only) const {
  cudaError_t worst = cudaSuccess;
  for (int i = 0; i < kStreams; ++i) {
    const cudaError_t q = gathers_only ? cudaEventQuery(gathered[i]) : cudaStreamQuery(streams[i]);
    if (q == cudaErrorNotReady) {
      if (worst == cudaSuccess) worst = q;
    } else if (q != cudaSuccess) {
      worst = q;
    }
  }
  return worst;
}

KvLink::~KvLink() {
  if (wedged) {  // a stream of this link never came back: nothing here may wait for the device
    region.p = nullptr;
    region.bytes = 0;
    return;
  }
  if (peer && peer_is_ipc) cudaIpcCloseMemHandle(peer);
  if (release_stream) cudaStreamDestroy(release_stream);
  for (cudaStream_t s : streams)
    if (s) cudaStreamDestroy(s);
  for (cudaEvent_t e : gathered)
    if (e) cudaEventDestroy(e);
}

KvLink& Backend::link_of(int link) {
  RB_REQUIRE(link >= 0 && link < static_cast<int>(links_.size()) && links_[link], "kv link: no such link");
  return *links_[link];
}

int Backend::kv_link_create(int n_slots, size_t slot_bytes, void* handle_out) {
  set_device();
  RB_REQUIRE(n_slots >= 1 && n_slots <= kMaxSlots && handle_out, "kv_link_create: bad arguments");
  const size_t bb = kv_block_bytes();
  RB_REQUIRE(slot_bytes >= 2 * bb && slot_bytes % 256 == 0, "kv_link_create: a slot holds at least one K and one V block and is a multiple of 256 bytes");
  auto l = std::make_unique<KvLink>();
  l->n_slots = n_slots;
  l->slot_bytes = slot_bytes;
  l->region = DeviceBuf(kControlBytes + static_cast<size_t>(n_slots) * slot_bytes);
  RB_CUDA(cudaMemset(l->region.p, 0, kControlBytes));
  for (cudaStream_t& s : l->streams) RB_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  RB_CUDA(cudaStreamCreateWithFlags(&l->release_stream, cudaStreamNonBlocking));
  l->release_words.ensure(kControlBytes);
  for (size_t i = 0; i < kControlBytes / 4; ++i) l->release_words.as<uint32_t>()[i] = 0x7fffffffu;  // satisfies every >= wait on this end
  for (cudaEvent_t& e : l->gathered) RB_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  LinkHandle h{};
  h.magic = kLinkMagic;
  h.n_slots = n_slots;
  h.slot_bytes = slot_bytes;
  RB_CUDA(cudaIpcGetMemHandle(&h.mem, l->region.p));
  std::memcpy(handle_out, &h, sizeof(h));
  wait_value_fn();  // fail now rather than at the first message
  std::lock_guard<std::mutex> lock(copy_mu_);
  links_.push_back(std::move(l));
  return static_cast<int>(links_.size()) - 1;
}

void Backend::kv_link_connect(int link, const void* peer_handle) {
  set_device();
  RB_REQUIRE(peer_handle != nullptr, "kv_link_connect: null handle");
  std::lock_guard<std::mutex> lock(copy_mu_);
  KvLink& l = link_of(link);
  RB_REQUIRE(l.peer == nullptr, "kv_link_connect: already connected");
  LinkHandle h;
  std::memcpy(&h, peer_handle, sizeof(h));
  RB_REQUIRE(h.magic == kLinkMagic, "kv_link_connect: not a link handle");
  RB_REQUIRE(h.n_slots == l.n_slots && h.slot_bytes == l.slot_bytes, "kv_link_connect: the two ends were created with different rings");
  void* p = nullptr;
  RB_CUDA(cudaIpcOpenMemHandle(&p, h.mem, cudaIpcMemLazyEnablePeerAccess));
  l.peer = p;
  l.peer_is_ipc = true;
}

// The two ends live in one process (an IPC handle cannot be opened by the process that made it):
// each end takes the other's region by its address. Backends on different devices get peer
// access to each other first.
void Backend::kv_link_connect_local(int link, Backend& other, int other_link) {
  RB_REQUIRE(&other != this, "kv_link_connect_local: a link joins two backends");
  if (other.device_ != device_) {
    for (int pass = 0; pass < 2; ++pass) {
      RB_CUDA(cudaSetDevice(pass == 0 ? device_ : other.device_));
      const cudaError_t e = cudaDeviceEnablePeerAccess(pass == 0 ? other.device_ : device_, 0);
      if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) RB_CUDA(e);
      cudaGetLastError();
    }
  }
  set_device();
  // lock the two backends in address order
  Backend* first = this < &other ? this : &other;
  Backend* second = this < &other ? &other : this;
  std::lock_guard<std::mutex> la(first->copy_mu_);
  std::lock_guard<std::mutex> lb(second->copy_mu_);
  KvLink& a = link_of(link);
  KvLink& b = other.link_of(other_link);
  RB_REQUIRE(a.peer == nullptr && b.peer == nullptr, "kv_link_connect_local: already connected");
  RB_REQUIRE(a.n_slots == b.n_slots && a.slot_bytes == b.slot_bytes, "kv_link_connect_local: the two ends were created with different rings");
  a.peer = b.region.p;
  b.peer = a.region.p;
}

void Backend::kv_link_close(int link) {
  set_device();
  std::lock_guard<std::mutex> lock(copy_mu_);
  KvLink& l = link_of(link);
  // The caller has synchronised the hop (rb200_kv_hop_sync) before closing; a link that is
  // still busy here is waiting for a peer that will not come.
  if (l.busy() == cudaErrorNotReady) links_release();
  cudaGetLastError();
  links_[link].reset();
}

void Backend::kv_link_send_layers(int link, int layer0, int n_layers, const int32_t* blocks, int n) {
  set_device();
  RB_REQUIRE(n_layers >= 1, "kv_link_send_layers: no layers");
  check_layer(layer0);
  check_layer(layer0 + n_layers - 1);
  check_blocks(blocks, n);
  if (n == 0) return;
  std::lock_guard<std::mutex> lock(copy_mu_);
  KvLink& l = link_of(link);
  RB_REQUIRE(l.peer != nullptr, "kv_link_send_layers: the link is not connected");
  if (l.broken) fail(RB200_ERR_RUNTIME, "kv link: broken by an earlier timeout");
  const size_t bb = kv_block_bytes();
  const long long vec = static_cast<long long>(bb / 16);
  const int parts = link_parts(vec, n);
  // The gather must see these layers' appends of the latest forward pass: a stream this call
  // uses waits for the event of the last layer of its message, unless that has completed already
  // (the layers of a pass complete in order).
  int waited_for[KvLink::kStreams];
  for (int& w : waited_for) w = -1;
  for (const LinkMsg& msg : link_messages(l.slot_bytes, bb, layer0, n_layers, n)) {
    const uint32_t k = l.sent++;
    cudaStream_t st = l.streams[k % KvLink::kStreams];
    const int last = msg.layer + msg.layers - 1;
    if (waited_for[k % KvLink::kStreams] < last) {
      const bool pending = cudaEventQuery(layer_done_[last]) != cudaSuccess;
      cudaGetLastError();
      if (pending) RB_CUDA(cudaStreamWaitEvent(st, layer_done_[last], 0));
      waited_for[k % KvLink::kStreams] = last;
    }
    if (k >= static_cast<uint32_t>(l.n_slots)) stream_wait_geq(st, ack_of(l.region.p, l, k), k - l.n_slots + 1);
    IdList ids;
    ids.n = msg.m;
    std::memcpy(ids.ids, blocks + msg.b0, static_cast<size_t>(msg.m) * 4);
    const size_t bytes = 2 * static_cast<size_t>(msg.m) * bb * msg.layers;
    const size_t off = static_cast<size_t>(msg.layer) * layer_elems();
    char* mine = slot_of(l.region.p, l, k);
    char* theirs = slot_of(l.peer, l, k);
    dim3 grid(msg.m, 2, static_cast<unsigned>(parts * msg.layers));
    // Folding the signal into the gather kernel (last CTA done stores the counter) measured slower:
    // every thread then pays a system-wide fence behind its peer stores.
    count_launch(2);
    link_gather_kernel<<<grid, 256, 0, st>>>(kc_.as<uint4>() + off / 8, vc_.as<uint4>() + off / 8, ids, vec,
                                             static_cast<long long>(layer_elems() / 8), parts,
                                             reinterpret_cast<uint4*>(sm_copy() ? theirs : mine));
    RB_CUDA(cudaEventRecord(l.gathered[k % KvLink::kStreams], st));  // from here on the message no longer reads the pages
    if (!sm_copy()) RB_CUDA(cudaMemcpyAsync(theirs, mine, bytes, cudaMemcpyDefault, st));  // peer copy, by address
    link_signal_kernel<<<1, 1, 0, st>>>(arrived_of(l.peer, l, k), k + 1);
    RB_CUDA(cudaGetLastError());
  }
}

void Backend::kv_link_recv_layers(int link, int layer0, int n_layers, const int32_t* blocks, int n) {
  set_device();
  RB_REQUIRE(n_layers >= 1, "kv_link_recv_layers: no layers");
  check_layer(layer0);
  check_layer(layer0 + n_layers - 1);
  check_blocks(blocks, n);
  if (n == 0) return;
  std::lock_guard<std::mutex> lock(copy_mu_);
  KvLink& l = link_of(link);
  RB_REQUIRE(l.peer != nullptr, "kv_link_recv_layers: the link is not connected");
  if (l.broken) fail(RB200_ERR_RUNTIME, "kv link: broken by an earlier timeout");
  const size_t bb = kv_block_bytes();
  const long long vec = static_cast<long long>(bb / 16);
  const int parts = link_parts(vec, n);
  for (const LinkMsg& msg : link_messages(l.slot_bytes, bb, layer0, n_layers, n)) {
    const uint32_t k = l.received++;
    cudaStream_t st = l.streams[k % KvLink::kStreams];
    stream_wait_geq(st, arrived_of(l.region.p, l, k), k + 1);
    IdList ids;
    ids.n = msg.m;
    std::memcpy(ids.ids, blocks + msg.b0, static_cast<size_t>(msg.m) * 4);
    const size_t off = static_cast<size_t>(msg.layer) * layer_elems();
    dim3 grid(msg.m, 2, static_cast<unsigned>(parts * msg.layers));
    count_launch(2);
    link_scatter_kernel<<<grid, 256, 0, st>>>(kc_.as<uint4>() + off / 8, vc_.as<uint4>() + off / 8, ids, vec,
                                              static_cast<long long>(layer_elems() / 8), parts,
                                              reinterpret_cast<const uint4*>(slot_of(l.region.p, l, k)));
    link_signal_kernel<<<1, 1, 0, st>>>(ack_of(l.peer, l, k), k + 1);
    RB_CUDA(cudaGetLastError());
  }
}

// Consumes the messages of n_layers layers of n blocks the peer has sent (or will send) without
// landing them anywhere: the receiver had no room for the request and drops the frame
// (engine/src/kv_transfer.cpp:284-288), but the ring must move on.
void Backend::kv_link_skip_layers(int link, int n_layers, int n) {
  set_device();
  RB_REQUIRE(n >= 0 && n_layers >= 1, "kv_link_skip_layers: bad counts");
  if (n == 0) return;
  std::lock_guard<std::mutex> lock(copy_mu_);
  KvLink& l = link_of(link);
  RB_REQUIRE(l.peer != nullptr, "kv_link_skip_layers: the link is not connected");
  if (l.broken) fail(RB200_ERR_RUNTIME, "kv link: broken by an earlier timeout");
  const size_t n_msgs = link_messages(l.slot_bytes, kv_block_bytes(), 0, n_layers, n).size();
  for (size_t i = 0; i < n_msgs; ++i) {
    const uint32_t k = l.received++;
    cudaStream_t st = l.streams[k % KvLink::kStreams];
    stream_wait_geq(st, arrived_of(l.region.p, l, k), k + 1);
    count_launch();
    link_signal_kernel<<<1, 1, 0, st>>>(ack_of(l.peer, l, k), k + 1);
    RB_CUDA(cudaGetLastError());
  }
}

// Waits until everything enqueued on one link has run, at most timeout_ms; on the deadline the
// link's waits are released, it is marked broken and the call fails.
void Backend::kv_link_wait(int link, int timeout_ms) {
  set_device();
  if (timeout_ms <= 0) timeout_ms = 60000;
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  for (;;) {
    {
      std::lock_guard<std::mutex> lock(copy_mu_);
      KvLink& l = link_of(link);
      const cudaError_t a = l.busy();
      if (a != cudaErrorNotReady && a != cudaSuccess) RB_CUDA(a);
      if (a == cudaSuccess) {
        if (l.broken) fail(RB200_ERR_RUNTIME, "kv link: broken by an earlier timeout");
        return;
      }
      if (std::chrono::steady_clock::now() > deadline) {
        links_release();
        fail(RB200_ERR_RUNTIME, "kv_link_wait: timed out; the link is broken");
      }
    }
    std::this_thread::yield();
  }
}

// Waits until every message sent so far has read its pages out of the cache (its gather has run;
// the bytes may still be on their way): from then on the sender's blocks may be reused. relay frees
// a request's blocks once its last frame is written (engine/src/kv_transfer.cpp:139-160), which
// read_kv_layer's synchronous copy made safe; a sender over a link calls this instead.
void Backend::kv_link_wait_gathered(int link, int timeout_ms) {
  set_device();
  if (timeout_ms <= 0) timeout_ms = 60000;
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  for (;;) {
    {
      std::lock_guard<std::mutex> lock(copy_mu_);
      KvLink& l = link_of(link);
      const cudaError_t a = l.busy(true);
      if (a != cudaErrorNotReady && a != cudaSuccess) RB_CUDA(a);
      if (a == cudaSuccess) {
        if (l.broken) fail(RB200_ERR_RUNTIME, "kv link: broken by an earlier timeout");
        return;
      }
      if (std::chrono::steady_clock::now() > deadline) {
        links_release();
        fail(RB200_ERR_RUNTIME, "kv_link_wait_gathered: timed out (the receiver does not free ring slots); the link is broken");
      }
    }
    std::this_thread::yield();
  }
}

// True when every link stream is idle. On `deadline` (links_sync gave up), every wait a peer has
// not satisfied is released from the host by writing the awaited counters, and the links are
// marked broken: what their last messages scattered is not to be used.
bool Backend::links_idle() {
  for (auto& l : links_) {
    if (!l) continue;
    for (cudaStream_t s : l->streams) {
      const cudaError_t q = cudaStreamQuery(s);
      if (q == cudaErrorNotReady) return false;
      if (q != cudaSuccess) RB_CUDA(q);
    }
  }
  return true;
}

void Backend::links_release() {
  // Every wait here is bounded: the counters are written on a stream that carries nothing else,
  // and the link's streams are polled, not synchronised. A link still busy two seconds later
  // (its streams sit behind work this end cannot release) is abandoned: marked wedged, its
  // region never freed, and the process stops making device-wide synchronising calls.
  for (auto& l : links_) {
    if (!l || l->wedged) continue;
    if (l->busy() != cudaErrorNotReady) continue;
    l->broken = true;
    cudaMemcpyAsync(l->region.p, l->release_words.p, kControlBytes, cudaMemcpyHostToDevice, l->release_stream);
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(2);
    bool busy = true;
    while (busy && std::chrono::steady_clock::now() < deadline) {
      busy = l->busy() == cudaErrorNotReady || cudaStreamQuery(l->release_stream) == cudaErrorNotReady;
      if (busy) std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
    if (busy) {
      l->wedged = true;
      g_device_wedged.store(true);
    }
  }
  cudaGetLastError();
}

}  // namespace rb200

extern "C" int rb200_kv_link_plan(size_t slot_bytes, size_t block_bytes, int n_layers, int n, int32_t* layers_per_message_out) {
  if (block_bytes == 0 || slot_bytes < 2 * block_bytes || slot_bytes % 256 != 0 || n_layers < 1 || n < 0) return -1;
  if (n == 0) {
    if (layers_per_message_out) *layers_per_message_out = 0;
    return 0;
  }
  const std::vector<rb200::LinkMsg> msgs = rb200::link_messages(slot_bytes, block_bytes, 0, n_layers, n);
  int most = 0;
  for (const rb200::LinkMsg& m : msgs)
    if (m.m == n) most = std::max(most, m.layers);
  if (layers_per_message_out) *layers_per_message_out = most;
  return static_cast<int>(msgs.size());
}
