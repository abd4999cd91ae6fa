// relay's transfer engine (KVSender / KVReceiver / PrefillWorker / Engine, unmodified) driven
// over a K/V link: the Layer payloads cross GPU to GPU, everything else stays on the TCP
// connection. Built by `make -C oracle reftests` against relay's headers and engine objects;
// run by tests/test_gpu_reference_suite.py on a GPU.
//
// What is checked (the same properties relay's own tests/test_transfer.cpp:236-300 and
// tests/test_faults.cpp:118-215 check over a socket):
//   * prefill on one backend + decode on another gives the tokens one engine alone gives, with
//     whole-prompt and with 10-token prefill chunks (a block then travels once per chunk that
//     touches it and the last version must win);
//   * the same with a decode side too small for the traffic, where the receiver drops Layer
//     frames (and the link must drop their pages) and recomputes;
//   * only frame headers and the small frames crossed the host connection;
//   * a host connection cut after any number of bytes loses nothing and leaks nothing: every
//     request is either delivered in full or reported failed once, both sides get all their
//     blocks back, and nothing hangs.
// RB200_LINK_DEVICES="p,d" puts the prefill backend on device p and the decode backend on
// device d (default "0,0": two backends sharing one GPU).
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <limits>
#include <map>
#include <mutex>
#include <random>
#include <set>
#include <thread>

#include "relay/engine.h"
#include "relay/kv_transfer.h"
#include "relay/transport.h"
#include "relay/weights.h"
#include "relay_b200_transfer.h"

using namespace relay;

namespace {

int g_failures = 0;
#define EXPECT(cond)                                                        \
  do {                                                                      \
    if (!(cond)) {                                                          \
      ++g_failures;                                                         \
      std::fprintf(stderr, "  FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
    }                                                                       \
  } while (0)

using Tokens = std::map<std::uint64_t, std::vector<int>>;
using ConnPair = std::pair<std::unique_ptr<Connection>, std::unique_ptr<Connection>>;

constexpr int kBlock = 8;
int g_prefill_device = 0, g_decode_device = 0;

ConnPair tcp_pair() {
  TcpListener listener(0);
  std::unique_ptr<Connection> client;
  std::thread t([&] { client = tcp_connect("127.0.0.1", listener.port()); });
  auto server = listener.accept();
  t.join();
  return {std::move(client), std::move(server)};
}

// Counts what is sent, and after `limit` bytes cuts the connection under both sides (the fault
// is made on the host: part of a frame may have gone out, the rest never will).
class CountingCut final : public Connection {
 public:
  CountingCut(Connection& inner, std::size_t limit) : inner_(inner), limit_(limit) {}
  void send(const Slice* slices, int n) override {
    std::size_t total = 0;
    for (int i = 0; i < n; ++i) total += slices[i].len;
    if (sent_ + total <= limit_) {
      inner_.send(slices, n);
      sent_ += total;
      return;
    }
    std::size_t room = limit_ - sent_;
    std::vector<Slice> head;
    for (int i = 0; i < n && room > 0; ++i) {
      const std::size_t k = std::min(room, slices[i].len);
      head.push_back({slices[i].data, k});
      room -= k;
    }
    if (!head.empty()) inner_.send(head.data(), static_cast<int>(head.size()));
    sent_ = limit_;
    inner_.close();
    throw ConnectionClosed("cut by the test");
  }
  void recv(void* dst, std::size_t len) override { inner_.recv(dst, len); }
  void close() override { inner_.close(); }
  std::string describe() const override { return "cut(" + inner_.describe() + ")"; }
  std::size_t sent() const { return sent_; }

 private:
  Connection& inner_;
  std::size_t limit_, sent_ = 0;
};

std::vector<Request> requests(std::uint32_t seed, int vocab, int count, int max_len) {
  std::mt19937 rng(seed);
  std::vector<Request> rs;
  for (int i = 0; i < count; ++i) {
    Request r;
    r.id = 100 + i;
    const int len = 1 + static_cast<int>(rng() % max_len);
    for (int t = 0; t < len; ++t) r.prompt.push_back(static_cast<int>(rng() % vocab));
    r.params.max_new_tokens = 1 + static_cast<int>(rng() % 7);  // 1: done at its first token
    r.params.ignore_eos = true;
    if (rng() % 2) {
      r.params.temperature = 0.8f;
      r.params.seed = rng();
    }
    rs.push_back(r);
  }
  return rs;
}

Tokens one_engine(const HostWeights& w, const std::vector<Request>& rs) {
  auto be = make_cuda_backend(w, 64, kBlock, g_prefill_device, 1024, 64 * kBlock);
  Engine e(*be, {256, 64});
  for (const auto& r : rs) e.add(r);
  return e.run_all();
}

struct Outcome {
  Tokens tokens;                       // by request: first token from the prefill side, the rest from decode
  std::set<std::uint64_t> failed;      // reported by the prefill worker as not delivered
  std::size_t host_bytes = 0;          // what the sender wrote to the host connection
  TransferStats sent, received;
  bool receiver_error = false;
  int in_flight = 0, prefill_free = -1, decode_free = -1;
};

// Prefill on one backend, decode on another; the frames over TCP, the pages over a link.
Outcome two_engines(const HostWeights& w, const std::vector<Request>& rs, int prefill_budget, int decode_blocks,
                    std::size_t cut_after = std::numeric_limits<std::size_t>::max()) {
  Outcome o;
  auto pb = make_cuda_backend(w, 64, kBlock, g_prefill_device, 1024, 64 * kBlock);
  auto db = make_cuda_backend(w, decode_blocks, kBlock, g_decode_device, 1024, decode_blocks * kBlock);
  // a ring of 3 slots of 4 blocks: long prompts travel as several messages and wrap the ring
  const std::size_t slot = 4 * 2 * pb->kv_block_bytes();
  b200::KvLinkEnd pe = b200::kv_link_create(*pb, 3, slot), de = b200::kv_link_create(*db, 3, slot);
  b200::kv_link_connect_local(*pb, pe.link, *db, de.link);
  {
    Engine decode(*db, {256, 64});
    ConnPair tcp = tcp_pair();
    CountingCut wire(*tcp.first, cut_after);
    auto tx = b200::kv_link_sender_connection(wire, *pb, pe.link);
    auto rx = b200::kv_link_receiver_connection(*tcp.second, *db, de.link, 20000);
    KVReceiver receiver(decode, *db, *rx);
    std::map<std::uint64_t, int> first;
    std::vector<std::uint64_t> failed;
    {
      KVSender sender(*pb, *tx);
      PrefillWorker pw(*pb, sender, prefill_budget);
      for (const auto& r : rs) pw.add(r);
      while (pw.has_work())
        for (const TokenEvent& e : pw.step()) first[e.id] = e.token;
      try {
        sender.flush();
      } catch (const ConnectionClosed&) {
      }
      failed = pw.take_failed();
      o.prefill_free = pw.free_blocks();
      o.sent = sender.stats();
    }
    o.host_bytes = wire.sent();
    tcp.first->close();  // the prefill side is done (after a cut: closed already)
    receiver.join();
    o.receiver_error = receiver.error() != nullptr;
    o.in_flight = receiver.in_flight();
    o.received = receiver.stats();
    Tokens rest = decode.run_all();
    o.decode_free = decode.free_blocks();
    o.failed.insert(failed.begin(), failed.end());
    EXPECT(o.failed.size() == failed.size());  // each failure reported once
    for (const auto& r : rs) {
      if (o.failed.count(r.id)) {
        EXPECT(rest.count(r.id) == 0);  // never both delivered and failed
        continue;
      }
      auto f = first.find(r.id);
      EXPECT(f != first.end());
      if (f == first.end()) continue;
      std::vector<int> got{f->second};
      if (r.params.max_new_tokens > 1) {
        EXPECT(rest.count(r.id) == 1);
        got.insert(got.end(), rest[r.id].begin(), rest[r.id].end());
      }
      o.tokens[r.id] = got;
    }
  }
  b200::kv_link_close(*pb, pe.link);
  b200::kv_link_close(*db, de.link);
  return o;
}

void expect_clean(const Outcome& o, int decode_blocks) {
  EXPECT(!o.receiver_error);
  EXPECT(o.in_flight == 0);
  EXPECT(o.prefill_free == 64);
  EXPECT(o.decode_free == decode_blocks);
}

void same_tokens_as_one_engine(const HostWeights& w) {
  std::fprintf(stderr, "[ RUN  ] two engines over a link give one engine's tokens\n");
  const auto rs = requests(11, w.config.vocab, 8, 64);
  const Tokens want = one_engine(w, rs);
  for (int budget : {512, 10}) {
    Outcome o = two_engines(w, rs, budget, 64);
    expect_clean(o, 64);
    EXPECT(o.failed.empty());
    EXPECT(o.tokens == want);
    EXPECT(o.sent.requests == rs.size());
    // the pages did not cross the host connection: it carried far less than the K/V it announced
    EXPECT(o.sent.kv_bytes > 0 && o.host_bytes * 8 < o.sent.kv_bytes);
    std::fprintf(stderr, "  %d-token prefill steps: %llu K/V bytes over the link, %zu bytes over TCP\n", budget,
                 static_cast<unsigned long long>(o.sent.kv_bytes), o.host_bytes);
  }
}

void a_decode_side_without_room_drops_frames_and_recomputes(const HostWeights& w) {
  std::fprintf(stderr, "[ RUN  ] a decode side without room drops Layer frames from the link too\n");
  const auto rs = requests(11, w.config.vocab, 8, 64);
  const Tokens want = one_engine(w, rs);
  Outcome o = two_engines(w, rs, 512, 12);  // 12 blocks of 8 tokens: most transfers find no room
  expect_clean(o, 12);
  EXPECT(o.failed.empty());
  EXPECT(o.tokens == want);
  EXPECT(o.received.recomputed > 0);
  std::fprintf(stderr, "  %llu transfers fell back to recompute\n", static_cast<unsigned long long>(o.received.recomputed));
}

void a_cut_anywhere_loses_nothing_and_leaks_nothing(const HostWeights& w) {
  std::fprintf(stderr, "[ RUN  ] a host connection cut anywhere loses nothing and leaks nothing\n");
  const char* env = std::getenv("RELAY_FAULT_SEEDS");
  const std::uint32_t seeds = env && *env ? static_cast<std::uint32_t>(std::atoi(env)) : 24;
  int delivered = 0, failed = 0;
  for (std::uint32_t seed = 0; seed < seeds; ++seed) {
    const auto rs = requests(1000 + seed, w.config.vocab, 1 + static_cast<int>(seed % 4), 40);
    const Tokens want = one_engine(w, rs);
    const std::size_t total = two_engines(w, rs, 16, 32).host_bytes;  // what crosses without a fault
    std::mt19937_64 rng(seed * 7919u + 1);
    Outcome o = two_engines(w, rs, 16, 32, rng() % (total + 1));
    expect_clean(o, 32);
    for (const auto& [id, toks] : o.tokens) {
      // delivered in full (token values are compared in the runs without a fault above: on a GPU
      // the batch a token was computed in may reorder floating-point sums)
      EXPECT(toks.size() == want.at(id).size());
      ++delivered;
    }
    failed += static_cast<int>(o.failed.size());
    EXPECT(o.tokens.size() + o.failed.size() == rs.size());
  }
  std::fprintf(stderr, "  %u cuts: %d requests delivered, %d reported failed\n", seeds, delivered, failed);
  EXPECT(delivered > 0 && failed > 0);
}

}  // namespace

int main() {
  if (const char* d = std::getenv("RB200_LINK_DEVICES")) std::sscanf(d, "%d,%d", &g_prefill_device, &g_decode_device);
  const HostWeights w = HostWeights::load(RELAY_FIXTURES "/llama-gqa-tied-bf16");
  try {
    same_tokens_as_one_engine(w);
    a_decode_side_without_room_drops_frames_and_recomputes(w);
    a_cut_anywhere_loses_nothing_and_leaks_nothing(w);
  } catch (const std::exception& e) {
    ++g_failures;
    std::fprintf(stderr, "  FAILED: exception: %s\n", e.what());
  }
  std::fprintf(stderr, "%d failed\n", g_failures);
  return g_failures ? 1 : 0;
}
