// relay's transfer engine over a K/V link, without a change to relay's sources.
//
// KVSender::send_layer (engine/src/kv_transfer.cpp:107-128) gathers a layer's blocks with
// Backend::read_kv_layer and writes [header][payload] to its Connection; KVReceiver::handle
// (engine/src/kv_transfer.cpp:269-301) reads the header, reads the payload, and lands it with
// Backend::write_kv_layer. Both Backend and Connection are virtual interfaces, so the payload
// can change its road from outside: the B200 backend (relay_b200/csrc/adapter.cpp) and a
// Connection wrapper made here agree that, on a wrapped connection,
//   * read_kv_layer does not copy the pages to the host but sends them over the link
//     (rb200_kv_link_send_layer), and the wrapper then writes only the Layer frame's header;
//   * the wrapper answers the receiver's read of the payload without reading anything, and
//     write_kv_layer lands the pages from the link (rb200_kv_link_recv_layer) and waits for
//     them; a Layer frame the receiver drops (no room for the request) is dropped from the
//     link too (rb200_kv_link_skip_layer).
// Every frame header, the Hello / Begin / End / Abort frames and with them the ordering and
// failure semantics stay on the host connection exactly as relay has them.
//
// C++ (relay's language), compiled against relay's headers; the functions are defined in
// relay_b200/csrc/adapter.cpp. `backend` must be one made by relay::make_cuda_backend of this
// library; anything else throws std::invalid_argument.
#pragma once

#include <cstddef>
#include <memory>

#include "relay/backend.h"
#include "relay/transport.h"
#include "relay_b200.h"

namespace relay {
namespace b200 {

struct KvLinkEnd {
  int link = -1;                                     // this end's id on its backend
  unsigned char handle[RB200_KV_LINK_HANDLE_BYTES];  // what the other end needs to connect (another process)
};

// One end of a link on `backend`: a ring of n_slots slots of slot_bytes (see rb200_kv_link_create).
KvLinkEnd kv_link_create(Backend& backend, int n_slots, std::size_t slot_bytes);
// The other end lives in another process: its handle came over the host connection.
void kv_link_connect(Backend& backend, int link, const void* peer_handle);
// Both ends live in this process.
void kv_link_connect_local(Backend& a, int link_a, Backend& b, int link_b);
void kv_link_close(Backend& backend, int link);

// Wraps the connection a KVSender writes to. While the wrapper lives, read_kv_layer on `backend`
// sends over `link` instead of copying to the host.
std::unique_ptr<Connection> kv_link_sender_connection(Connection& inner, Backend& backend, int link);
// Wraps the connection a KVReceiver reads from. While the wrapper lives, write_kv_layer on
// `backend` lands pages from `link`; `timeout_ms` bounds each wait for them.
std::unique_ptr<Connection> kv_link_receiver_connection(Connection& inner, Backend& backend, int link,
                                                        int timeout_ms = 30000);

}  // namespace b200
}  // namespace relay
