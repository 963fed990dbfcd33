// rchan wire protocol ("reliable channel") and its connection interface.
// Byte-compatible with the reference (doc/rchan.txt,
// include/stdml/bits/collective/connection.hpp:13-109):
//   handshake  : client sends conn_header {u16 type, u16 src_port, u32 src_ipv4},
//                server answers connection_ack {u32 token};
//   message    : u32 name_len, name, u32 flags, u32 len, data   (host byte order).
// Here it carries the control plane (bootstrap, consistency checks, elastic
// commits) and the host-memory collectives; device buffers never travel over it.
#pragma once
#include <cstddef>
#include <cstdint>
#include <memory>
#include <optional>
#include <string>

#include <stdml/bits/collective/address.hpp>

namespace stdml::collective::rchan
{
enum conn_type : uint16_t {
    conn_ping,
    conn_control,
    conn_collective,
    conn_peer_to_peer,
    conn_mpi,
    conn_send,
    conn_recv,
    // [128, 255) are free for user protocols (see examples/example_rchan.cpp)
    conn_user_first = 128,
};

struct conn_header {
    uint16_t type;
    uint16_t src_port;
    uint32_t src_ipv4;
};
static_assert(sizeof(conn_header) == 8, "conn_header is 8 bytes on the wire");

struct connection_ack {
    uint32_t token;
};

struct message_header {
    static constexpr uint32_t wait_recv_buf = 1u << 0;   // rendezvous: read into a posted buffer
    static constexpr uint32_t is_response = 1u << 1;
    static constexpr uint32_t request_failed = 1u << 2;

    uint32_t name_len;
    char *name;
    uint32_t flags;
};

struct message {
    uint32_t len;
    void *data;
};

struct received_header {
    uint32_t name_len = 0;
    std::string name;
    uint32_t flags = 0;
    uint32_t len = 0;
};

// Reads one message from a connection in two steps, so the handler can decide
// where the body goes after it has seen the header.
class message_reader
{
  public:
    virtual ~message_reader() = default;
    // nullopt: the peer closed the connection
    virtual std::optional<received_header> read_header() = 0;
    // exactly header.len bytes into data; false on a broken connection
    virtual bool read_body(void *data) = 0;
};

class msg_handler
{
  public:
    virtual ~msg_handler() = default;
    // return false to stop serving this connection
    virtual bool operator()(const received_header &mh, message_reader *reader,
                            const peer_id &src) = 0;
};

class connection
{
  public:
    // Connects (retrying until the peer is up or `patience_ms` runs out; negative:
    // the connect timeout of the configuration), performs the handshake.  Throws
    // peer_failure (a std::runtime_error) when the patience runs out.
    static std::unique_ptr<connection> dial(const peer_id remote, const conn_type type,
                                            const peer_id local, int64_t patience_ms = -1);
    // One attempt with a deadline (always TCP); null if `remote` does not answer.
    // dial() is patient because a peer may still be starting; this is for
    // messages to members that may be dying.
    static std::unique_ptr<connection> dial_once(const peer_id remote, const conn_type type,
                                                 const peer_id local, int timeout_ms);
    virtual ~connection() = default;
    virtual conn_type type() const = 0;
    virtual peer_id src() const = 0;
    virtual std::unique_ptr<message_reader> next() = 0;
    // header and body leave in one gathered write; thread-safe
    virtual void send(const char *name, const void *data, size_t size, uint32_t flags = 0) = 0;
};

// default 120 s; STDML_COLLECTIVE_CONNECT_TIMEOUT_MS overrides; <= 0 waits forever
int64_t connect_timeout_ms();

// One conn_ping handshake (connect, header, ack) with a deadline: the round
// trip in microseconds, or -1 if `remote` does not answer within timeout_ms.
// The reference defines conn_ping but never uses it (connection.hpp:14 there).
double ping(const peer_id &remote, const peer_id &local, int timeout_ms);
}  // namespace stdml::collective::rchan
