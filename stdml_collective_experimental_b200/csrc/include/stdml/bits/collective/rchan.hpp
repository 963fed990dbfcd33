// rchan endpoints: a server that accepts connections and feeds messages to a
// conn_handler, a client that keeps one outgoing connection per target, and a
// pool of clients keyed by connection type.  Same surface as the reference
// (include/stdml/bits/collective/rchan.hpp:13-85).
#pragma once
#include <cstddef>
#include <cstdint>
#include <map>
#include <memory>
#include <mutex>

#include <stdml/bits/collective/address.hpp>
#include <stdml/bits/collective/connection.hpp>

namespace stdml::collective::rchan
{
class conn_handler
{
  protected:
    // one message: header -> h(header, reader, src); false when the stream ended
    bool handle_next(connection *conn, msg_handler *h);
    // messages until the stream ends; returns how many were handled
    size_t handle_to_end(connection *conn, msg_handler *h);

  public:
    virtual ~conn_handler() = default;
    // called on the connection's own thread; returns the number of messages
    virtual size_t operator()(std::unique_ptr<connection> conn) = 0;
};

class client
{
  public:
    virtual ~client() = default;
    virtual void send(const peer_id target, const char *name, const void *data, size_t size,
                      uint32_t flags = 0) = 0;
    virtual std::unique_ptr<connection> dial(peer_id target, conn_type type) = 0;
    // drop the connections to these peers
    virtual void reset_peers(const peer_list &ids) = 0;
    // how long a first connection to a peer is retried (negative: the configured
    // connect timeout).  Long while members may still be starting, short once
    // all of them have been seen alive: then a refused connection means a dead peer.
    virtual void set_dial_patience_ms(int64_t ms) = 0;
    static std::unique_ptr<client> New(peer_id self, conn_type type);
};

class client_pool
{
    const peer_id self_;
    std::mutex mu_;
    std::map<conn_type, std::unique_ptr<client>> clients_;
    int64_t patience_ms_ = -1;

  public:
    explicit client_pool(const peer_id self) : self_(self) {}
    client *require(conn_type type);
    void reset_peers(const peer_list &ids);
    void set_dial_patience_ms(int64_t ms);
};

class server
{
  public:
    virtual ~server() = default;
    virtual void serve() = 0;  // blocks until stop()
    virtual void start() = 0;  // serve on a background thread
    virtual void stop() = 0;   // closes the listener and every connection, joins
    static std::unique_ptr<server> New(const peer_id self, conn_handler *handler);
};
}  // namespace stdml::collective::rchan
