// The transport is extensible: a user protocol on its own connection type
// (>= 128) with its own message handler, next to the collective traffic.
//   example_rchan            runs a server and a client in one process
#include <atomic>
#include <cstdio>
#include <string>
#include <thread>

#include <stdml/bits/collective/rchan.hpp>

using namespace stdml::collective;

static constexpr rchan::conn_type conn_echo = static_cast<rchan::conn_type>(130);

struct echo_handler : rchan::msg_handler {
    std::atomic<int> seen{0};
    bool operator()(const rchan::received_header &mh, rchan::message_reader *reader,
                    const peer_id &src) override
    {
        std::string body(mh.len, '\0');
        if (!reader->read_body(body.data())) { return false; }
        std::printf("[%s] %s: %s\n", src.str().c_str(), mh.name.c_str(), body.c_str());
        ++seen;
        return true;
    }
};

struct echo_conn_handler : rchan::conn_handler {
    echo_handler h;
    size_t operator()(std::unique_ptr<rchan::connection> conn) override
    {
        if (conn->type() != conn_echo) { return 0; }
        return handle_to_end(conn.get(), &h);
    }
};

int main()
{
    const peer_id server_id = *parse_peer_id("127.0.0.1:19999");
    const peer_id client_id = *parse_peer_id("127.0.0.1:19998");
    echo_conn_handler handler;
    auto server = rchan::server::New(server_id, &handler);
    server->start();
    {
        auto client = rchan::client::New(client_id, conn_echo);
        for (int i = 0; i < 3; ++i) {
            const std::string msg = "hello " + std::to_string(i);
            client->send(server_id, "greeting", msg.data(), msg.size());
        }
    }
    for (int i = 0; i < 200 && handler.h.seen < 3; ++i) {
        std::this_thread::sleep_for(std::chrono::milliseconds(5));
    }
    server->stop();
    return handler.h.seen == 3 ? 0 : 1;
}
