// Raw transport throughput, no collectives:
//   stdml_collective_bench_send_recv s <host:port> <bytes>    server
//   stdml_collective_bench_send_recv c <host:port> <bytes> [batches] [per-batch]   client
// The client sends batches of messages of <bytes> bytes on a user connection
// type and logs MiB/s per batch; the server counts and discards them.
// (Reference counterpart: apps/stdml_collective_bench_send_recv.cpp:72-123.)
#include <atomic>
#include <chrono>
#include <cstdio>
#include <thread>
#include <vector>

#include <stdml/bits/collective/rchan.hpp>
#include <stdml/bits/collective/stat.hpp>

using namespace stdml::collective;

static constexpr rchan::conn_type conn_bench = static_cast<rchan::conn_type>(129);

struct sink : rchan::msg_handler {
    std::vector<char> scratch;
    std::atomic<size_t> messages{0}, bytes{0};
    bool operator()(const rchan::received_header &mh, rchan::message_reader *reader,
                    const peer_id &) override
    {
        if (scratch.size() < mh.len) { scratch.resize(mh.len); }
        if (!reader->read_body(scratch.data())) { return false; }
        ++messages;
        bytes += mh.len;
        return true;
    }
};

struct sink_conn : rchan::conn_handler {
    sink h;
    size_t operator()(std::unique_ptr<rchan::connection> conn) override
    {
        const size_t n = handle_to_end(conn.get(), &h);
        std::printf("connection from %s closed after %zu messages, %s\n",
                    conn->src().str().c_str(), n, rchan::show_size(h.bytes).c_str());
        return n;
    }
};

int main(int argc, char *argv[])
{
    if (argc < 4) {
        std::fprintf(stderr, "usage: %s s|c <host:port> <bytes> [batches] [per-batch]\n", argv[0]);
        return 2;
    }
    const auto addr = parse_peer_id(argv[2]);
    if (!addr) {
        std::fprintf(stderr, "bad address %s\n", argv[2]);
        return 2;
    }
    const size_t size = std::strtoull(argv[3], nullptr, 10);
    if (argv[1][0] == 's') {
        sink_conn handler;
        auto server = rchan::server::New(*addr, &handler);
        const int seconds = argc > 4 ? std::atoi(argv[4]) : 0;
        if (seconds > 0) {
            server->start();
            std::this_thread::sleep_for(std::chrono::seconds(seconds));
            server->stop();
        } else {
            server->serve();
        }
        return 0;
    }
    const int batches = argc > 4 ? std::atoi(argv[4]) : 100;
    const int per_batch = argc > 5 ? std::atoi(argv[5]) : 100;
    std::vector<char> payload(size, 'x');
    auto client = rchan::client::New(peer_id{(127u << 24) | 1u, 0}, conn_bench);
    for (int b = 0; b < batches; ++b) {
        const auto t0 = std::chrono::steady_clock::now();
        for (int i = 0; i < per_batch; ++i) {
            client->send(*addr, "payload", payload.data(), payload.size());
        }
        const std::chrono::duration<double> d = std::chrono::steady_clock::now() - t0;
        std::printf("batch %d: %.1f MiB/s\n", b + 1, size * per_batch / d.count() / 1048576.0);
    }
    return 0;
}
