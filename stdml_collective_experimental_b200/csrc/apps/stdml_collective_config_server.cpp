// stdml_collective_config_server: the elastic configuration service on its own
// (the launcher embeds the same service with -builtin-config-port).
//
//   stdml_collective_config_server -port 9100 [-init cluster.json] [-ttl seconds]
//
// GET  /config            -> the current {"Runners":[...],"Workers":[...]}
// PUT  /config  <json>    -> validate and store a proposal (400 when malformed)
// Workers read it through KUNGFU_CONFIG_SERVER=http://host:9100/config.  In the
// reference this role is played by KungFu's Go launcher (-builtin-config-port).
#include <chrono>
#include <csignal>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <mutex>
#include <sstream>
#include <thread>

#include <stdml/bits/collective/address.hpp>
#include <stdml/bits/collective/http.hpp>

using namespace stdml::collective;

static volatile std::sig_atomic_t g_stop = 0;
static void on_signal(int) { g_stop = 1; }

int main(int argc, char *argv[])
{
    int port = 9100, ttl = 0;
    std::string stored = cluster_config().json();
    for (int i = 1; i < argc; ++i) {
        if (std::strcmp(argv[i], "-port") == 0 && i + 1 < argc) {
            port = std::atoi(argv[++i]);
        } else if (std::strcmp(argv[i], "-ttl") == 0 && i + 1 < argc) {
            ttl = std::atoi(argv[++i]);
        } else if (std::strcmp(argv[i], "-init") == 0 && i + 1 < argc) {
            std::ifstream in(argv[++i]);
            std::stringstream ss;
            ss << in.rdbuf();
            if (!cluster_config::from_json(ss.str())) {
                std::fprintf(stderr, "%s: %s is not a cluster configuration\n", argv[0], argv[i]);
                return 2;
            }
            stored = ss.str();
        } else {
            std::fprintf(stderr, "usage: %s -port P [-init cluster.json] [-ttl seconds]\n", argv[0]);
            return 2;
        }
    }
    std::mutex mu;
    int version = 0;
    http_server server(static_cast<uint16_t>(port), [&](const http_server::request &rq) {
        http_response rs;
        rs.status = 200;
        std::lock_guard<std::mutex> lk(mu);
        if (rq.method == "PUT" || rq.method == "POST") {
            if (!cluster_config::from_json(rq.body)) {
                rs.status = 400;
                rs.body = "{\"error\":\"malformed cluster\"}";
                return rs;
            }
            if (rq.body != stored) {
                stored = rq.body;
                ++version;
                std::printf("proposal %d: %s\n", version, stored.c_str());
                std::fflush(stdout);
            }
        }
        rs.body = stored;
        return rs;
    });
    std::signal(SIGINT, on_signal);
    std::signal(SIGTERM, on_signal);
    server.start();
    std::printf("config server on http://127.0.0.1:%u/config\n", server.port());
    std::fflush(stdout);
    const auto t0 = std::chrono::steady_clock::now();
    while (!g_stop) {
        std::this_thread::sleep_for(std::chrono::milliseconds(50));
        if (ttl > 0 && std::chrono::steady_clock::now() - t0 > std::chrono::seconds(ttl)) { break; }
    }
    server.stop();
    return 0;
}
