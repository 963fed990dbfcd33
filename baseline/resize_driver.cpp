// Times an elastic resize, peer::resize(sess, config_provider), of whichever
// implementation this file is compiled against: the reference
// (src/stdml/collective/peer.cpp:214-218 there) or this library, whose public
// API has the same shape.  No launcher is involved: the configuration comes from a file that the harness rewrites, and
// the harness starts the joiners itself with the reference's environment
// contract (KUNGFU_SELF_SPEC / KUNGFU_INIT_PEERS / KUNGFU_INIT_CLUSTER_VERSION).
// Only the public API that both implementations share is used; this file is a
// measuring harness, not part of the library.
//
//   REF_RESIZE_CONFIG=<file with "ip:port,ip:port,..."> resize-driver <max_step>
//
// Every step: one small all_reduce (so that members stay in step), then resize().
// Rank 0 of each membership prints "resized <old> -> <new> <milliseconds>".
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <optional>
#include <string>
#include <thread>

#include <stdml/collective>

using namespace stdml::collective;

int main(int argc, char *argv[])
{
    const int max_step = argc > 1 ? std::atoi(argv[1]) : 100;
    const char *path = std::getenv("REF_RESIZE_CONFIG");
    if (path == nullptr) { return 2; }
    auto provider = [path]() -> std::optional<cluster_config> {
        std::ifstream f(path);
        std::string line;
        if (!std::getline(f, line)) { return {}; }
        const auto workers = parse_peer_list(line);
        if (!workers) { return {}; }
        return cluster_config(peer_list{}, *workers);
    };
    auto p = peer::from_env();
    auto sess = p.join_elastic();
    int step = 0;
    bool synced = false;
    while (step < max_step) {
        if (!synced) {
            step = sess->all_reduce(step, max);
            synced = true;
            if (step >= max_step) { break; }
        }
        int one = 1;
        const int members = sess->all_reduce(one, sum);
        (void)members;
        const size_t old_size = sess->size();
        const auto t0 = std::chrono::steady_clock::now();
        const auto result = p.resize(sess, provider);
        const double ms =
            std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
        if (result.detached) {
            std::printf("detached at step %d\n", step);
            std::fflush(stdout);
            return 0;
        }
        if (result.changed) {
            if (sess->rank() == 0) {
                std::printf("resized %zu -> %zu %.3f ms (step %d)\n", old_size, sess->size(), ms, step);
                std::fflush(stdout);
            }
            synced = false;
        }
        ++step;
        std::this_thread::sleep_for(std::chrono::milliseconds(20));
    }
    if (sess->rank() == 0) { std::printf("finished size %zu\n", sess->size()); }
    return 0;
}
