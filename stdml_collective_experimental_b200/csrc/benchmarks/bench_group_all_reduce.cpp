// bench_group_all_reduce <AxB | sizes-file> <steps> [warmup]
// One group_all_reduce of the whole tensor set per step; every rank submits the
// tensors in its own rotated order with futures that resolve later, the case
// that hangs the reference on sets above 76 tensors
// (benchmarks/bench_group_all_reduce.cpp:73-85, src/stdml/collective/session.cpp:85).
#include <chrono>
#include <future>
#include <iostream>
#include <thread>

#include <stdml/collective>

#include "common.hpp"

using namespace stdml::collective;

int main(int argc, char *argv[])
{
    if (argc < 3) {
        std::fprintf(stderr, "usage: %s <AxB | sizes-file> <steps> [warmup]\n", argv[0]);
        return 2;
    }
    const std::string workload = argv[1];
    const int steps = std::atoi(argv[2]);
    const int warmup = argc > 3 ? std::atoi(argv[3]) : 0;
    const auto sizes = bench::parse_workload(workload);
    bench::model m(sizes);
    const double bytes = 4.0 * m.elements();

    auto p = peer::from_env();
    session sess = p.join();
    const double multiplier = 4.0 * (sess.size() - 1);
    const size_t n = m.send.size();
    auto step = [&] {
        std::vector<std::promise<workspace>> promises(n);
        std::vector<std::future<workspace>> futures;
        for (auto &pr : promises) { futures.push_back(pr.get_future()); }
        std::thread producer([&] {
            const size_t shift = sess.rank() * (n / std::max<size_t>(1, sess.size()));
            for (size_t k = 0; k < n; ++k) {
                const size_t i = (k + shift) % n;
                promises[i].set_value(workspace{m.send[i].data(), m.recv[i].data(),
                                                m.send[i].size(), f32, sum, m.names[i]});
            }
        });
        sess.group_all_reduce(std::move(futures));
        producer.join();
    };
    std::vector<double> metrics;
    for (int i = 0; i < warmup + steps; ++i) {
        const auto t0 = std::chrono::steady_clock::now();
        step();
        const std::chrono::duration<double> d = std::chrono::steady_clock::now() - t0;
        const double metric = bench::gib(multiplier * bytes) / d.count();
        if (i >= warmup) { metrics.push_back(metric); }
        if (sess.rank() == 0) {
            std::cout << (i < warmup ? "warmup " : "step ") << i + 1 << " "
                      << rchan::show_rate(metric) << " | " << rchan::show_duration(d) << std::endl;
        }
    }
    bool ok = true;
    for (const auto &r : m.recv) { ok = ok && (r.empty() || r[0] == float(sess.size())); }
    if (sess.rank() == 0) {
        std::cout << "FINAL RESULT: " << workload << " " << rchan::show_rate(bench::mean(metrics))
                  << " | " << p.config() << " | " << (ok ? "verified" : "WRONG") << std::endl;
    }
    return ok ? 0 : 1;
}
