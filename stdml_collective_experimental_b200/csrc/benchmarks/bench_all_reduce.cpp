// bench_all_reduce <AxB | sizes-file> <steps> [warmup]
// Per step every tensor is all-reduced (f32 sum), one after another, on host
// memory; rank 0 prints the reference's metric
//   "GiB/s" = 4 (np - 1) total_bytes / seconds / 2^30
// (benchmarks/bench_all_reduce.cpp:132,146 in the reference) so that numbers
// from both implementations are directly comparable.
#include <chrono>
#include <iostream>

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
    if (sess.rank() == 0) {
        log(PRINT) << sizes.size() << "tensors," << rchan::show_size(static_cast<size_t>(bytes));
    }
    const double multiplier = 4.0 * (sess.size() - 1);
    auto stage = [&](const char *name, int n) {
        std::vector<double> metrics;
        for (int i = 0; i < n; ++i) {
            const auto t0 = std::chrono::steady_clock::now();
            for (size_t k = 0; k < m.send.size(); ++k) {
                sess.all_reduce(m.send[k].data(), m.recv[k].data(), m.send[k].size(), f32, sum,
                                m.names[k]);
            }
            const std::chrono::duration<double> d = std::chrono::steady_clock::now() - t0;
            metrics.push_back(bench::gib(multiplier * bytes) / d.count());
            if (sess.rank() == 0) {
                std::cout << name << " " << i + 1 << " " << rchan::show_rate(metrics.back())
                          << " | " << rchan::show_duration(d) << std::endl;
            }
        }
        return metrics;
    };
    stage("warmup", warmup);
    const auto t0 = std::chrono::steady_clock::now();
    const auto metrics = stage("step", steps);
    const std::chrono::duration<double> total = std::chrono::steady_clock::now() - t0;
    if (sess.rank() == 0) {
        std::cout << "took: " << total.count() * 1e3 << " ms for " << steps << " steps" << std::endl;
        std::cout << "FINAL RESULT: " << workload << " " << rchan::show_rate(bench::mean(metrics))
                  << " | " << p.config() << " | " << strategy_name(sess.get_strategy())
                  << std::endl;
    }
    return 0;
}
