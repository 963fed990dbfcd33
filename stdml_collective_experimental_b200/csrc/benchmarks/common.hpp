// Shared pieces of the C++ benchmarks: workload parsing ("AxB" = B tensors of A
// elements, or a file with one element count per line, the reference's
// formats: benchmarks/bench_all_reduce.cpp:174-194) and the synthetic model.
#pragma once
#include <cstdio>
#include <fstream>
#include <numeric>
#include <stdexcept>
#include <string>
#include <vector>

namespace bench
{
inline std::vector<size_t> parse_workload(const std::string &w)
{
    unsigned long a = 0, b = 0;
    char tail;
    if (std::sscanf(w.c_str(), "%lux%lu%c", &a, &b, &tail) == 2) {
        return std::vector<size_t>(b, a);
    }
    std::ifstream in(w);
    if (!in) { throw std::runtime_error("cannot open workload file " + w); }
    std::vector<size_t> sizes;
    size_t n;
    while (in >> n) { sizes.push_back(n); }
    return sizes;
}

// send buffers hold 1, receive buffers -1, like the reference's fake model
struct model {
    std::vector<std::string> names;
    std::vector<std::vector<float>> send, recv;

    explicit model(const std::vector<size_t> &sizes)
    {
        for (size_t i = 0; i < sizes.size(); ++i) {
            names.push_back("variable:" + std::to_string(i));
            send.emplace_back(sizes[i], 1.0f);
            recv.emplace_back(sizes[i], -1.0f);
        }
    }

    size_t elements() const
    {
        size_t n = 0;
        for (const auto &s : send) { n += s.size(); }
        return n;
    }
};

inline double gib(double bytes) { return bytes / 1073741824.0; }

inline double mean(const std::vector<double> &xs)
{
    return xs.empty() ? 0.0 : std::accumulate(xs.begin(), xs.end(), 0.0) / xs.size();
}
}  // namespace bench
