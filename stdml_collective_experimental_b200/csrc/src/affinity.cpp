#include <sched.h>

#include <stdml/bits/collective/affinity.hpp>
#include <stdml/bits/collective/buffer.hpp>

extern "C" int stdml_collective_set_affinity(int n, const int *cpus)
{
    cpu_set_t set;
    CPU_ZERO(&set);
    for (int i = 0; i < n; ++i) { CPU_SET(cpus[i], &set); }
    return sched_setaffinity(0, sizeof(set), &set);
}

namespace stdml::collective
{
std::vector<int> affinity_slice(const std::vector<int> &allowed, size_t rank, size_t size)
{
    if (size == 0 || allowed.empty()) { return {}; }
    if (allowed.size() < size) { return {allowed[rank % allowed.size()]}; }
    const auto [b, e] = even_part(allowed.size(), size, rank % size);
    return std::vector<int>(allowed.begin() + b, allowed.begin() + e);
}

bool set_affinity(size_t rank, size_t size)
{
    cpu_set_t cur;
    CPU_ZERO(&cur);
    if (sched_getaffinity(0, sizeof(cur), &cur) != 0) { return false; }
    std::vector<int> allowed;
    for (int c = 0; c < CPU_SETSIZE; ++c) {
        if (CPU_ISSET(c, &cur)) { allowed.push_back(c); }
    }
    const std::vector<int> mine = affinity_slice(allowed, rank, size);
    if (mine.empty()) { return false; }
    return stdml_collective_set_affinity(static_cast<int>(mine.size()), mine.data()) == 0;
}
}  // namespace stdml::collective
