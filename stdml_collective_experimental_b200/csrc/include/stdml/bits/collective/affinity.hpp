// CPU pinning of a rank: rank r of n gets the r-th of n equal slices of the
// CPUs this process may run on.  Counterpart of
// include/stdml/bits/collective/affinity.hpp / src/stdml/collective/affinity.cpp:48-66
// (whose Linux helper sets CPU i instead of cpus[i]; fixed here).
#pragma once
#include <cstddef>
#include <vector>

namespace stdml::collective
{
// CPUs of slice `rank` of `size` out of `allowed`
std::vector<int> affinity_slice(const std::vector<int> &allowed, size_t rank, size_t size);
// false when the platform refuses
bool set_affinity(size_t rank, size_t size);
}  // namespace stdml::collective

extern "C" int stdml_collective_set_affinity(int n, const int *cpus);
