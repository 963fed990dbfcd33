// Counting latch: add(n), done(), wait() until the count is back to zero.
// Counterpart of include/stdml/bits/collective/waitgroup.hpp.
#pragma once
#include <condition_variable>
#include <cstddef>
#include <mutex>

namespace stdml::sync
{
class wait_group
{
    std::mutex mu_;
    std::condition_variable cv_;
    size_t pending_ = 0;

  public:
    void add(size_t n = 1);
    void done();
    void wait();
};
}  // namespace stdml::sync
