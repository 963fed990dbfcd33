// Fixed-size worker pool.  Counterpart of
// include/stdml/bits/collective/thread_pool.hpp:9-58: New, add, wait, and
// par() which runs a batch of closures and returns when all have finished
// (the caller's thread runs the first one, like the reference's par1).
#pragma once
#include <cstddef>
#include <functional>
#include <memory>
#include <vector>

namespace stdml::sync
{
class thread_pool
{
  public:
    using task = std::function<void()>;

    virtual ~thread_pool() = default;

    static thread_pool *New(size_t n);
    static std::unique_ptr<thread_pool> make(size_t n);

    virtual size_t size() const = 0;
    virtual void add(task f) = 0;
    // blocks until every task added so far has finished
    virtual void wait() = 0;
    // runs all of fs (caller participates); rethrows the first exception
    virtual void par(std::vector<task> fs) = 0;
};
}  // namespace stdml::sync
