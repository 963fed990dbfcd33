// Bounded blocking MPMC queue (capacity 1 by default): the hand-off primitive
// between network threads and collective callers.  Counterpart of the
// reference's channel<T> (include/stdml/bits/collective/channel.hpp:11-55),
// with a timed get added so that waits can be bounded.
#pragma once
#include <chrono>
#include <condition_variable>
#include <deque>
#include <mutex>
#include <optional>
#include <utility>

namespace stdml::collective
{
template <typename T>
class channel
{
    const size_t cap_;
    std::mutex mu_;
    std::condition_variable not_empty_, not_full_;
    std::deque<T> q_;

  public:
    explicit channel(size_t cap = 1) : cap_(cap > 0 ? cap : 1) {}

    T get()
    {
        std::unique_lock<std::mutex> lk(mu_);
        not_empty_.wait(lk, [&] { return !q_.empty(); });
        T x = std::move(q_.front());
        q_.pop_front();
        not_full_.notify_one();
        return x;
    }

    std::optional<T> try_get()
    {
        std::lock_guard<std::mutex> lk(mu_);
        if (q_.empty()) { return {}; }
        T x = std::move(q_.front());
        q_.pop_front();
        not_full_.notify_one();
        return x;
    }

    template <typename Rep, typename Period>
    std::optional<T> get_for(const std::chrono::duration<Rep, Period> &d)
    {
        std::unique_lock<std::mutex> lk(mu_);
        if (!not_empty_.wait_for(lk, d, [&] { return !q_.empty(); })) { return {}; }
        T x = std::move(q_.front());
        q_.pop_front();
        not_full_.notify_one();
        return x;
    }

    void put(T x)
    {
        std::unique_lock<std::mutex> lk(mu_);
        not_full_.wait(lk, [&] { return q_.size() < cap_; });
        q_.push_back(std::move(x));
        not_empty_.notify_one();
    }
};
}  // namespace stdml::collective
