#include <condition_variable>
#include <deque>
#include <exception>
#include <mutex>
#include <thread>

#include <stdml/bits/collective/thread_pool.hpp>
#include <stdml/bits/collective/waitgroup.hpp>

namespace stdml::sync
{
void wait_group::add(size_t n)
{
    std::lock_guard<std::mutex> lk(mu_);
    pending_ += n;
}

void wait_group::done()
{
    std::lock_guard<std::mutex> lk(mu_);
    if (pending_ > 0 && --pending_ == 0) { cv_.notify_all(); }
}

void wait_group::wait()
{
    std::unique_lock<std::mutex> lk(mu_);
    cv_.wait(lk, [&] { return pending_ == 0; });
}

namespace
{
class pool_impl final : public thread_pool
{
    std::mutex mu_;
    std::condition_variable work_cv_, idle_cv_;
    std::deque<task> queue_;
    size_t running_ = 0;
    bool stopping_ = false;
    std::vector<std::thread> workers_;

    void loop()
    {
        for (;;) {
            task f;
            {
                std::unique_lock<std::mutex> lk(mu_);
                work_cv_.wait(lk, [&] { return stopping_ || !queue_.empty(); });
                if (queue_.empty()) { return; }
                f = std::move(queue_.front());
                queue_.pop_front();
                ++running_;
            }
            try {
                f();
            } catch (...) {
                // add() has no way to report; par() wraps its tasks itself
            }
            {
                std::lock_guard<std::mutex> lk(mu_);
                --running_;
                if (queue_.empty() && running_ == 0) { idle_cv_.notify_all(); }
            }
        }
    }

  public:
    explicit pool_impl(size_t n)
    {
        n = n > 0 ? n : 1;
        workers_.reserve(n);
        for (size_t i = 0; i < n; ++i) { workers_.emplace_back([this] { loop(); }); }
    }

    ~pool_impl() override
    {
        {
            std::lock_guard<std::mutex> lk(mu_);
            stopping_ = true;
        }
        work_cv_.notify_all();
        for (auto &t : workers_) { t.join(); }
    }

    size_t size() const override { return workers_.size(); }

    void add(task f) override
    {
        {
            std::lock_guard<std::mutex> lk(mu_);
            queue_.push_back(std::move(f));
        }
        work_cv_.notify_one();
    }

    void wait() override
    {
        std::unique_lock<std::mutex> lk(mu_);
        idle_cv_.wait(lk, [&] { return queue_.empty() && running_ == 0; });
    }

    void par(std::vector<task> fs) override
    {
        if (fs.empty()) { return; }
        wait_group wg;
        std::mutex err_mu;
        std::exception_ptr err;
        auto guarded = [&](task &f) {
            try {
                f();
            } catch (...) {
                std::lock_guard<std::mutex> lk(err_mu);
                if (!err) { err = std::current_exception(); }
            }
        };
        wg.add(fs.size() - 1);
        for (size_t i = 1; i < fs.size(); ++i) {
            add([&, i] {
                guarded(fs[i]);
                wg.done();
            });
        }
        guarded(fs[0]);
        wg.wait();
        if (err) { std::rethrow_exception(err); }
    }
};
}  // namespace

thread_pool *thread_pool::New(size_t n) { return new pool_impl(n); }

std::unique_ptr<thread_pool> thread_pool::make(size_t n)
{
    return std::unique_ptr<thread_pool>(new pool_impl(n));
}
}  // namespace stdml::sync
