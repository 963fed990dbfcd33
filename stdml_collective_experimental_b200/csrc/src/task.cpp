#include <atomic>
#include <cstdlib>
#include <cxxabi.h>
#include <thread>

#include <stdml/bits/collective/task.hpp>
#include <stdml/bits/collective/thread_pool.hpp>

namespace stdml::collective
{
namespace
{
std::atomic<size_t> g_tasks{0};

class pool_runtime final : public runtime
{
    std::unique_ptr<sync::thread_pool> pool_;

  public:
    explicit pool_runtime(size_t m) : pool_(sync::thread_pool::make(m)) {}

    void par(std::vector<std::unique_ptr<task>> &tasks) override
    {
        // Each worker owns a strided subset of the tasks and polls them
        // round-robin, so a task that waits for its peer never starves one
        // that could run (there may be far more tasks than workers).
        // A task that throws ends the whole set: the other workers stop polling
        // (their tasks may wait for something that will never come) and the
        // first exception reaches the caller through the pool.
        const size_t workers = std::min(pool_->size() + 1, tasks.size());
        std::atomic<bool> failed{false};
        std::vector<sync::thread_pool::task> fs;
        for (size_t w = 0; w < workers; ++w) {
            fs.emplace_back([&tasks, &failed, w, workers] {
                size_t left = 0;
                for (size_t i = w; i < tasks.size(); i += workers) { ++left; }
                std::vector<bool> done(tasks.size(), false);
                try {
                    while (left > 0 && !failed.load(std::memory_order_relaxed)) {
                        bool progressed = false;
                        for (size_t i = w; i < tasks.size(); i += workers) {
                            if (done[i]) { continue; }
                            tasks[i]->poll();
                            if (tasks[i]->finished()) {
                                done[i] = true;
                                --left;
                                progressed = true;
                            }
                        }
                        if (!progressed) { std::this_thread::yield(); }
                    }
                } catch (...) {
                    failed.store(true);
                    throw;
                }
            });
        }
        pool_->par(std::move(fs));
    }
};
}  // namespace

size_t task_count() { return g_tasks.load(); }

std::string demangled(const std::type_info &ti)
{
    int status = 0;
    char *s = abi::__cxa_demangle(ti.name(), nullptr, nullptr, &status);
    std::string out = (status == 0 && s != nullptr) ? s : ti.name();
    std::free(s);
    return out;
}

runtime *runtime::New(size_t m) { return new pool_runtime(m); }

task::task() { ++g_tasks; }

void task::finish()
{
    while (!finished()) {
        poll();
        if (!finished()) { std::this_thread::yield(); }
    }
}

task *task::par(std::vector<std::unique_ptr<task>> tasks, runtime *rt)
{
    return new parallel_tasks(std::move(tasks), rt);
}

task *task::seq(std::vector<std::unique_ptr<task>> tasks)
{
    return new sequence_tasks(std::move(tasks));
}

void simple_task::poll()
{
    if (!done_) {
        f_();
        done_ = true;
    }
}

void poll_task::poll()
{
    if (!done_ && ready_()) {
        if (then_) { then_(); }
        done_ = true;
    }
}

void sequence_tasks::poll()
{
    while (next_ < tasks_.size()) {
        task &t = *tasks_[next_];
        if (!t.finished()) { t.poll(); }
        if (!t.finished()) { return; }
        ++next_;
    }
}

bool sequence_tasks::finished()
{
    while (next_ < tasks_.size() && tasks_[next_]->finished()) { ++next_; }
    return next_ == tasks_.size();
}

parallel_tasks::parallel_tasks(std::vector<std::unique_ptr<task>> tasks, runtime *rt)
    : tasks_(std::move(tasks)), done_(tasks_.size(), false), remaining_(tasks_.size()), rt_(rt)
{
}

void parallel_tasks::poll()
{
    if (remaining_ == 0) { return; }
    if (rt_ != nullptr) {
        rt_->par(tasks_);
        remaining_ = 0;
        return;
    }
    for (size_t i = 0; i < tasks_.size(); ++i) {
        if (done_[i]) { continue; }
        tasks_[i]->poll();
        if (tasks_[i]->finished()) {
            done_[i] = true;
            --remaining_;
        }
    }
}
}  // namespace stdml::collective
