// Polled task trees: the async runtime of the library.  A task makes progress
// only when poll()ed and never blocks; seq/par compose tasks; finish() polls
// to completion on the calling thread; runtime::par spreads the children of a
// parallel node over worker threads.  Same API as the reference
// (include/stdml/bits/collective/task.hpp:26-190; usage contract:
// examples/example-task.cpp).  The device path uses the same interface to
// wait for CUDA events without blocking a thread (see event_task in
// stdml/bits/collective/device.hpp).
#pragma once
#include <atomic>
#include <chrono>
#include <cstddef>
#include <functional>
#include <memory>
#include <string>
#include <typeinfo>
#include <utility>
#include <vector>

#include <stdml/bits/collective/log.hpp>
#include <stdml/bits/collective/stat.hpp>

namespace stdml::collective
{
class task;

class runtime
{
  public:
    virtual ~runtime() = default;
    // m worker threads
    static runtime *New(size_t m);
    // runs every task to completion; returns when all have finished
    virtual void par(std::vector<std::unique_ptr<task>> &tasks) = 0;
};

// number of task objects constructed so far in this process
size_t task_count();

std::string demangled(const std::type_info &ti);

template <typename T>
std::string task_name()
{
    return demangled(typeid(T));
}

class task
{
  public:
    task();
    virtual ~task() = default;

    virtual void poll() = 0;
    virtual bool finished() = 0;

    // poll until finished (spins; yields the CPU between rounds)
    void finish();

    static task *par(std::vector<std::unique_ptr<task>> tasks, runtime *rt = nullptr);
    static task *seq(std::vector<std::unique_ptr<task>> tasks);

    template <typename F, typename L>
    static std::vector<std::unique_ptr<task>> fmap(const F &f, const L &xs)
    {
        std::vector<std::unique_ptr<task>> ts;
        for (const auto &x : xs) { ts.emplace_back(f(x)); }
        return ts;
    }
};

class noop_task : public task
{
  public:
    void poll() override {}
    bool finished() override { return true; }
};

// runs f once, on the first poll
class simple_task : public task
{
    std::function<void()> f_;
    bool done_ = false;

  public:
    explicit simple_task(std::function<void()> f) : f_(std::move(f)) {}
    void poll() override;
    bool finished() override { return done_; }
};

// polls `ready` until it returns true, then runs `then` once
class poll_task : public task
{
    std::function<bool()> ready_;
    std::function<void()> then_;
    bool done_ = false;

  public:
    explicit poll_task(std::function<bool()> ready, std::function<void()> then = {})
        : ready_(std::move(ready)), then_(std::move(then))
    {
    }
    void poll() override;
    bool finished() override { return done_; }
};

class sequence_tasks : public task
{
    std::vector<std::unique_ptr<task>> tasks_;
    size_t next_ = 0;

  public:
    explicit sequence_tasks(std::vector<std::unique_ptr<task>> tasks) : tasks_(std::move(tasks)) {}
    void poll() override;
    bool finished() override;
};

class parallel_tasks : public task
{
    std::vector<std::unique_ptr<task>> tasks_;
    std::vector<bool> done_;
    size_t remaining_;
    runtime *rt_;

  public:
    explicit parallel_tasks(std::vector<std::unique_ptr<task>> tasks, runtime *rt = nullptr);
    void poll() override;
    bool finished() override { return remaining_ == 0; }
};

// wraps a task and logs how often it was polled and how long it lived
template <typename Task>
class monitored_task : public task
{
    using clock = std::chrono::steady_clock;
    Task inner_;
    size_t polls_ = 0;
    clock::time_point t0_ = clock::now();

  public:
    explicit monitored_task(Task t) : inner_(std::move(t)) {}

    ~monitored_task() override
    {
        if (log_enabled()) {
            const std::chrono::duration<double> d = clock::now() - t0_;
            log() << "polled" << polls_ << "times | took" << rchan::show_duration(d) << "| @"
                  << task_name<Task>();
        }
    }

    void poll() override
    {
        ++polls_;
        inner_.poll();
    }

    bool finished() override { return inner_.finished(); }
};

class task_builder
{
    std::vector<std::unique_ptr<task>> tasks_;

  public:
    void operator<<(task *t) { tasks_.emplace_back(t); }
    void operator<<(std::unique_ptr<task> t) { tasks_.emplace_back(std::move(t)); }
    size_t size() const { return tasks_.size(); }
    task *par(runtime *rt = nullptr) { return task::par(std::move(tasks_), rt); }
    task *seq() { return task::seq(std::move(tasks_)); }
};
}  // namespace stdml::collective
