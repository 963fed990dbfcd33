// Device-side helpers of the public API that need no CUDA headers:
//   event_task   a polled task that finishes when a CUDA event has completed,
//                so device collectives compose with the task runtime
//                (seq / par trees, runtime::par) without blocking a thread;
//   device_available / device_count.
// The reference has no device path (README:9 lists it as a TODO).
#pragma once
#include <memory>

#include <stdml/bits/collective/task.hpp>

namespace stdml::collective
{
bool device_available();
int device_count();

class event_task : public task
{
    void *event_;  // cudaEvent_t, owned
    bool done_ = false;
    bool failed_ = false;

  public:
    // records a new event on `stream` (nullptr: the legacy default stream)
    explicit event_task(void *stream);
    ~event_task() override;
    void poll() override;
    bool finished() override { return done_; }
    bool failed() const { return failed_; }
};
}  // namespace stdml::collective
