#include <cuda_runtime.h>

#include <stdml/bits/collective/device.hpp>

#include "device_world.hpp"

namespace stdml::collective
{
bool device_available() { return cuda::cuda_available(); }
int device_count() { return cuda::cuda_device_count(); }

event_task::event_task(void *stream) : event_(nullptr)
{
    cudaEvent_t e = nullptr;
    if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventRecord(e, static_cast<cudaStream_t>(stream)) != cudaSuccess) {
        (void)cudaGetLastError();
        failed_ = true;
        done_ = true;
    }
    event_ = e;
}

event_task::~event_task()
{
    if (event_ != nullptr) { (void)cudaEventDestroy(static_cast<cudaEvent_t>(event_)); }
}

void event_task::poll()
{
    if (done_) { return; }
    const cudaError_t st = cudaEventQuery(static_cast<cudaEvent_t>(event_));
    if (st == cudaSuccess) {
        done_ = true;
    } else if (st != cudaErrorNotReady) {
        (void)cudaGetLastError();
        failed_ = true;
        done_ = true;
    }
}
}  // namespace stdml::collective
