// Implementation of stdmlc_all_reduce_noalloc (see noalloc_all_reduce.h for the
// contract).  The scratch array below is a file-scope device variable: in host
// code its name is only a handle for the runtime, not a device address, so the
// address is obtained once per device with cudaGetSymbolAddress and that
// pointer is what the kernel receives.
#include <cstring>
#include <mutex>
#include <string>

#include <cuda_runtime.h>

#include "comm.cuh"
#include "noalloc_all_reduce.h"

extern "C" const char *stdmlc_last_error();

namespace stdml::collective::cuda
{
void set_last_error(const std::string &msg);  // capi_cuda.cpp

namespace
{
constexpr size_t kRegionBytes = kDataOffset + STDMLC_NOALLOC_MAX_BYTES;  // pad + staging
static_assert(STDMLC_NOALLOC_SCRATCH_BYTES == STDMLC_NOALLOC_MAX_RANKS * kRegionBytes,
              "scratch layout: one (signal pad, staging) region per rank");
static_assert(kRegionBytes % 256 == 0, "regions keep the array's alignment");

// Signal pads and staging of every emulated rank.  Held by every GPU that
// loads this module until the process exits.
static __device__ __align__(256) unsigned char g_noalloc_scratch[STDMLC_NOALLOC_SCRATCH_BYTES];
// Where a kernel records a wait that ran out (device memory: nothing here may
// allocate pinned host memory either).
static __device__ StatusBlock g_noalloc_status;

constexpr int kMaxDevices = 64;
std::mutex g_mu;
unsigned char *g_scratch_ptr[kMaxDevices];
StatusBlock *g_status_ptr[kMaxDevices];
int g_sms[kMaxDevices];

int fail(int code, const std::string &msg)
{
    set_last_error(msg);
    return code;
}

// Once per device, with that device current.
int setup_device(int dev)
{
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_scratch_ptr[dev] != nullptr) { return 0; }
    void *scratch = nullptr;
    void *status = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&scratch, g_noalloc_scratch);
    if (e == cudaSuccess) { e = cudaGetSymbolAddress(&status, g_noalloc_status); }
    int sms = 0;
    if (e == cudaSuccess) { e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return fail(1, std::string("stdmlc_all_reduce_noalloc: device set-up failed: ") +
                           cudaGetErrorString(e));
    }
    g_status_ptr[dev] = static_cast<StatusBlock *>(status);
    g_sms[dev] = sms;
    g_scratch_ptr[dev] = static_cast<unsigned char *>(scratch);
    return 0;
}
}  // namespace
}  // namespace stdml::collective::cuda

using namespace stdml::collective::cuda;

// Copies the device-resident status block back to the host: one asynchronous
// copy into the caller's own array and a wait for `stream`.  Nothing allocates.
extern "C" int stdmlc_all_reduce_noalloc_status(int *out7, void *stream)
{
    if (out7 == nullptr) { return fail(2, "stdmlc_all_reduce_noalloc_status: null output"); }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        (void)cudaGetLastError();
        return fail(1, "stdmlc_all_reduce_noalloc_status: no current CUDA device");
    }
    for (int i = 0; i < 7; ++i) { out7[i] = 0; }
    if (g_status_ptr[dev] == nullptr) { return 0; }  // never called on this device: healthy
    StatusBlock st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(&st, g_status_ptr[dev], sizeof(st), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) { e = cudaStreamSynchronize(s); }
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return fail(1, std::string("stdmlc_all_reduce_noalloc_status: ") + cudaGetErrorString(e));
    }
    out7[0] = st.code;
    out7[1] = st.rank;
    out7[2] = st.block;
    out7[3] = st.peer;
    out7[4] = st.phase;
    out7[5] = static_cast<int>(st.want);
    out7[6] = static_cast<int>(st.have);
    if (st.code == kStatusTimeout) {
        return fail(4, "stdmlc_all_reduce_noalloc: a bounded wait of the last call ran out "
                       "(two calls overlapping on the GPU?); its outputs are incomplete");
    }
    return st.code == kStatusOk ? 0 : fail(1, "stdmlc_all_reduce_noalloc: the last call failed");
}

extern "C" int stdmlc_all_reduce_noalloc(const void *const *in, void *const *out, int nranks,
                                         unsigned long long count, int dt, int op, double scale,
                                         void *stream)
{
    static const size_t sizes[12] = {1, 2, 4, 8, 1, 2, 4, 8, 2, 2, 4, 8};
    if (in == nullptr || out == nullptr) {
        return fail(2, "stdmlc_all_reduce_noalloc: null pointer table");
    }
    if (nranks < 1 || nranks > STDMLC_NOALLOC_MAX_RANKS) {
        return fail(2, "stdmlc_all_reduce_noalloc: nranks must be in [1, " +
                           std::to_string(STDMLC_NOALLOC_MAX_RANKS) + "]");
    }
    if (dt < 0 || dt > 11 || op < 0 || op > 4 || (op == 4 && dt >= 8)) {
        return fail(2, "stdmlc_all_reduce_noalloc: undefined (dtype, op) pair");
    }
    const unsigned long long bytes = count * sizes[dt];
    if (count > STDMLC_NOALLOC_MAX_BYTES || bytes > STDMLC_NOALLOC_MAX_BYTES) {
        return fail(2, "stdmlc_all_reduce_noalloc: " + std::to_string(bytes) +
                           " bytes per buffer exceed the fixed scratch (" +
                           std::to_string(STDMLC_NOALLOC_MAX_BYTES) +
                           " bytes); use a device session for larger messages");
    }
    for (int r = 0; r < nranks; ++r) {
        if (in[r] == nullptr || out[r] == nullptr) {
            return fail(2, "stdmlc_all_reduce_noalloc: null buffer for rank " + std::to_string(r));
        }
    }
    if (count == 0) { return 0; }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        (void)cudaGetLastError();
        return fail(1, "stdmlc_all_reduce_noalloc: no current CUDA device");
    }
    if (const int rc = setup_device(dev); rc != 0) { return rc; }
    unsigned char *scratch = g_scratch_ptr[dev];
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    // The signal pads must start from zero: the previous call (or a call that
    // gave up) may have left any epoch in them.
    cudaError_t e = cudaSuccess;
    for (int r = 0; r < nranks && e == cudaSuccess; ++r) {
        e = cudaMemsetAsync(scratch + r * kRegionBytes, 0, sizeof(SignalPad), s);
    }
    if (e == cudaSuccess) { e = cudaMemsetAsync(g_status_ptr[dev], 0, sizeof(StatusBlock), s); }
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return fail(1, std::string("stdmlc_all_reduce_noalloc: memset failed: ") +
                           cudaGetErrorString(e));
    }

    CommCtx ctx;
    std::memset(&ctx, 0, sizeof(ctx));
    for (int r = 0; r < nranks; ++r) { ctx.base[r] = reinterpret_cast<char *>(scratch + r * kRegionBytes); }
    ctx.status = g_status_ptr[dev];
    ctx.timeout_ns = 2000000000ull;
    ctx.max_spins = 1u << 28;
    ctx.world = nranks;
    ctx.rank = 0;

    AllReduceArgs a;
    std::memset(&a, 0, sizeof(a));
    for (int r = 0; r < nranks; ++r) {
        a.src[r] = in[r];
        a.dst[r] = out[r];
    }
    for (int r = 0; r < nranks; ++r) { a.data[r] = a.push[r] = ctx.base[r] + kDataOffset; }
    a.off = kDataOffset;
    a.count = count;
    a.nvec = (bytes + 15) / 16;
    a.algo = kAlgoOneShot;
    a.user_dtype = dt;
    a.root = -1;
    a.has_scale = scale != 1.0 ? 1 : 0;
    a.scale = scale;
    a.phases = kPhaseAll;

    // all rows of the grid wait on one another: they must be resident together
    const unsigned long long per_block = static_cast<unsigned long long>(kThreads) * 4;
    unsigned long long blocks = (a.nvec + per_block - 1) / per_block;
    const unsigned long long cap = static_cast<unsigned long long>(g_sms[dev] / nranks);
    if (blocks > cap) { blocks = cap; }
    if (blocks < 1) { blocks = 1; }
    const int rc = launch_all_reduce(ctx, a, dt, op, static_cast<int>(blocks), nranks, stream);
    if (rc != 0) {
        (void)cudaGetLastError();
        return fail(1, std::string("stdmlc_all_reduce_noalloc: launch failed: ") +
                           (rc > 0 ? cudaGetErrorString(static_cast<cudaError_t>(rc))
                                   : "kernel not built"));
    }
    return 0;
}
