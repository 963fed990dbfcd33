// C ABI of the device data plane (loaded from Python with ctypes, usable from
// C).  Every function returns 0 on success and a non-zero code on failure;
// stdmlc_last_error() then holds the message (thread-local).
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>

#include "capi_cuda.h"
#include "device_session.hpp"

using namespace stdml::collective::cuda;

namespace
{
thread_local std::string g_error;

template <typename F>
int guarded(F f)
{
    try {
        f();
        return 0;
    } catch (const DeviceTimeout &e) {
        g_error = e.what();
        return STDMLC_ERR_TIMEOUT;
    } catch (const std::invalid_argument &e) {
        g_error = e.what();
        return STDMLC_ERR_ARGS;
    } catch (const std::bad_alloc &) {
        g_error = "symmetric heap exhausted";
        return STDMLC_ERR_NOMEM;
    } catch (const std::exception &e) {
        g_error = e.what();
        return STDMLC_ERR_RUNTIME;
    } catch (...) {  // nothing may unwind through the C boundary
        g_error = "unknown C++ exception";
        return STDMLC_ERR_RUNTIME;
    }
}

DeviceSession *S(void *h)
{
    if (h == nullptr) { throw std::invalid_argument("null device session handle"); }
    return static_cast<DeviceSession *>(h);
}
}  // namespace

namespace stdml::collective::cuda
{
void set_last_error(const std::string &msg) { g_error = msg; }
}  // namespace stdml::collective::cuda

extern "C" {
const char *stdmlc_last_error() { return g_error.c_str(); }

int stdmlc_cuda_device_count() { return cuda_device_count(); }

int stdmlc_pointer_kind(const void *p) { return pointer_kind(p); }

int stdmlc_dw_create(void **out, int rank, int world, int device, int loopback,
                     unsigned long long heap_bytes, unsigned long long staging_bytes,
                     const char *key, const char *backend, int enable_nvls, int setup_timeout_ms,
                     unsigned long long wait_timeout_ms)
{
    *out = nullptr;
    return guarded([&] {
        DeviceWorldOptions o;
        o.rank = rank;
        o.world = world;
        o.device = device;
        o.loopback = loopback != 0;
        o.heap_bytes = heap_bytes;
        o.staging_bytes = staging_bytes;
        if (key != nullptr) { o.key = key; }
        if (backend != nullptr && backend[0] != 0) { o.backend = backend; }
        o.enable_nvls = enable_nvls != 0;
        if (setup_timeout_ms > 0) { o.setup_timeout_ms = setup_timeout_ms; }
        if (wait_timeout_ms > 0) { o.wait_timeout_ms = wait_timeout_ms; }
        *out = new DeviceSession(DeviceWorld::create(o));
    });
}

int stdmlc_dw_destroy(void *h)
{
    return guarded([&] { delete static_cast<DeviceSession *>(h); });  // null is a no-op, as for free()
}

int stdmlc_dw_info(void *h, int what, unsigned long long *out)
{
    return guarded([&] {
        DeviceWorld &w = S(h)->world();
        switch (what) {
        case STDMLC_INFO_RANK:
            *out = w.rank();
            break;
        case STDMLC_INFO_WORLD:
            *out = w.world();
            break;
        case STDMLC_INFO_VRANKS:
            *out = w.vranks();
            break;
        case STDMLC_INFO_HAS_NVLS:
            *out = w.has_nvls() ? 1 : 0;
            break;
        case STDMLC_INFO_ARENA_BYTES:
            *out = w.arena_bytes();
            break;
        case STDMLC_INFO_STAGING_BYTES:
            *out = w.staging_bytes();
            break;
        case STDMLC_INFO_LAUNCHES:
            *out = S(h)->launches();
            break;
        case STDMLC_INFO_BACKEND:
            *out = std::strcmp(w.backend(), "vmm") == 0   ? 1
                   : std::strcmp(w.backend(), "ipc") == 0 ? 2
                                                          : 0;
            break;
        default:
            throw std::invalid_argument("stdmlc_dw_info: unknown item");
        }
    });
}

int stdmlc_dw_alloc(void *h, unsigned long long bytes, unsigned long long *off)
{
    return guarded([&] { *off = S(h)->world().alloc(bytes); });
}

int stdmlc_dw_release(void *h, unsigned long long off)
{
    return guarded([&] { S(h)->world().release(off); });
}

int stdmlc_dw_ptr(void *h, int rank, unsigned long long off, void **out)
{
    return guarded([&] { *out = S(h)->world().ptr(rank, off); });
}

int stdmlc_dw_mc_ptr(void *h, unsigned long long off, void **out)
{
    return guarded([&] { *out = S(h)->world().mc_ptr(off); });
}

int stdmlc_dw_set_tuning(void *h, int max_blocks, long long oneshot_max_bytes,
                         long long nvls_oneshot_max_bytes, long long wait_timeout_ms)
{
    return guarded([&] {
        S(h)->world().set_tuning(
            max_blocks, oneshot_max_bytes < 0 ? SIZE_MAX : static_cast<size_t>(oneshot_max_bytes),
            nvls_oneshot_max_bytes < 0 ? SIZE_MAX : static_cast<size_t>(nvls_oneshot_max_bytes));
        if (wait_timeout_ms > 0) {
            S(h)->world().set_wait_timeout_ms(static_cast<unsigned long long>(wait_timeout_ms));
        }
    });
}

int stdmlc_dw_set_knob(void *h, const char *name, long long value)
{
    return guarded([&] { S(h)->set_knob(name != nullptr ? name : "", value); });
}

int stdmlc_dw_drop_registrations(void *h)
{
    return guarded([&] { S(h)->drop_registrations(); });
}

int stdmlc_dw_all_reduce(void *h, const void *const *in, void *const *out,
                         unsigned long long count, int dt, int op, double scale, int algo,
                         void *stream)
{
    return guarded([&] { S(h)->all_reduce(in, out, count, dt, op, scale, algo, stream); });
}

int stdmlc_dw_reduce(void *h, const void *const *in, void *const *out, unsigned long long count,
                     int dt, int op, int root, double scale, void *stream)
{
    return guarded([&] { S(h)->reduce(in, out, count, dt, op, root, scale, stream); });
}

int stdmlc_dw_group_all_reduce(void *h, unsigned long long n, const void *const *ins,
                               void *const *outs, const unsigned long long *counts, int dt, int op,
                               int user_dt, double scale, int algo, void *stream)
{
    static_assert(sizeof(unsigned long long) == sizeof(size_t), "LP64 expected");
    return guarded([&] {
        S(h)->group_all_reduce(n, ins, outs, reinterpret_cast<const size_t *>(counts), dt, op,
                               user_dt, scale, algo, stream);
    });
}

int stdmlc_dw_all_gather(void *h, const void *const *in, void *const *out,
                         unsigned long long count, int dt, void *stream)
{
    return guarded([&] { S(h)->all_gather(in, out, count, dt, stream); });
}

int stdmlc_dw_broadcast(void *h, const void *const *in, void *const *out,
                        unsigned long long count, int dt, int root, void *stream)
{
    return guarded([&] { S(h)->broadcast(in, out, count, dt, root, stream); });
}

int stdmlc_dw_barrier(void *h, void *stream)
{
    return guarded([&] { S(h)->barrier(stream); });
}

int stdmlc_dw_barrier_rows(void *h, int rows, void *stream)
{
    return guarded([&] {
        const int rc = S(h)->world().barrier_rows(rows, stream);
        if (rc != 0) { throw std::runtime_error("launch failed: cudaError " + std::to_string(rc)); }
    });
}

int stdmlc_dw_raw_all_reduce(void *h, unsigned long long off, const void *const *src,
                             void *const *dst, unsigned long long count, int dt, int op, int algo,
                             int blocks, int root, int end_barrier, int has_scale, double scale,
                             void *stream)
{
    return guarded([&] {
        AllReduceCall c;
        c.off = off;
        c.src = src;
        c.dst = dst;
        c.count = count;
        c.dt = dt;
        c.op = op;
        c.algo = algo;
        c.blocks = blocks;
        c.root = root;
        c.end_barrier = end_barrier != 0;
        c.has_scale = has_scale != 0;
        c.scale = scale;
        const int rc = S(h)->world().all_reduce(c, stream);
        if (rc != 0) { throw std::runtime_error("launch failed: cudaError " + std::to_string(rc)); }
    });
}

int stdmlc_dw_status(void *h, int *out7)
{
    return guarded([&] {
        const DeviceStatus s = S(h)->world().poll_status();
        out7[0] = s.code;
        out7[1] = s.rank;
        out7[2] = s.block;
        out7[3] = s.peer;
        out7[4] = s.phase;
        out7[5] = static_cast<int>(s.want);
        out7[6] = static_cast<int>(s.have);
    });
}

int stdmlc_dw_check(void *h)
{
    return guarded([&] { S(h)->check(); });
}

int stdmlc_dw_recover(void *h)
{
    return guarded([&] { S(h)->world().recover(); });
}
}
