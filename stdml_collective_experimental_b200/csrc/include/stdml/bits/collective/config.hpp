// Process-wide settings, read once from the environment.  Variable names and
// truthy spellings (true|on|1, any case) are the reference's
// (src/stdml/collective/config.cpp:11-34, env.cpp:28-40); the entries below the
// line are new (device path).
#pragma once
#include <cstddef>
#include <cstdint>
#include <optional>
#include <ostream>
#include <string>

namespace stdml::collective
{
enum runtime_type {
    rt_multi_thread,  // a thread per graph edge
    rt_thread_pool,   // the same work items on a fixed pool
    rt_async,         // polled task tree
    rt_coro,          // accepted, runs as rt_async
    rt_go,            // accepted, runs as rt_thread_pool (no external Go runtime here)
};

struct system_config {
    runtime_type rt = rt_multi_thread;
    size_t thread_pool_size = 0;
    bool use_affinity = false;
    // ---- device path
    std::string device_algo = "auto";  // STDML_COLLECTIVE_ALGO: auto|oneshot|twoshot|nvls
    int64_t timeout_ms = 20000;        // STDML_COLLECTIVE_TIMEOUT_MS
    bool use_nvls = true;              // STDML_COLLECTIVE_NVLS
    // ---- failure detection on the host path: how long a collective waits for a
    // peer's message before it throws (0 = for ever, as the reference does)
    int64_t host_timeout_ms = 0;       // STDML_COLLECTIVE_HOST_TIMEOUT_MS
    // ---- members on several hosts: reduce inside each host, all-reduce among one
    // leader per host, broadcast inside each host (always for device buffers)
    bool hierarchical = false;         // STDML_COLLECTIVE_HIERARCHICAL
};

std::ostream &operator<<(std::ostream &os, const system_config &c);
const char *runtime_name(runtime_type rt);

system_config parse_system_config_from_env();

// environment helpers
std::string safe_getenv(const char *name);  // "" when unset
bool parse_env_bool(const char *name);      // true|on|1, case-insensitive
std::optional<int64_t> parse_env_int(const char *name);
}  // namespace stdml::collective
