#include <algorithm>
#include <cctype>
#include <cstdlib>
#include <thread>

#include <stdml/bits/collective/config.hpp>

namespace stdml::collective
{
std::string safe_getenv(const char *name)
{
    const char *v = std::getenv(name);
    return v == nullptr ? std::string() : std::string(v);
}

bool parse_env_bool(const char *name)
{
    std::string v = safe_getenv(name);
    std::transform(v.begin(), v.end(), v.begin(),
                   [](unsigned char c) { return static_cast<char>(std::tolower(c)); });
    return v == "true" || v == "on" || v == "1";
}

std::optional<int64_t> parse_env_int(const char *name)
{
    const std::string v = safe_getenv(name);
    if (v.empty()) { return {}; }
    char *end = nullptr;
    const long long n = std::strtoll(v.c_str(), &end, 10);
    if (end == v.c_str() || *end != '\0') { return {}; }
    return n;
}

const char *runtime_name(runtime_type rt)
{
    switch (rt) {
    case rt_multi_thread:
        return "rt_multi_thread";
    case rt_thread_pool:
        return "rt_thread_pool";
    case rt_async:
        return "rt_async";
    case rt_coro:
        return "rt_coro";
    case rt_go:
        return "rt_go";
    }
    return "rt_unknown";
}

std::ostream &operator<<(std::ostream &os, const system_config &c)
{
    os << "runtime: " << runtime_name(c.rt);
    if (c.thread_pool_size > 0) { os << ", pool: " << c.thread_pool_size; }
    if (c.use_affinity) { os << ", affinity"; }
    return os;
}

system_config parse_system_config_from_env()
{
    system_config c;
    const size_t cores = std::max(1u, std::thread::hardware_concurrency());
    if (parse_env_bool("STDML_COLLECTIVE_USE_THREAD_POOL")) {
        c.rt = rt_thread_pool;
        c.thread_pool_size = cores;
    }
    if (parse_env_bool("STDML_COLLECTIVE_USE_ASYNC")) { c.rt = rt_async; }
    if (parse_env_bool("STDML_COLLECTIVE_USE_GO_RUNTIME")) {
        c.rt = rt_go;
        c.thread_pool_size = cores;
    }
    if (const auto n = parse_env_int("STDML_COLLECTIVE_THREAD_POOL_SIZE"); n && *n > 0) {
        c.thread_pool_size = static_cast<size_t>(*n);
    }
    c.use_affinity = parse_env_bool("STDML_COLLECTIVE_USE_AFFINITY");
    const std::string algo = safe_getenv("STDML_COLLECTIVE_ALGO");
    if (!algo.empty()) { c.device_algo = algo; }
    if (const auto t = parse_env_int("STDML_COLLECTIVE_TIMEOUT_MS"); t && *t > 0) {
        c.timeout_ms = *t;
    }
    if (const auto t = parse_env_int("STDML_COLLECTIVE_HOST_TIMEOUT_MS"); t && *t > 0) {
        c.host_timeout_ms = *t;
    }
    c.hierarchical = parse_env_bool("STDML_COLLECTIVE_HIERARCHICAL");
    const std::string nvls = safe_getenv("STDML_COLLECTIVE_NVLS");
    if (nvls == "0" || nvls == "off" || nvls == "false") { c.use_nvls = false; }
    return c;
}
}  // namespace stdml::collective
