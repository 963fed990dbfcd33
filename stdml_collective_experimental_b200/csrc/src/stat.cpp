#include <cstdio>
#include <fstream>
#include <functional>
#include <iostream>
#include <mutex>
#include <sstream>
#include <thread>

#include <stdml/bits/collective/config.hpp>
#include <stdml/bits/collective/json.hpp>
#include <stdml/bits/collective/log.hpp>
#include <stdml/bits/collective/stat.hpp>

namespace stdml::collective::rchan
{
namespace
{
struct table {
    std::atomic<int> on{parse_env_bool("STDML_COLLECTIVE_ENABLE_TRACE") ? 1 : 0};
    std::mutex mu;
    std::vector<stat_event> events;
    const stat_clock::time_point start = stat_clock::now();

    table() { events.reserve(1 << 16); }

    ~table()
    {
        if (!events.empty() && on.load() != 0) { dump(std::cout); }
    }

    void dump(std::ostream &os)
    {
        std::lock_guard<std::mutex> lk(mu);
        for (const auto &e : events) {
            const double ms = (e.t1 - e.t0) * 1e3;
            char line[512];
            const double gbs = e.t1 > e.t0 ? e.payload / (e.t1 - e.t0) / 1e9 : 0.0;
            std::snprintf(line, sizeof(line), "`` %s %llu %.9f %.9f %.6fms %zu %.3fGB/s\n",
                          e.name.c_str(), static_cast<unsigned long long>(e.thread), e.t0, e.t1,
                          ms, e.payload, gbs);
            os << line;
        }
    }
};

table &tab()
{
    static table t;
    return t;
}

double since_start(stat_clock::time_point t)
{
    return std::chrono::duration<double>(t - tab().start).count();
}
}  // namespace

void stat_enable() { tab().on.store(1); }
void stat_disable() { tab().on.store(0); }
bool stat_enabled() { return tab().on.load(std::memory_order_relaxed) != 0; }

void stat_record(const char *name, stat_clock::time_point t0, stat_clock::time_point t1,
                 size_t payload)
{
    table &t = tab();
    stat_event e;
    e.name = name;
    e.thread = std::hash<std::thread::id>()(std::this_thread::get_id()) % 1000000;
    e.t0 = since_start(t0);
    e.t1 = since_start(t1);
    e.payload = payload;
    std::lock_guard<std::mutex> lk(t.mu);
    t.events.push_back(std::move(e));
}

std::vector<stat_event> stat_events()
{
    table &t = tab();
    std::lock_guard<std::mutex> lk(t.mu);
    return t.events;
}

void stat_clear()
{
    table &t = tab();
    std::lock_guard<std::mutex> lk(t.mu);
    t.events.clear();
}

void stat_report(std::ostream &os) { tab().dump(os); }

bool stat_write_chrome_trace(const std::string &path)
{
    std::ofstream f(path);
    if (!f) { return false; }
    f << "{\"traceEvents\":[";
    bool first = true;
    for (const auto &e : stat_events()) {
        if (!first) { f << ","; }
        first = false;
        f << "{\"name\":" << json::quote(e.name) << ",\"ph\":\"X\",\"pid\":0,\"tid\":" << e.thread
          << ",\"ts\":" << static_cast<long long>(e.t0 * 1e6)
          << ",\"dur\":" << static_cast<long long>((e.t1 - e.t0) * 1e6)
          << ",\"args\":{\"bytes\":" << e.payload << "}}";
    }
    f << "]}\n";
    return static_cast<bool>(f);
}

std::string show_duration(std::chrono::duration<double> d)
{
    const double s = d.count();
    char buf[64];
    if (s < 1e-6) {
        std::snprintf(buf, sizeof(buf), "%6.4gns", s * 1e9);
    } else if (s < 1e-3) {
        std::snprintf(buf, sizeof(buf), "%6.4gus", s * 1e6);
    } else if (s < 1) {
        std::snprintf(buf, sizeof(buf), "%6.4gms", s * 1e3);
    } else {
        std::snprintf(buf, sizeof(buf), "%6.4gs", s);
    }
    return buf;
}

std::string show_rate(double gib_per_s)
{
    char buf[96];
    std::snprintf(buf, sizeof(buf), "%.3f GiB/s (%.3f MiB/s)", gib_per_s, gib_per_s * 1024.0);
    return buf;
}

std::string show_size(size_t bytes)
{
    char buf[64];
    const double b = static_cast<double>(bytes);
    if (bytes < (1u << 10)) {
        std::snprintf(buf, sizeof(buf), "%zu B", bytes);
    } else if (bytes < (1u << 20)) {
        std::snprintf(buf, sizeof(buf), "%.2f KiB", b / 1024.0);
    } else if (bytes < (1u << 30)) {
        std::snprintf(buf, sizeof(buf), "%.2f MiB", b / 1048576.0);
    } else {
        std::snprintf(buf, sizeof(buf), "%.2f GiB", b / 1073741824.0);
    }
    return buf;
}

rate_scope::rate_scope(site_context &site, size_t bytes)
    : site_(site), bytes_(bytes), t0_(stat_clock::now())
{
}

rate_scope::~rate_scope()
{
    const std::chrono::duration<double> d = stat_clock::now() - t0_;
    const uint64_t n = ++site_.calls;
    const double gib = d.count() > 0 ? bytes_ / d.count() / 1073741824.0 : 0.0;
    log(PRINT) << "#" << n << " | rate:" << show_rate(gib) << " | took:" << show_duration(d)
               << "  @" << site_.name;
}

latency_scope::latency_scope(site_context &site) : site_(site), t0_(stat_clock::now()) {}

latency_scope::~latency_scope()
{
    const std::chrono::duration<double> d = stat_clock::now() - t0_;
    const uint64_t n = ++site_.calls;
    log(PRINT) << "#" << n << " | took:" << show_duration(d) << "  @" << site_.name;
}
}  // namespace stdml::collective::rchan
