// Rank-local tracing and metrics.
//   * event table: {name, thread, t0, t1, payload bytes}; recorded by RAII
//     scopes when tracing is on (STDML_COLLECTIVE_ENABLE_TRACE or stat_enable()).
//     At exit (or on stat_report()) each event is printed as a line starting
//     with two back-ticks: name, thread, t0, t1, ms, payload, GB/s -- the format
//     the reference prints (src/stdml/collective/stat.cpp:27-58) so its timeline
//     scripts keep working -- and stat_write_chrome_trace() writes the same
//     events as Chrome trace JSON.
//   * rate / latency scope loggers with the reference's macro names
//     (include/stdml/bits/collective/stat.hpp:121-218).
// Unlike the reference, the profile macro is not compiled out: it costs one
// relaxed atomic load when tracing is off.
#pragma once
#include <atomic>
#include <chrono>
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace stdml::collective::rchan
{
using stat_clock = std::chrono::steady_clock;

struct stat_event {
    std::string name;
    uint64_t thread;
    double t0, t1;  // seconds since process start
    size_t payload;
};

void stat_enable();
void stat_disable();
bool stat_enabled();
void stat_record(const char *name, stat_clock::time_point t0, stat_clock::time_point t1,
                 size_t payload);
std::vector<stat_event> stat_events();
void stat_clear();
void stat_report(std::ostream &os);
bool stat_write_chrome_trace(const std::string &path);

std::string show_duration(std::chrono::duration<double> d);
std::string show_rate(double gib_per_s);
std::string show_size(size_t bytes);

// records [construction, destruction) under `name` when tracing is enabled
class scope
{
    const char *name_;
    size_t payload_;
    bool on_;
    stat_clock::time_point t0_;

  public:
    scope(const char *name, size_t payload = 0)
        : name_(name), payload_(payload), on_(stat_enabled())
    {
        if (on_) { t0_ = stat_clock::now(); }
    }
    ~scope()
    {
        if (on_) { stat_record(name_, t0_, stat_clock::now(), payload_); }
    }
};

// per call-site counters behind LOG_SCOPE_RATE / LOG_SCOPE_LATENCY
struct site_context {
    const char *name;
    std::atomic<uint64_t> calls{0};
    explicit site_context(const char *n) : name(n) {}
};

class rate_scope
{
    site_context &site_;
    size_t bytes_;
    stat_clock::time_point t0_;

  public:
    rate_scope(site_context &site, size_t bytes);
    ~rate_scope();
};

class latency_scope
{
    site_context &site_;
    stat_clock::time_point t0_;

  public:
    explicit latency_scope(site_context &site);
    ~latency_scope();
};
}  // namespace stdml::collective::rchan

#define STDML_CAT_(a, b) a##b
#define STDML_CAT(a, b) STDML_CAT_(a, b)

#define STDML_COLLECTIVE_PROFILE_RATE(name, payload)                           \
    ::stdml::collective::rchan::scope STDML_CAT(_stdml_scope_, __LINE__)(name, payload)

#define LOG_SCOPE_RATE(name, bytes)                                            \
    static ::stdml::collective::rchan::site_context STDML_CAT(_stdml_site_, __LINE__)(name); \
    ::stdml::collective::rchan::rate_scope STDML_CAT(_stdml_rate_, __LINE__)(   \
        STDML_CAT(_stdml_site_, __LINE__), bytes)

#define LOG_SCOPE_LATENCY(name)                                                \
    static ::stdml::collective::rchan::site_context STDML_CAT(_stdml_site_, __LINE__)(name); \
    ::stdml::collective::rchan::latency_scope STDML_CAT(_stdml_lat_, __LINE__)( \
        STDML_CAT(_stdml_site_, __LINE__))

#define LOG_EXPR_LATENCY(e)                                                    \
    [&]() {                                                                    \
        LOG_SCOPE_LATENCY(#e);                                                 \
        return (e);                                                            \
    }()
