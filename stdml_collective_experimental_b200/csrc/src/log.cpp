#include <atomic>
#include <cstdio>
#include <functional>
#include <thread>

#include <stdml/bits/collective/config.hpp>
#include <stdml/bits/collective/log.hpp>

namespace stdml::collective
{
namespace
{
std::atomic<int> &log_flag()
{
    static std::atomic<int> flag{parse_env_bool("STDML_COLLECTIVE_ENABLE_LOG") ? 1 : 0};
    return flag;
}

const char *prefix_of(log_level l)
{
    switch (l) {
    case DEBUG:
        return "[D]";
    case INFO:
        return "[I]";
    case WARN:
        return "[W]";
    case ERROR:
        return "[E]";
    default:
        return "";
    }
}
}  // namespace

void enable_log() { log_flag().store(1); }
void disable_log() { log_flag().store(0); }
bool log_enabled() { return log_flag().load(std::memory_order_relaxed) != 0; }

logger::logger(log_level level)
    : level_(level), active_(level == PRINT || level >= WARN || log_enabled())
{
}

logger::logger(logger &&other)
    : level_(other.level_), active_(other.active_), first_(other.first_),
      line_(std::move(other.line_))
{
    other.active_ = false;
}

logger::~logger()
{
    if (!active_) { return; }
    std::string out;
    if (level_ != PRINT) {
        const size_t tid = std::hash<std::thread::id>()(std::this_thread::get_id()) % 100000;
        out = std::string(prefix_of(level_)) + " " + std::to_string(tid) + " ";
    }
    out += line_.str();
    out += '\n';
    FILE *f = level_ == PRINT ? stdout : stderr;
    std::fwrite(out.data(), 1, out.size(), f);
    std::fflush(f);
}
}  // namespace stdml::collective
