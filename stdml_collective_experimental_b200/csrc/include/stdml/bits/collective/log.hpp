// Line logger.  `log() << a << b;` prints one line "[D] <thread> a b" to stderr
// when logging is enabled (STDML_COLLECTIVE_ENABLE_LOG or enable_log());
// `log(PRINT)` always prints, to stdout, without a prefix.  Items are separated
// by single spaces, as in the reference (include/stdml/bits/collective/log.hpp,
// src/stdml/collective/log.cpp:13-50).  A line is assembled privately and
// written with one call, so no global lock is held while it is formatted.
#pragma once
#include <sstream>
#include <string>

namespace stdml::collective
{
enum log_level { DEBUG, INFO, WARN, ERROR, PRINT };

void enable_log();
void disable_log();
bool log_enabled();

class logger
{
    log_level level_;
    bool active_;
    bool first_ = true;
    std::ostringstream line_;

  public:
    explicit logger(log_level level);
    logger(logger &&other);
    ~logger();

    template <typename T>
    logger &operator<<(const T &x)
    {
        if (active_) {
            if (!first_) { line_ << ' '; }
            first_ = false;
            line_ << x;
        }
        return *this;
    }
};

inline logger log(log_level level = DEBUG) { return logger(level); }
}  // namespace stdml::collective
