// patient: "has it been quiet for long enough to speak again?"  Used to keep
// repeated warnings (accept failures, retries) to one per interval.  Counterpart
// of include/stdml/bits/collective/patient.hpp.
#pragma once
#include <chrono>
#include <string>

#include <stdml/bits/collective/stat.hpp>

namespace stdml::collective
{
class patient
{
    using clock = std::chrono::steady_clock;
    std::chrono::nanoseconds threshold_;
    clock::time_point last_;

  public:
    explicit patient(int seconds) : patient(std::chrono::seconds(seconds)) {}

    explicit patient(std::chrono::nanoseconds threshold = std::chrono::seconds(1))
        : threshold_(threshold), last_(clock::now())
    {
    }

    std::string show() const
    {
        return rchan::show_duration(std::chrono::duration<double>(threshold_));
    }

    void reset() { last_ = clock::now(); }

    // still within the quiet interval since the last reset()
    bool ok() const { return clock::now() - last_ < threshold_; }

    // true at most once per interval: if (p.lost()) { log(...); }
    bool lost()
    {
        if (ok()) { return false; }
        reset();
        return true;
    }
};
}  // namespace stdml::collective
