// ANSI colour helpers for terminal output (log prefixes, launcher messages).
// Counterpart of include/stdml/bits/collective/xterm.hpp.
#pragma once
#include <ostream>
#include <string>

#include <unistd.h>

namespace stdml::collective::xterm
{
struct colour {
    int fg;  // 30..37, 90..97
    bool bold = false;
};

inline constexpr colour red{31}, green{32}, yellow{33}, blue{34}, magenta{35}, cyan{36}, grey{90};

inline bool is_terminal(int fd = 1) { return ::isatty(fd) != 0; }

inline std::string paint(const std::string &text, colour c, bool enable = true)
{
    if (!enable) { return text; }
    return "\x1b[" + std::string(c.bold ? "1;" : "") + std::to_string(c.fg) + "m" + text + "\x1b[0m";
}

// os << with(xterm::green, "ok")
struct painted {
    colour c;
    std::string text;
};

inline painted with(colour c, std::string text) { return painted{c, std::move(text)}; }

inline std::ostream &operator<<(std::ostream &os, const painted &p)
{
    return os << paint(p.text, p.c);
}
}  // namespace stdml::collective::xterm
