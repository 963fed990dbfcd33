// Tiny assertion helpers for the C++ test programs: a failed check prints the
// location and makes the process exit non-zero at the end (or at once with
// REQUIRE), so the forked ranks of prun() report failures to the parent.
#pragma once
#include <cstdio>
#include <cstdlib>
#include <string>

namespace testing
{
inline int &failures()
{
    static int n = 0;
    return n;
}

inline void fail(const char *file, int line, const std::string &what)
{
    std::fprintf(stderr, "%s:%d: check failed: %s\n", file, line, what.c_str());
    ++failures();
}

inline int result(const char *name)
{
    if (failures() == 0) {
        std::printf("%s: OK\n", name);
        return 0;
    }
    std::printf("%s: %d check(s) FAILED\n", name, failures());
    return 1;
}
}  // namespace testing

#define CHECK(cond)                                                            \
    do {                                                                       \
        if (!(cond)) { ::testing::fail(__FILE__, __LINE__, #cond); }           \
    } while (0)

#define CHECK_MSG(cond, msg)                                                   \
    do {                                                                       \
        if (!(cond)) { ::testing::fail(__FILE__, __LINE__, std::string(#cond) + " : " + (msg)); } \
    } while (0)

#define REQUIRE(cond)                                                          \
    do {                                                                       \
        if (!(cond)) {                                                         \
            ::testing::fail(__FILE__, __LINE__, #cond);                        \
            std::exit(1);                                                      \
        }                                                                      \
    } while (0)
