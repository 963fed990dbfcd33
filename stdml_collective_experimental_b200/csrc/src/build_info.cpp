#include <iostream>

#include <stdml/bits/collective/build_info.hpp>

#ifndef STDML_GIT_COMMIT
#define STDML_GIT_COMMIT "unknown"
#endif

namespace stdml::collective
{
build_info get_build_info()
{
    build_info b;
    b.version = "0.1.0";
    b.git_commit = STDML_GIT_COMMIT;
    b.build_time = __DATE__ " " __TIME__;
#if defined(__clang__)
    b.cxx_compiler = std::string("clang ") + __clang_version__;
#elif defined(__GNUC__)
    b.cxx_compiler = std::string("g++ ") + __VERSION__;
#else
    b.cxx_compiler = "unknown";
#endif
    b.cuda_arch = "sm_100a";
    return b;
}

void show_build_info(std::ostream &os)
{
    const build_info b = get_build_info();
    os << "stdml-collective (B200) " << b.version << "\n"
       << "  git commit  : " << b.git_commit << "\n"
       << "  built       : " << b.build_time << "\n"
       << "  c++ compiler: " << b.cxx_compiler << "\n"
       << "  cuda arch   : " << b.cuda_arch << "\n";
}

void show_build_info() { show_build_info(std::cout); }
}  // namespace stdml::collective
