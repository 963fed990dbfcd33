// Where this binary came from: compiler, build time, git commit (when the
// build system passes -DSTDML_GIT_COMMIT=...), CUDA architecture.  Counterpart
// of include/stdml/bits/collective/build_info.hpp.
#pragma once
#include <ostream>
#include <string>

namespace stdml::collective
{
struct build_info {
    std::string version, git_commit, build_time, cxx_compiler, cuda_arch;
};
build_info get_build_info();
void show_build_info(std::ostream &os);
void show_build_info();
}  // namespace stdml::collective
