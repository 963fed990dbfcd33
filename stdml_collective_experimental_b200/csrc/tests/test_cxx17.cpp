// The public headers must be usable from a C++17 translation unit (the
// reference checks the same: tests/build/c++17.cpp).  Built with -std=c++17.
#include <stdml/collective>
#include <stdml/mpi.h>

int main()
{
    auto p = stdml::collective::peer::single();
    stdml::collective::session s = p.join();
    return s.all_reduce(1) == 1 ? 0 : 1;
}
