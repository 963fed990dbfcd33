// C ABI of the host runtime (loaded from Python with ctypes).
#include <cstring>
#include <stdexcept>
#include <string>

#include <stdml/bits/collective/dtype.hpp>

namespace sc = stdml::collective;

extern "C" {
const char *stdmlc_version() { return "0.1.0"; }

int stdmlc_dtype_size(int dt)
{
    return static_cast<int>(sc::dtype_size_nothrow(static_cast<sc::dtype>(dt)));
}

// out[i] = in[0][i] op ... op in[n-1][i], rank-ascending; the CPU oracle of the
// device kernels.  Returns 0, or 2 for an undefined (dtype, op) pair.
int stdmlc_reduce_many(void *out, const void *const *in, unsigned long long n,
                       unsigned long long count, int dt, int op, double scale)
{
    try {
        sc::reduce_many(out, in, n, count, static_cast<sc::dtype>(dt),
                        static_cast<sc::reduce_op>(op), scale);
        return 0;
    } catch (const std::exception &) {
        return 2;
    }
}

int stdmlc_reduce(void *x, const void *y, const void *z, unsigned long long count, int dt, int op)
{
    try {
        sc::reduce(x, y, z, count, static_cast<sc::dtype>(dt), static_cast<sc::reduce_op>(op));
        return 0;
    } catch (const std::exception &) {
        return 2;
    }
}
}
