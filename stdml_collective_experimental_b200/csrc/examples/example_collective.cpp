// Self-checking tour of the collectives; exits non-zero on a wrong result.
#include <cstdio>
#include <vector>

#include <stdml/collective>

using namespace stdml::collective;

int main()
{
    auto p = peer::from_env();
    session sess = p.join();
    const int n = static_cast<int>(sess.size()), r = static_cast<int>(sess.rank());
    int bad = 0;

    std::vector<float> g(1000, float(r + 1)), avg(1000);
    sess.all_reduce(g.data(), avg.data(), g.size(), f32, sum, "grad");
    for (float v : avg) { bad += v != n * (n + 1) / 2.0f; }

    std::vector<int> all(n);
    sess.all_gather(&r, all.data(), 1, "ranks");
    for (int i = 0; i < n; ++i) { bad += all[i] != i; }

    const double seed = sess.broadcast(3.25 + r);
    bad += seed != 3.25;

    bad += sess.all_reduce(r, max) != n - 1;
    bad += !sess.consistent(n);

    std::printf("rank %d/%d: %s\n", r, n, bad == 0 ? "OK" : "WRONG");
    return bad == 0 ? 0 : 1;
}
