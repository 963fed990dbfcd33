// Two-level all_reduce (reduce inside each host, all-reduce among one leader
// per host, broadcast inside each host) against the closed form, started by
// one runner per emulated host (loopback aliases) with
// STDML_COLLECTIVE_HIERARCHICAL=1.  Host counts may be uneven.
//   stdml_collective_run -H 127.0.0.2:3,127.0.0.3:2 -np 5 -self <ip> ... test_two_level
#include <cstdio>
#include <future>
#include <numeric>
#include <vector>

#include <stdml/collective>

#include "testing.hpp"

using namespace stdml::collective;

int main()
{
    peer p = peer::from_env();
    session sess = p.join();
    const size_t n = sess.size(), r = sess.rank();
    REQUIRE(sess.config().hierarchical);
    bool several = false;
    for (const auto &q : sess.peers()) { several = several || q.ipv4 != sess.peers()[0].ipv4; }
    REQUIRE(several);

    for (size_t count : {size_t(1), size_t(1000), size_t(300000), size_t(700001)}) {
        std::vector<double> x(count), y(count, -1);
        for (size_t i = 0; i < count; ++i) { x[i] = double(r + 1) * double(i % 97); }
        sess.all_reduce(x.data(), y.data(), count, f64, sum, "s" + std::to_string(count));
        const double tri = double(n * (n + 1) / 2);
        for (size_t i = 0; i < count; i += 1 + count / 50) { CHECK(y[i] == tri * double(i % 97)); }
        CHECK(y[count - 1] == tri * double((count - 1) % 97));
        // in place, another operator and type
        std::vector<int32_t> z(count, int32_t(r) - 2);
        sess.all_reduce(z.data(), z.data(), count, i32, min, "m" + std::to_string(count));
        CHECK(z[0] == -2 && z[count - 1] == -2);
        std::vector<int32_t> hi(count, int32_t(r));
        sess.all_reduce(hi.data(), hi.data(), count, i32, max, "x" + std::to_string(count));
        CHECK(hi[count / 2] == int32_t(n - 1));
    }
    // a fused group with futures that resolve out of order
    std::vector<std::vector<float>> in(12), out(12);
    std::vector<std::promise<workspace>> ps(12);
    std::vector<std::future<workspace>> fs;
    for (size_t t = 0; t < 12; ++t) {
        in[t].assign(100 + 5000 * t, float(r + t));
        out[t].assign(in[t].size(), -1.0f);
        fs.push_back(ps[t].get_future());
    }
    std::thread producer([&] {
        for (size_t k = 0; k < 12; ++k) {
            const size_t t = (k * 5 + r) % 12;  // a different order on every rank
            workspace w;
            w.send = in[t].data();
            w.recv = out[t].data();
            w.count = in[t].size();
            w.dt = f32;
            w.op = sum;
            w.name = "g" + std::to_string(t);
            ps[t].set_value(w);
        }
    });
    sess.group_all_reduce(std::move(fs));
    producer.join();
    for (size_t t = 0; t < 12; ++t) {
        const float want = float(n * (n - 1) / 2 + n * t);
        CHECK(out[t].front() == want && out[t].back() == want);
    }
    // the scalar helpers and the barrier go the same way
    CHECK(sess.all_reduce(int64_t(r), max) == int64_t(n - 1));
    sess.barrier();
    std::printf("rank %zu/%zu: %s\n", r, n, testing::failures() == 0 ? "OK" : "WRONG");
    return testing::failures() == 0 ? 0 : 1;
}
