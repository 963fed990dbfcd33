// Multi-process integration test of the host (TCP) collectives.
//
//   test_collectives <np>        forks np ranks on 127.0.0.1:10000.. (prun)
//   test_collectives             uses the launcher's environment (KungFu /
//                                OpenMPI / torchrun variables)
// Strategy and runtime come from KUNGFU_ALLREDUCE_STRATEGY and
// STDML_COLLECTIVE_USE_{THREAD_POOL,ASYNC}.  The matrix extends the
// reference's (tests/integration/test_all_reduce.cpp: counts x dtypes x two
// value patterns, sum only) with every operator, bf16/f16, messages larger
// than one 1 MiB chunk, send/recv, reduce, gather, consistent, and a
// 300-tensor group whose futures resolve in a different order on every rank.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <future>
#include <numeric>
#include <thread>
#include <vector>

#include <stdml/collective>

#include "testing.hpp"

using namespace stdml::collective;

template <typename T>
static void check_all_reduce_typed(session &sess, size_t count)
{
    const size_t n = sess.size(), r = sess.rank();
    const std::string tag = std::string(dtype_name(type<T>())) + ":" + std::to_string(count);
    {  // every rank contributes its rank: sum = n(n-1)/2
        std::vector<T> x(count, static_cast<T>(r)), y(count, static_cast<T>(99));
        sess.all_reduce(x.data(), y.data(), count, sum, "a:" + tag);
        for (const T v : y) { CHECK_MSG(v == static_cast<T>(n * (n - 1) / 2), tag); }
        sess.all_reduce(x.data(), x.data(), count, sum, "b:" + tag);  // in place
        for (const T v : x) { CHECK_MSG(v == static_cast<T>(n * (n - 1) / 2), tag + " in place"); }
    }
    if (n <= 6) {  // 1 << rank: sum = 2^n - 1 (fits an int8)
        std::vector<T> x(count, static_cast<T>(1u << r)), y(count);
        sess.all_reduce(x.data(), y.data(), count, sum, "c:" + tag);
        for (const T v : y) { CHECK_MSG(v == static_cast<T>((1u << n) - 1), tag); }
    }
    {  // position-dependent values, min / max / prod
        std::vector<T> x(count), lo(count), hi(count), pr(count);
        for (size_t i = 0; i < count; ++i) { x[i] = static_cast<T>((i + 3 * r) % 5 + 1); }
        sess.all_reduce(x.data(), lo.data(), count, min, "d:" + tag);
        sess.all_reduce(x.data(), hi.data(), count, max, "e:" + tag);
        for (size_t i = 0; i < count; ++i) {
            T wlo = static_cast<T>(100), whi = static_cast<T>(0);
            for (size_t q = 0; q < n; ++q) {
                const T v = static_cast<T>((i + 3 * q) % 5 + 1);
                wlo = std::min(wlo, v);
                whi = std::max(whi, v);
            }
            CHECK_MSG(lo[i] == wlo && hi[i] == whi, tag + " min/max");
        }
        std::vector<T> two(count, static_cast<T>(r % 2 == 0 ? 2 : 1));
        sess.all_reduce(two.data(), pr.data(), count, prod, "f:" + tag);
        const T want = static_cast<T>(1u << ((n + 1) / 2));
        if (n <= 12) {
            for (const T v : pr) { CHECK_MSG(v == want, tag + " prod"); }
        }
    }
}

static void check_all_reduce(session &sess)
{
    for (size_t count : {1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 100, 1024}) {
        check_all_reduce_typed<int8_t>(sess, count);
        check_all_reduce_typed<int16_t>(sess, count);
        check_all_reduce_typed<int32_t>(sess, count);
        check_all_reduce_typed<int64_t>(sess, count);
        check_all_reduce_typed<uint8_t>(sess, count);
        check_all_reduce_typed<uint16_t>(sess, count);
        check_all_reduce_typed<uint32_t>(sess, count);
        check_all_reduce_typed<uint64_t>(sess, count);
        check_all_reduce_typed<float>(sess, count);
        check_all_reduce_typed<double>(sess, count);
    }
    // several 1 MiB chunks, spread over ring roots by chunk name
    check_all_reduce_typed<float>(sess, 700001);
    check_all_reduce_typed<int32_t>(sess, (3u << 18) + 5);
    // 16-bit floats (the reference aborts on these)
    const size_t n = sess.size(), r = sess.rank();
    for (dtype dt : {bf16, f16}) {
        std::vector<uint16_t> x(37), y(37);
        const uint16_t mine = dt == bf16 ? float_to_bf16(float(r) + 0.5f) : float_to_f16(float(r) + 0.5f);
        std::fill(x.begin(), x.end(), mine);
        sess.all_reduce(x.data(), y.data(), x.size(), dt, sum, std::string("h:") + dtype_name(dt));
        const float want = n * (n - 1) / 2.0f + 0.5f * n;
        for (const uint16_t v : y) {
            CHECK((dt == bf16 ? bf16_to_float(v) : f16_to_float(v)) == want);
        }
    }
    // bit_xor on integers; undefined on floats
    std::vector<uint32_t> bits(9, 1u << r), out(9);
    sess.all_reduce(bits.data(), out.data(), 9, bit_xor, "x");
    for (const uint32_t v : out) { CHECK(v == (1u << n) - 1u); }
    bool threw = false;
    float f = 1, g = 0;
    try {
        sess.all_reduce(&f, &g, 1, f32, bit_xor, "bad");
    } catch (const std::invalid_argument &) {
        threw = true;
    }
    CHECK(threw);
    // zero elements is a no-op, not an error
    sess.all_reduce(&f, &g, 0, f32, sum, "empty");
    // scalar helpers
    CHECK(sess.all_reduce(int(r), max) == int(n - 1));
    CHECK(sess.all_reduce(1.5) == 1.5 * n);
}

static void check_group(session &sess)
{
    const size_t n = sess.size(), r = sess.rank();
    const size_t tensors = 300;
    std::vector<std::vector<float>> xs(tensors), ys(tensors);
    std::vector<std::promise<workspace>> promises(tensors);
    std::vector<std::future<workspace>> futures;
    for (size_t i = 0; i < tensors; ++i) {
        const size_t count = 1 + (i * 37) % 3000;
        xs[i].assign(count, float(r + i));
        ys[i].assign(count, -1.0f);
        futures.push_back(promises[i].get_future());
    }
    // every rank makes its tensors ready in a different (rotated) order, slowly
    std::thread producer([&] {
        for (size_t k = 0; k < tensors; ++k) {
            const size_t i = (k + r * 97) % tensors;
            workspace w{xs[i].data(), ys[i].data(), xs[i].size(), f32, sum,
                        "variable:" + std::to_string(i)};
            promises[i].set_value(w);
            if (k % 50 == 0) { std::this_thread::sleep_for(std::chrono::milliseconds(2)); }
        }
    });
    sess.group_all_reduce(std::move(futures));
    producer.join();
    for (size_t i = 0; i < tensors; ++i) {
        const float want = float(n * (n - 1) / 2 + n * i);
        for (const float v : ys[i]) { CHECK_MSG(v == want, "group tensor " + std::to_string(i)); }
    }
    // ready tensors with a fused scale
    std::vector<workspace> ws;
    for (size_t i = 0; i < 5; ++i) {
        xs[i].assign(xs[i].size(), 2.0f);
        ws.push_back(workspace{xs[i].data(), ys[i].data(), xs[i].size(), f32, sum,
                               "scaled:" + std::to_string(i)});
    }
    sess.group_all_reduce(ws, 1.0 / n);
    for (size_t i = 0; i < 5; ++i) {
        for (const float v : ys[i]) { CHECK(std::fabs(v - 2.0f) < 1e-6f); }
    }
}

static void check_others(session &sess)
{
    const size_t n = sess.size(), r = sess.rank();
    for (size_t count : {1, 2, 10, 70000}) {
        std::vector<int> x(count), y(count * n, -1);
        std::iota(x.begin(), x.end(), int(r * 1000));
        sess.all_gather(x.data(), y.data(), count, "ag" + std::to_string(count));
        for (size_t q = 0; q < n; ++q) {
            for (size_t i = 0; i < count; ++i) { CHECK(y[q * count + i] == int(q * 1000 + i)); }
        }
        std::vector<int> z(count * n, -1);
        sess.gather(x.data(), z.data(), count, i32, "g" + std::to_string(count));
        if (r == 0) { CHECK(z == y); }
        std::vector<int> b(count, -5);
        sess.broadcast(x.data(), b.data(), count, i32, "bc" + std::to_string(count));
        for (size_t i = 0; i < count; ++i) { CHECK(b[i] == int(i)); }
        // any root (the last rank here), in place on the root
        const size_t root = n - 1;
        std::vector<int> br = x;
        sess.broadcast(br.data(), br.data(), count, i32, "bcr" + std::to_string(count), nullptr, root);
        for (size_t i = 0; i < count; ++i) { CHECK(br[i] == int(root * 1000 + i)); }
        // reduce and gather to the last rank, reduce in place
        std::vector<int> rr = x;
        sess.reduce(rr.data(), rr.data(), count, i32, sum, "rdr" + std::to_string(count), nullptr, root);
        if (r == root) {
            for (size_t i = 0; i < count; ++i) { CHECK(rr[i] == int(1000 * n * (n - 1) / 2 + n * i)); }
        } else {
            CHECK(rr == x);
        }
        std::vector<int> gr(count * n, -1);
        sess.gather(x.data(), gr.data(), count, i32, "gr" + std::to_string(count), root);
        if (r == root) { CHECK(gr == y); }
        // reduce_scatter and all_to_all
        std::vector<int> rsin(count * n), rsout(count, -1);
        for (size_t i = 0; i < rsin.size(); ++i) { rsin[i] = int(i) + int(r); }
        sess.reduce_scatter(rsin.data(), rsout.data(), count, i32, sum, "rs" + std::to_string(count));
        for (size_t i = 0; i < count; ++i) {
            CHECK(rsout[i] == int(n) * int(r * count + i) + int(n * (n - 1) / 2));
        }
        std::vector<int> a2in(count * n), a2out(count * n, -1);
        for (size_t q = 0; q < n; ++q) {
            for (size_t i = 0; i < count; ++i) { a2in[q * count + i] = int(r * 100000 + q * 1000 + i % 1000); }
        }
        sess.all_to_all(a2in.data(), a2out.data(), count, i32, "a2a" + std::to_string(count));
        for (size_t q = 0; q < n; ++q) {
            for (size_t i = 0; i < count; i += 1 + count / 7) {
                CHECK(a2out[q * count + i] == int(q * 100000 + r * 1000 + i % 1000));
            }
        }
        std::vector<int> red(count, -7);
        sess.reduce(x.data(), red.data(), count, i32, sum, "rd" + std::to_string(count));
        if (r == 0) {
            for (size_t i = 0; i < count; ++i) {
                CHECK(red[i] == int(1000 * n * (n - 1) / 2 + n * i));
            }
        } else {
            CHECK(red[0] == -7);
        }
    }
    CHECK(sess.broadcast(int(r)) == 0);
    struct pod {
        double a;
        int b;
    };
    const pod p = sess.broadcast(pod{r + 0.25, int(r) - 3});
    CHECK(p.a == 0.25 && p.b == -3);

    // one session used from several threads at once: operations with distinct
    // names do not disturb each other, whatever order the threads run in
    {
        std::atomic<int> wrong{0};
        std::vector<std::thread> ths;
        for (int t = 0; t < 4; ++t) {
            ths.emplace_back([&, t] {
                for (int i = 0; i < 10; ++i) {
                    const size_t count = 1000 * (t + 1) + i;
                    std::vector<int64_t> x(count, int64_t(r) * (t + 1) + i), y(count, -1);
                    sess.all_reduce(x.data(), y.data(), count, i64, sum, "mt" + std::to_string(t));
                    const int64_t want = int64_t(n * (n - 1) / 2) * (t + 1) + int64_t(n) * i;
                    if (y.front() != want || y.back() != want) { ++wrong; }
                    std::vector<int> g(3 * n, -1), mine(3, int(r) + 10 * t);
                    sess.all_gather(mine.data(), g.data(), 3, "mtg" + std::to_string(t));
                    for (size_t q = 0; q < n; ++q) {
                        if (g[3 * q] != int(q) + 10 * t) { ++wrong; }
                    }
                }
            });
        }
        for (auto &th : ths) { th.join(); }
        CHECK(wrong.load() == 0);
    }

    // sub-groups: evens and odds reduce among themselves while the whole group
    // goes on working; a sub-group of a sub-group; ranks in a chosen order
    if (n >= 2) {
        std::vector<size_t> mine_group;
        for (size_t q = r % 2; q < n; q += 2) { mine_group.push_back(q); }
        auto half = sess.subgroup(mine_group, r % 2 == 0 ? "evens" : "odds");
        REQUIRE(half != nullptr);
        CHECK(half->size() == mine_group.size() && half->rank() == r / 2);
        int64_t got = half->all_reduce(int64_t(r), sum);
        int64_t want = 0;
        for (size_t q : mine_group) { want += int64_t(q); }
        CHECK(got == want);
        CHECK(sess.all_reduce(int64_t(1), sum) == int64_t(n));  // the parent is undisturbed
        std::vector<int> blocks(half->size(), -1);
        const int me = int(r);
        half->all_gather(&me, blocks.data(), 1, "who");
        for (size_t i = 0; i < mine_group.size(); ++i) { CHECK(blocks[i] == int(mine_group[i])); }
        if (half->size() >= 2) {
            auto pair = half->subgroup({1, 0}, "first-two-swapped");
            if (half->rank() < 2) {
                REQUIRE(pair != nullptr);
                CHECK(pair->rank() == 1 - half->rank());
                CHECK(pair->broadcast(int(r)) == int(mine_group[1]));  // its rank 0 is the half's rank 1
            } else {
                CHECK(pair == nullptr);
            }
        }
        CHECK(sess.subgroup({(r + 1) % n}, "not-me") == nullptr || n == 1);
        sess.barrier();
    }

    // consistent: same bytes everywhere / one rank differs / lengths differ
    int same = 42;
    CHECK(sess.consistent(same));
    int diff = r == n - 1 ? 43 : 42;
    CHECK(sess.consistent(diff) == (n == 1));
    std::vector<char> blob(r == 0 ? 3 : 4, 'x');
    CHECK(sess.consistent(blob.data(), blob.size()) == (n == 1));

    // point to point ring: rank r sends to r+1; too small a buffer is refused
    if (n > 1) {
        std::vector<float> out(1000, float(r)), in(1000, -1.0f);
        std::thread t([&] { sess.send(out.data(), out.size(), f32, (r + 1) % n, "ring"); });
        sess.recv(in.data(), in.size(), f32, (r + n - 1) % n, "ring");
        t.join();
        for (const float v : in) { CHECK(v == float((r + n - 1) % n)); }
        std::thread t2([&] { sess.send(out.data(), 8, f32, (r + 1) % n, "short"); });
        bool threw = false;
        try {
            sess.recv(in.data(), 4, f32, (r + n - 1) % n, "short");
        } catch (const std::length_error &) {
            threw = true;
        }
        t2.join();
        CHECK(threw);
    }
    // async interface: two operations in flight, polled from this thread
    {
        std::vector<float> a(300000, float(r)), b(1000, 1.0f), ra(a.size()), rb(b.size());
        auto t1 = sess.async_all_reduce(a.data(), ra.data(), a.size(), f32, sum, "async:a");
        auto t2 = sess.async_all_reduce(b.data(), rb.data(), b.size(), f32, max, "async:b");
        while (!t1->finished() || !t2->finished()) {
            t1->poll();
            t2->poll();
        }
        CHECK(ra[0] == float(n * (n - 1) / 2) && ra.back() == ra[0] && rb[0] == 1.0f);
    }
    sess.barrier();
}

static int run_rank(session &sess)
{
    check_all_reduce(sess);
    check_others(sess);
    check_group(sess);
    sess.barrier();
    return testing::failures();
}

int main(int argc, char *argv[])
{
    if (argc > 1) {
        const int np = std::atoi(argv[1]);
        try {
            prun(np, [](session &sess) {
                if (run_rank(sess) != 0) { throw std::runtime_error("checks failed"); }
            });
        } catch (const std::exception &e) {
            std::printf("test-collectives np=%d: FAILED (%s)\n", np, e.what());
            return 1;
        }
        std::printf("test-collectives np=%d: OK\n", np);
        return 0;
    }
    auto p = peer::from_env();
    session sess = p.join();
    run_rank(sess);
    return testing::result("test-collectives");
}
