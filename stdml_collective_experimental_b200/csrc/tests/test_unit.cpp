// Host unit tests (no network): reducers, partitions, graphs, cluster
// configuration encodings, JSON, HTTP helpers, channels, slots, thread pool,
// task trees.  The reference's unit tests only print (tests/unit/*.cpp); these
// assert.
#include <atomic>
#include <cmath>
#include <cstring>
#include <thread>

#include <stdml/bits/collective/affinity.hpp>
#include <stdml/bits/collective/execution.hpp>
#include <stdml/bits/collective/http.hpp>
#include <stdml/bits/collective/json.hpp>
#include <stdml/bits/collective/net/ioutil.hpp>
#include <stdml/bits/collective/net/tcp.hpp>
#include <stdml/bits/collective/patient.hpp>
#include <stdml/bits/collective/xterm.hpp>
#include <stdml/bits/collective/waitgroup.hpp>
#include <stdml/collective>

#include "../src/shm_ring.hpp"
#include "testing.hpp"

using namespace stdml::collective;

static void test_dtype()
{
    CHECK(dtype_size(bf16) == 2 && dtype_size(f16) == 2 && dtype_size(f64) == 8 &&
          dtype_size(u8) == 1);
    CHECK(type<float>() == f32 && type<int64_t>() == i64 && type<uint16_t>() == u16);
    CHECK(!reduce_supported(f32, bit_xor) && reduce_supported(i8, bit_xor));
    int a[4] = {1, 5, -3, 7}, b[4] = {2, 4, -9, 7}, c[4];
    reduce(c, a, b, 4, i32, sum);
    CHECK(c[0] == 3 && c[2] == -12);
    reduce(c, a, b, 4, i32, min);
    CHECK(c[1] == 4 && c[2] == -9);
    reduce(c, a, b, 4, i32, max);
    CHECK(c[1] == 5 && c[2] == -3);
    reduce(c, a, b, 4, i32, prod);
    CHECK(c[3] == 49);
    reduce(c, a, b, 4, i32, bit_xor);
    CHECK(c[0] == 3 && c[3] == 0);
    bool threw = false;
    float x[1] = {1}, y[1] = {2}, z[1];
    try {
        reduce(z, x, y, 1, f32, bit_xor);
    } catch (const std::invalid_argument &) {
        threw = true;
    }
    CHECK(threw);
    // 16-bit floats round to nearest even and survive a round trip
    for (float v : {0.0f, 1.0f, -2.5f, 3.14159f, 65504.0f, 1e-5f, 1e-8f}) {
        CHECK(std::fabs(bf16_to_float(float_to_bf16(v)) - v) <= std::fabs(v) * 0.0079f);
        const float h = f16_to_float(float_to_f16(v));
        CHECK(std::fabs(h - v) <= std::fabs(v) * 0.001f + 6e-8f);
    }
    CHECK(float_to_bf16(1.00390625f) == 0x3f80);  // tie -> even
    CHECK(float_to_f16(65520.0f) == 0x7c00);       // overflow -> inf
    uint16_t hs[2] = {float_to_bf16(1.5f), float_to_bf16(2.25f)}, hz[2];
    const void *ins[3] = {hs, hs, hs};
    reduce_many(hz, ins, 3, 2, bf16, sum, 0.5);
    CHECK(bf16_to_float(hz[0]) == 2.25f && bf16_to_float(hz[1]) == 3.375f);
}

static void test_partition()
{
    const auto p = even_partition(10, 3);
    CHECK(p.size() == 3 && p[0].first == 0 && p[0].second == 4 && p[1].second == 7 &&
          p[2].second == 10);
    float s[10], r[10];
    workspace w{s, r, 10, f32, sum, "x"};
    const auto parts = w.split(3);
    CHECK(parts.size() == 3 && parts[1].name == "part::x[4:7]" && parts[1].count == 3);
    CHECK(parts[1].send == s + 4 && parts[1].recv == r + 4);
    CHECK((workspace{s, r, 0, f32, sum, ""}.split_by_bytes(1 << 20).empty()));
    CHECK((workspace{s, r, 10, f32, sum, ""}.split_by_bytes(16).size() == 3));
    CHECK(w.split(100).size() == 10);
}

static void test_topology()
{
    const auto st = make_graph_pair_list(star, 4);
    CHECK(st.pairs.size() == 1);
    const graph &rg = st.pairs[0].reduce_graph, &bg = st.pairs[0].broadcast_graph;
    CHECK(rg.self_loop(0) && rg.prevs(0).size() == 3 && rg.nexts(2).size() == 1 &&
          rg.nexts(2)[0] == 0);
    CHECK(!bg.self_loop(0) && bg.nexts(0).size() == 3 && bg.prevs(3)[0] == 0);
    const auto rl = make_graph_pair_list(ring, 4);
    CHECK(rl.pairs.size() == 4);
    for (size_t r = 0; r < 4; ++r) {
        const graph &g = rl.pairs[r].reduce_graph, &b = rl.pairs[r].broadcast_graph;
        CHECK(g.nexts(r).empty() && g.prevs(r).size() == 1 && g.prevs(r)[0] == (r + 3) % 4);
        CHECK(g.prevs((r + 1) % 4).empty() && g.nexts((r + 1) % 4)[0] == (r + 2) % 4);
        CHECK(b.prevs(r).empty() && b.nexts(r)[0] == (r + 1) % 4 && b.nexts((r + 3) % 4).empty());
    }
    CHECK(make_graph_pair_list(ring, 1).pairs.size() == 1);
    // binary tree: n rotated trees; every non-root has one parent, at most two
    // children, the reduce graph is the broadcast graph reversed, depth <= log2
    for (size_t n : {2u, 5u, 8u, 13u}) {
        const auto tl = make_graph_pair_list(binary_tree, n);
        CHECK(tl.pairs.size() == n);
        for (size_t r = 0; r < n; ++r) {
            const graph &g = tl.pairs[r].reduce_graph, &b = tl.pairs[r].broadcast_graph;
            CHECK(b.prevs(r).empty() && g.nexts(r).empty() && g.self_loop(r) && !b.self_loop(r));
            for (size_t v = 0; v < n; ++v) {
                CHECK(b.nexts(v).size() <= 2 && b.nexts(v) == g.prevs(v));
                if (v != r) { CHECK(b.prevs(v).size() == 1 && g.nexts(v) == b.prevs(v)); }
                size_t hops = 0, at = v;
                while (at != r && hops <= n) {
                    at = b.prevs(at)[0];
                    ++hops;
                }
                size_t depth_bound = 0;
                while ((size_t(1) << depth_bound) <= n) { ++depth_bound; }
                CHECK(at == r && hops < depth_bound);
            }
        }
    }
    // clique: the star, once per rank as root
    for (size_t n : {2u, 5u}) {
        const auto cl = make_graph_pair_list(clique, n);
        CHECK(cl.pairs.size() == n);
        for (size_t r = 0; r < n; ++r) {
            const graph &g = cl.pairs[r].reduce_graph, &b = cl.pairs[r].broadcast_graph;
            CHECK(g.self_loop(r) && g.prevs(r).size() == n - 1 && g.nexts(r).empty());
            CHECK(b.nexts(r).size() == n - 1 && b.prevs(r).empty());
            for (size_t v = 0; v < n; ++v) {
                if (v != r) { CHECK(g.nexts(v).size() == 1 && g.nexts(v)[0] == r && b.prevs(v)[0] == r); }
            }
        }
    }
    CHECK(make_graph_pair_list(clique, 1).pairs.size() == 1);
    CHECK(std::string(strategy_name(clique)) == "CLIQUE" && parse_kungfu_startegy("clique") == clique);
    CHECK(std::string(strategy_name(binary_tree)) == "BINARY_TREE" &&
          parse_kungfu_startegy("tree") == binary_tree && parse_kungfu_startegy("Ring") == ring &&
          parse_kungfu_startegy(nullptr) == star);
    CHECK(rl.choose(6).first == &rl.pairs[2].reduce_graph);
    graph_builder gb(3);
    CHECK(gb.add_edge(0, 1) && !gb.add_edge(0, 1) && !gb.add_edge(1, 1) && !gb.add_edge(0, 9));
    CHECK(name_based_hash("ab") == 97u * 97u + 98u * 98u);
}

static void test_cluster_config()
{
    const auto id = parse_peer_id("10.1.2.3:8080");
    REQUIRE(id.has_value());
    CHECK(id->ipv4 == ((10u << 24) | (1u << 16) | (2u << 8) | 3u) && id->port == 8080);
    CHECK(id->str() == "10.1.2.3:8080");
    CHECK(!parse_peer_id("10.1.2:80") && !parse_peer_id("1.2.3.4:99999") && !parse_peer_id("x"));
    const auto ps = parse_peer_list("127.0.0.1:10000,127.0.0.1:10001");
    REQUIRE(ps.has_value());
    CHECK(ps->size() == 2 && *ps == peer_list::gen(2));
    CHECK(parse_peer_list("")->empty() && !parse_peer_list("a,b"));
    CHECK(ps->rank(peer_id{(127u << 24) | 1u, 10001}) == 1 && ps->rank(*id) == 2);

    cluster_config c(*parse_peer_list("127.0.0.1:38080"), peer_list::gen(2));
    const auto bytes = c.bytes();
    CHECK(bytes.size() == 8 + 6 * 3);
    uint32_t nr, nw;
    std::memcpy(&nr, bytes.data(), 4);
    std::memcpy(&nw, bytes.data() + 4, 4);
    CHECK(nr == 1 && nw == 2);
    uint32_t ip;
    uint16_t port;
    std::memcpy(&ip, bytes.data() + 8, 4);
    std::memcpy(&port, bytes.data() + 12, 2);
    CHECK(ip == 2130706433u && port == 38080);
    CHECK(cluster_config::from(bytes) == c);
    CHECK(!cluster_config::from(std::vector<std::byte>(7)));
    CHECK(c.json() ==
          "{\"Runners\":[{\"IPv4\":2130706433,\"Port\":38080}],\"Workers\":[{\"IPv4\":2130706433,"
          "\"Port\":10000},{\"IPv4\":2130706433,\"Port\":10001}]}");
    CHECK(cluster_config::from_json(c.json()) == c);
    CHECK(cluster_config::from_json(
              "{ \"Runners\": null, \"Workers\": [ {\"Port\": 1, \"IPv4\": 2} ] }")
              ->workers.size() == 1);
    CHECK(!cluster_config::from_json("{\"Runners\":[]}") && !cluster_config::from_json("nope"));
    const auto grown = c.resize(4);
    CHECK(grown.workers.size() == 4 && grown.workers[2].port == 10002 &&
          grown.workers[3].port == 10003 && grown.runners == c.runners);
    CHECK(grown.resize(1).workers.size() == 1);
    CHECK(cluster_config({}, peer_list::gen(2)).resize(5).workers.size() == 2);
    // two hosts: growth goes to the emptier one
    cluster_config two(*parse_peer_list("10.0.0.1:38080,10.0.0.2:38080"),
                       *parse_peer_list("10.0.0.1:10000,10.0.0.1:10001"));
    const auto g2 = two.resize(4);
    CHECK(g2.workers[2].str() == "10.0.0.2:10000" && g2.workers[3].str() == "10.0.0.2:10001");
    CHECK((*ps - peer_list::gen(1)).size() == 1);
}

static void test_json_http()
{
    const auto v = json::parse(" {\"a\": [1, -2.5, true, null, \"x\\n\\u0041\"], \"b\": {}} ");
    REQUIRE(v.has_value());
    CHECK(v->get("a")->items().size() == 5 && v->get("a")->items()[0].as_int() == 1);
    CHECK(v->get("a")->items()[1].as_double() == -2.5 && v->get("a")->items()[2].as_bool());
    CHECK(v->get("a")->items()[4].as_string() == "x\nA" && v->get("zz") == nullptr);
    CHECK(json::parse(v->dump())->dump() == v->dump());
    CHECK(!json::parse("{") && !json::parse("[1,]") && !json::parse("1 2") && !json::parse(""));
    CHECK(json::to_json(std::string("q\"")) == "\"q\\\"\"");
    CHECK(json::to_json(std::pair<std::string, int64_t>("k", 7)) == "\"k\":7");

    const auto u = http_parse_url("http://127.0.0.1:9100/config");
    REQUIRE(u.has_value());
    CHECK(u->host == "127.0.0.1" && u->port == 9100 && u->path == "/config");
    CHECK(http_parse_url("http://host")->port == 80 && http_parse_url("http://host")->path == "/");
    CHECK(!http_parse_url("ftp://x") && !http_parse_url("http://:80/") &&
          !http_parse_url("http://h:0x/"));
    CHECK(*http_content_length("HTTP/1.1 200 OK\r\ncontent-LENGTH:  42\r\n") == 42);
    CHECK(!http_content_length("HTTP/1.1 200 OK\r\n"));
    std::string stored = "{}";
    http_server srv(0, [&](const http_server::request &rq) {
        http_response rs;
        rs.status = 200;
        if (rq.method == "PUT") { stored = rq.body; }
        rs.body = stored;
        return rs;
    });
    srv.start();
    const std::string url = "http://127.0.0.1:" + std::to_string(srv.port()) + "/config";
    CHECK(http_get(url)->body == "{}");
    CHECK(http_put(url, "{\"x\":1}")->status == 200);
    CHECK(http_get(url)->body == "{\"x\":1}");
    srv.stop();
    CHECK(!http_get("http://127.0.0.1:1/none", 500));
}

static void test_sync_primitives()
{
    channel<int> ch(2);
    ch.put(1);
    ch.put(2);
    CHECK(ch.get() == 1 && *ch.try_get() == 2 && !ch.try_get());
    CHECK(!ch.get_for(std::chrono::milliseconds(10)));

    // slot: destination posted first (zero-copy), body first (parked), too small
    slot s;
    char dst[8] = {0};
    std::thread t([&] {
        std::this_thread::sleep_for(std::chrono::milliseconds(20));
        s.put(4, [](void *p) {
            std::memcpy(p, "abcd", 4);
            return true;
        });
    });
    CHECK(s.get(dst, 8) && std::memcmp(dst, "abcd", 4) == 0);
    t.join();
    s.put(3, [](void *p) {
        std::memcpy(p, "xyz", 3);
        return true;
    });
    CHECK(s.get(dst, 8) && std::memcmp(dst, "xyz", 3) == 0);
    s.put(8, [](void *p) {
        std::memset(p, 1, 8);
        return true;
    });
    CHECK(!s.get(dst, 4));
    auto polled = s.post_polled(dst, 8);
    CHECK(!polled());
    s.put(2, [](void *p) {
        std::memcpy(p, "ok", 2);
        return true;
    });
    CHECK(polled() && dst[0] == 'o');
    // a pending post: not ready, withdrawn (twice: the second time must not wait),
    // and a body that comes afterwards goes to the next receiver, not to the old buffer
    char old_buf[4] = {'-', '-', '-', '-'};
    slot::pending pd = s.post_pending(old_buf, 4);
    CHECK(pd.ready() == -1 && pd.wait(5) == -1);
    CHECK(pd.cancel() && pd.cancel());
    s.put(2, [](void *p) {
        std::memcpy(p, "zz", 2);
        return true;
    });
    CHECK(old_buf[0] == '-');
    CHECK(s.get(dst, 8) && dst[0] == 'z');
    // delivered before the cancel: cancel reports it and the data is there
    slot::pending pd2 = s.post_pending(old_buf, 4);
    s.put(2, [](void *p) {
        std::memcpy(p, "in", 2);
        return true;
    });
    CHECK(!pd2.cancel() && pd2.ready() == 1 && old_buf[0] == 'i');

    auto pool = stdml::sync::thread_pool::make(3);
    std::atomic<int> sum{0};
    std::vector<stdml::sync::thread_pool::task> fs;
    for (int i = 1; i <= 20; ++i) {
        fs.emplace_back([&sum, i] { sum += i; });
    }
    pool->par(std::move(fs));
    CHECK(sum == 210);
    for (int i = 0; i < 5; ++i) {
        pool->add([&sum] { sum += 1; });
    }
    pool->wait();
    CHECK(sum == 215);
    bool threw = false;
    try {
        pool->par({[] { throw std::runtime_error("boom"); }, [] {}});
    } catch (const std::runtime_error &) {
        threw = true;
    }
    CHECK(threw);
    std::vector<int> xs = {1, 2, 3, 4};
    std::atomic<int> acc{0};
    fmap(par, [&](int x) { acc += x; }, xs);
    fmap(seq, [&](int x) { acc += x; }, xs);
    fmap(pool.get(), [&](int x) { acc += x; }, xs);
    fmap(static_cast<stdml::sync::thread_pool *>(nullptr), [&](int x) { acc += x; }, xs);
    CHECK(acc == 40);
    stdml::sync::wait_group wg;
    wg.add(2);
    std::thread a([&] { wg.done(); }), b([&] { wg.done(); });
    wg.wait();
    a.join();
    b.join();
}

static void test_tasks()
{
    std::vector<int> order;
    auto step = [&](int v) { return new simple_task([&order, v] { order.push_back(v); }); };
    task_builder s1, s2, top;
    s1 << step(11);
    s1 << step(12);
    s2 << step(21);
    s2 << step(22);
    top << s1.seq();
    top << s2.seq();
    std::unique_ptr<task> t(top.par());
    CHECK(!t->finished());
    t->finish();
    CHECK(t->finished() && order.size() == 4);
    auto pos = [&](int v) { return std::find(order.begin(), order.end(), v) - order.begin(); };
    CHECK(pos(11) < pos(12) && pos(21) < pos(22));

    int polls = 0;
    bool fired = false;
    poll_task p([&] { return ++polls >= 3; }, [&] { fired = true; });
    p.finish();
    CHECK(polls == 3 && fired);

    std::unique_ptr<runtime> rt(runtime::New(4));
    std::atomic<int> n{0};
    std::vector<std::unique_ptr<task>> many;
    for (int i = 0; i < 50; ++i) {
        many.emplace_back(new simple_task([&n] { ++n; }));
    }
    std::unique_ptr<task> all(task::par(std::move(many), rt.get()));
    all->finish();
    CHECK(n == 50);
    const size_t before = task_count();
    noop_task nt;
    CHECK(task_count() == before + 1 && nt.finished());
    monitored_task<noop_task> mt{noop_task()};
    mt.poll();
    CHECK(mt.finished());
    CHECK(task_name<noop_task>() == "stdml::collective::noop_task");
}

static void test_misc()
{
    CHECK(affinity_slice({0, 1, 2, 3, 4, 5, 6, 7}, 1, 4) == std::vector<int>({2, 3}));
    CHECK(affinity_slice({0, 1}, 3, 4) == std::vector<int>({1}));
    CHECK(parse_kungfu_startegy("RING") == ring && parse_kungfu_startegy("ring") == ring &&
          parse_kungfu_startegy("STAR") == star && parse_kungfu_startegy(nullptr) == star);
    setenv("STDML_TEST_BOOL", "On", 1);
    CHECK(parse_env_bool("STDML_TEST_BOOL") && !parse_env_bool("STDML_TEST_UNSET"));
    setenv("STDML_COLLECTIVE_USE_ASYNC", "1", 1);
    CHECK(parse_system_config_from_env().rt == rt_async);
    unsetenv("STDML_COLLECTIVE_USE_ASYNC");
    setenv("STDML_COLLECTIVE_USE_THREAD_POOL", "true", 1);
    const auto cfg = parse_system_config_from_env();
    CHECK(cfg.rt == rt_thread_pool && cfg.thread_pool_size > 0);
    unsetenv("STDML_COLLECTIVE_USE_THREAD_POOL");
    rchan::stat_enable();
    {
        STDML_COLLECTIVE_PROFILE_RATE("unit", 128);
    }
    CHECK(rchan::stat_events().size() == 1 && rchan::stat_events()[0].payload == 128);
    CHECK(rchan::stat_write_chrome_trace("/tmp/stdml_unit_trace.json"));
    rchan::stat_disable();
    rchan::stat_clear();
    CHECK(get_build_info().cuda_arch == "sm_100a");
    // a single peer needs no network at all
    peer p = peer::single();
    session s = p.join();
    CHECK(s.rank() == 0 && s.size() == 1);
    int x = 5;
    CHECK(s.all_reduce(x) == 5 && s.broadcast(x) == 5 && s.consistent(x));
}

static void test_sockets_and_io_tasks()
{
    // echo server: u32 length + body in, the same back
    TcpServer server(0, localhost);
    server.start();
    std::thread srv([&] {
        server.serve([](std::unique_ptr<TcpSocket> s) {
            uint32_t n = 0;
            if (s->recv(&n, 4) != 0) { return; }
            std::vector<char> body(n);
            if (n > 0 && s->recv(body.data(), n) != 0) { return; }
            s->send(&n, 4);
            s->send(body.data(), n);
        });
    });
    {
        TcpClient client(server.port());
        client.dial();
        const std::string msg(100000, 'q');
        const auto reply = client.Talk(msg.data(), msg.size());
        CHECK(reply.size() == msg.size() && reply[99999] == 'q');
    }
    // the same exchange as polled tasks on non-blocking sockets, one thread
    {
        TcpClient client(server.port());
        client.dial();
        TcpSocket &sock = client.socket();
        sock.set_non_blocking(true);
        using io = basic_ioutil<TcpSocket, true>;
        std::vector<char> out(300000, 'z'), in(300000, 0);
        uint32_t n = static_cast<uint32_t>(out.size()), m = 0;
        task_builder steps;
        steps << io::new_write_task(sock, &n, 4);
        steps << io::new_write_task(sock, out.data(), out.size());
        steps << io::new_read_task(sock, &m, 4);
        steps << io::new_read_task(sock, in.data(), in.size());
        std::unique_ptr<task> all(steps.seq());
        all->finish();
        CHECK(m == n && in == out);
    }
    int code = 0;
    TcpClient nobody(1);
    nobody.dial(&code);
    CHECK(code != 0);
    server.stop();
    srv.join();

    patient p(std::chrono::milliseconds(20));
    CHECK(p.ok() && !p.lost());
    std::this_thread::sleep_for(std::chrono::milliseconds(30));
    CHECK(!p.ok() && p.lost() && p.ok());
    CHECK(xterm::paint("ok", xterm::green) == "\x1b[32mok\x1b[0m");
    CHECK(xterm::paint("ok", xterm::green, false) == "ok");
}

// The shared-memory ring on its own: a small ring forces many wrap-arounds and
// both kinds of sleep (full and empty); close() ends a blocked reader.
static void test_shm_ring()
{
    const size_t cap = 4096;
    const int mfd = ::memfd_create("test-ring", MFD_CLOEXEC);
    REQUIRE(mfd >= 0);
    REQUIRE(::ftruncate(mfd, static_cast<off_t>(rchan::shm_ring::bytes_for(cap))) == 0);
    rchan::shm_ring tx, rx;
    REQUIRE(tx.open(mfd, cap, true, -1));
    REQUIRE(rx.open(mfd, cap, false, -1));
    rchan::shm_ring wrong;
    CHECK(!wrong.open(mfd, 2 * cap, false, -1));  // capacity in the header does not match
    ::close(mfd);

    const size_t total = 1 << 20;
    std::vector<uint8_t> src(total), dst(total, 0);
    for (size_t i = 0; i < total; ++i) { src[i] = static_cast<uint8_t>((i * 2654435761u) >> 13); }
    std::thread producer([&] {
        size_t at = 0, step = 1;
        while (at < total) {  // pieces from 1 byte to several rings long
            const size_t k = std::min(step, total - at);
            CHECK(tx.write(src.data() + at, k));
            at += k;
            step = step * 3 + 1;
            if (step > 3 * cap) { step = 1; }
        }
    });
    size_t at = 0, step = 7;
    while (at < total) {
        const size_t k = std::min(step, total - at);
        CHECK(rx.read(dst.data() + at, k));
        at += k;
        step = (step * 5 + 3) % (2 * cap) + 1;
    }
    producer.join();
    CHECK(src == dst);

    // bytes written before close() are still delivered; after them the reader gets end-of-stream
    CHECK(tx.write("tail", 4));
    std::thread closer([&] {
        std::this_thread::sleep_for(std::chrono::milliseconds(20));
        tx.close();
    });
    char tail[4];
    CHECK(rx.read(tail, 4) && std::memcmp(tail, "tail", 4) == 0);
    char more;
    CHECK(!rx.read(&more, 1));  // blocks until close() wakes it
    closer.join();
    CHECK(!tx.write(src.data(), 2 * cap));  // a writer to a closed ring gives up once it is full
}

int main()
{
    test_shm_ring();
    test_sockets_and_io_tasks();
    test_dtype();
    test_partition();
    test_topology();
    test_cluster_config();
    test_json_http();
    test_sync_primitives();
    test_tasks();
    test_misc();
    return testing::result("test-unit");
}
