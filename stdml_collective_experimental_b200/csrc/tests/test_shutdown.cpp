// Clean teardown: many collectives, then an explicit stop; and failure
// detection on the host path: a rank that leaves before a collective makes the
// others throw peer_failure (no timeout needed), a rank that is alive but
// silent makes them throw when STDML_COLLECTIVE_HOST_TIMEOUT_MS runs out, a
// rank that never shows up ends the connect timeout, and conn_ping tells a
// live address from a dead one.
//   test_shutdown <np>
#include <chrono>
#include <cstdint>
#include <memory>
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <thread>
#include <vector>

#include <sys/wait.h>
#include <unistd.h>

#include <stdml/bits/collective/net/tcp.hpp>
#include <stdml/collective>

using namespace stdml::collective;

static int clean_shutdown(int np)
{
    try {
        prun(np, [](session &sess) {
            std::vector<float> x(1000, 1.0f), y(1000);
            for (int i = 0; i < 100; ++i) {
                sess.all_reduce(x.data(), y.data(), x.size(), f32, sum, "x" + std::to_string(i % 3));
                if (y[0] != float(sess.size())) { throw std::runtime_error("wrong sum"); }
            }
        });
    } catch (const std::exception &e) {
        std::printf("clean shutdown: FAILED (%s)\n", e.what());
        return 1;
    }
    return 0;
}

static int reap(const std::vector<pid_t> &kids, const char *what)
{
    int bad = 0;
    for (pid_t pid : kids) {
        int st = 0;
        ::waitpid(pid, &st, 0);
        if (!WIFEXITED(st) || WEXITSTATUS(st) != 0) {
            std::printf("%s: a rank ended with status %d\n", what, WIFEXITED(st) ? WEXITSTATUS(st) : -1);
            ++bad;
        }
    }
    if (bad != 0) { std::printf("%s: FAILED (%d ranks)\n", what, bad); }
    return bad;
}

// Rank 1 exits between two steps.  No timeout is configured: the others must
// learn from its closed connections that it has gone (peer_failure, within a
// few wait slices), directly or because the rank they wait for gave up.
static int peer_leaves(int np, bool async_runtime)
{
    if (async_runtime) { ::setenv("STDML_COLLECTIVE_USE_ASYNC", "1", 1); }
    std::vector<pid_t> kids;
    for (int r = 0; r < np; ++r) {
        const pid_t pid = ::fork();
        if (pid == 0) {
            int rc = 3;
            try {
                peer p = peer::from_fork(r, np);
                session sess = p.join();
                if (r == 1) { ::_exit(0); }  // gone between two steps
                const auto t0 = std::chrono::steady_clock::now();
                try {
                    std::vector<float> x(300000, 1.0f), y(300000);
                    sess.all_reduce(x.data(), y.data(), x.size(), f32, sum, "after");
                    rc = 4;  // must not succeed
                } catch (const peer_failure &e) {
                    const double s =
                        std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
                    rc = s < 5.0 ? 0 : 6;
                }
            } catch (const std::exception &e) {
                std::printf("rank %d: %s\n", r, e.what());
                rc = 5;
            }
            ::_exit(rc);
        }
        kids.push_back(pid);
    }
    const int bad = reap(kids, async_runtime ? "peer leaves (polled tasks)" : "peer leaves");
    ::unsetenv("STDML_COLLECTIVE_USE_ASYNC");
    return bad;
}

// Rank 1 stays alive but silent: only the timeout can end the wait.
static int peer_stalls(int np)
{
    ::setenv("STDML_COLLECTIVE_HOST_TIMEOUT_MS", "500", 1);
    std::vector<pid_t> kids;
    for (int r = 0; r < np; ++r) {
        const pid_t pid = ::fork();
        if (pid == 0) {
            int rc = 3;
            try {
                peer p = peer::from_fork(r, np);
                session sess = p.join();
                if (r == 1) {
                    std::this_thread::sleep_for(std::chrono::seconds(3));
                    ::_exit(0);
                }
                float x = 1, y = 0;
                sess.all_reduce(&x, &y, 1, f32, sum, "after");
                rc = 4;  // must not succeed
            } catch (const peer_failure &) {
                rc = r == 0 ? 7 : 0;  // rank 0 waits for the silent rank itself; the rest may see rank 0 go
            } catch (const std::runtime_error &e) {
                rc = std::string(e.what()).find("within 500 ms") != std::string::npos ? 0 : 5;
            }
            ::_exit(rc);
        }
        kids.push_back(pid);
    }
    const int bad = reap(kids, "peer stalls");
    ::unsetenv("STDML_COLLECTIVE_HOST_TIMEOUT_MS");
    return bad;
}

// Rank 0 dies before it has sent anything: rank 1 has no connection of it to
// watch, so after a dialler's patience it pings the address and gives up.
static int peer_dies_before_connecting()
{
    ::setenv("STDML_COLLECTIVE_CONNECT_TIMEOUT_MS", "500", 1);
    std::vector<pid_t> kids;
    for (int r = 0; r < 2; ++r) {
        const pid_t pid = ::fork();
        if (pid == 0) {
            int rc = 3;
            try {
                peer p = peer::from_list(r, *parse_peer_list("127.0.0.1:10460,127.0.0.1:10461"), star);
                if (r == 0) {
                    std::this_thread::sleep_for(std::chrono::milliseconds(300));
                    ::_exit(0);  // listened, never joined
                }
                session sess = p.join();
                rc = 4;  // must not succeed
            } catch (const peer_failure &) {
                rc = 0;
            } catch (const std::runtime_error &e) {
                // started too late to reach rank 0 at all
                rc = std::string(e.what()).find("could not reach") != std::string::npos ? 0 : 5;
            }
            ::_exit(rc);
        }
        kids.push_back(pid);
    }
    const int bad = reap(kids, "peer dies before connecting");
    ::unsetenv("STDML_COLLECTIVE_CONNECT_TIMEOUT_MS");
    return bad;
}

// Unplanned loss: rank 2 dies at step 3 of 8; the others catch peer_failure,
// call recover() and finish the remaining steps as a world of np - 1.
static int member_lost_and_recovered(int np, bool async_runtime)
{
    if (np < 3) { return 0; }
    if (async_runtime) { ::setenv("STDML_COLLECTIVE_USE_ASYNC", "1", 1); }
    std::vector<pid_t> kids;
    for (int r = 0; r < np; ++r) {
        const pid_t pid = ::fork();
        if (pid == 0) {
            int rc = 3;
            try {
                peer p = peer::from_fork(r, np);
                std::unique_ptr<session> sess = p.join_elastic();
                int recoveries = 0;
                int64_t step = 0;
                while (step < 8) {
                    if (r == 2 && step == 3) { ::_exit(0); }
                    try {
                        std::vector<float> x(50000, 1.0f), y(50000, 0.0f);
                        sess->all_reduce(x.data(), y.data(), x.size(), f32, sum, "g" + std::to_string(step));
                        if (y[0] != float(sess->size()) || y.back() != y[0]) { ::_exit(7); }
                        ++step;
                    } catch (const peer_failure &) {
                        const peer_list dropped = p.recover(sess);
                        ++recoveries;
                        if (dropped.size() != 1 || sess->size() != size_t(np - 1)) { ::_exit(8); }
                        // some may have finished the step that failed here: agree on where to go on
                        step = sess->all_reduce(step, max);
                    }
                }
                rc = (recoveries == 1 && sess->version() == 1) ? 0 : 9;
            } catch (const std::exception &e) {
                std::printf("rank %d: %s\n", r, e.what());
                std::fflush(stdout);
                rc = 5;
            }
            ::_exit(rc);
        }
        kids.push_back(pid);
    }
    const int bad = reap(kids, async_runtime ? "member lost and recovered (polled tasks)"
                                             : "member lost and recovered");
    ::unsetenv("STDML_COLLECTIVE_USE_ASYNC");
    return bad;
}

// Survivors whose probes disagree: rank 3 dies; rank 0's probe of rank 2, which
// is alive, is made to fail.  Ranks 0 and 1 must end up in ONE session of two
// members and finish; rank 2 must be told that it was left out (peer_failure
// from its own recover()), not form a session of its own.
static int survivors_disagree()
{
    const int np = 4;
    std::vector<pid_t> kids;
    for (int r = 0; r < np; ++r) {
        const pid_t pid = ::fork();
        if (pid == 0) {
            int rc = 3;
            try {
                peer p = peer::from_fork(r, np);
                std::unique_ptr<session> sess = p.join_elastic();
                const peer_list members = sess->peers();
                int64_t step = 0;
                bool left_out = false;
                while (step < 6 && !left_out) {
                    if (r == 3 && step == 2) { ::_exit(0); }
                    try {
                        std::vector<float> x(20000, 1.0f), y(20000, 0.0f);
                        sess->all_reduce(x.data(), y.data(), x.size(), f32, sum, "d" + std::to_string(step));
                        if (y[0] != float(sess->size())) { ::_exit(7); }
                        ++step;
                    } catch (const peer_failure &) {
                        try {
                            p.recover(sess, 300, [&](const peer_id &q) {
                                if (r == 0 && q == members[2]) { return false; }  // the injected miss
                                return p.ping(q, 300) >= 0;
                            });
                        } catch (const peer_failure &) {
                            left_out = true;
                            break;
                        }
                        if (sess->size() != 2 || sess->peers()[0] != members[0] ||
                            sess->peers()[1] != members[1]) {
                            ::_exit(8);
                        }
                        step = sess->all_reduce(step, max);
                    }
                }
                if (r == 2) {
                    rc = left_out ? 0 : 9;
                } else {
                    rc = (!left_out && sess->version() == 1) ? 0 : 10;
                }
            } catch (const std::exception &e) {
                std::printf("rank %d: %s\n", r, e.what());
                std::fflush(stdout);
                rc = 5;
            }
            ::_exit(rc);
        }
        kids.push_back(pid);
    }
    return reap(kids, "survivors disagree");
}

// Bytes that are not this protocol (a port scanner, an HTTP client, a half-sent
// header) must neither crash a peer nor disturb its collectives.
static int stray_connections()
{
    int bad = 0;
    try {
        prun(2, [&](session &sess) {
            const peer_id other = sess.peers()[1 - sess.rank()];
            const auto knock = [&](const std::string &bytes) {
                TcpClient c(other.port, other.ipv4);
                int code = 0;
                c.dial(&code);
                if (code == 0 && !bytes.empty()) { c.write(bytes.data(), bytes.size()); }
            };  // closed here
            knock("");                                   // connects and leaves
            knock("GET / HTTP/1.1\r\nHost: x\r\n\r\n");  // another protocol altogether
            knock(std::string("\x02\x00\x10\x27\x01\x00\x00\x7f", 8) +  // a valid handshake ...
                  std::string("\xff\xff\xff\x7f", 4));                    // ... then an absurd name length
            knock(std::string("\x02\x00\x10\x27\x01\x00\x00\x7f", 8) +
                  std::string("\x03\x00\x00\x00" "abc", 7));  // a header that stops half way
            for (int i = 0; i < 20; ++i) {
                std::vector<int> x(1000, int(sess.rank()) + i), y(1000);
                sess.all_reduce(x.data(), y.data(), x.size(), i32, sum, "after-strays");
                if (y[0] != 2 * i + 1 || y[999] != y[0]) { throw std::runtime_error("wrong sum"); }
            }
        });
    } catch (const std::exception &e) {
        std::printf("stray connections: FAILED (%s)\n", e.what());
        bad = 1;
    }
    return bad;
}

// conn_ping: a live peer answers, a dead address does not
static int ping_peers()
{
    int bad = 0;
    try {
        prun(2, [&](session &sess) {
            // prun gives each rank its peer through the session's client pool owner;
            // the handshake itself needs no session
            const peer_id other = sess.peers()[1 - sess.rank()];
            const double us = rchan::ping(other, sess.peers()[sess.rank()], 1000);
            if (us < 0) { throw std::runtime_error("a live peer did not answer the ping"); }
            const peer_id nobody{other.ipv4, static_cast<uint16_t>(other.port + 977)};
            if (rchan::ping(nobody, sess.peers()[sess.rank()], 200) >= 0) {
                throw std::runtime_error("a dead address answered the ping");
            }
            sess.barrier();
        });
    } catch (const std::exception &e) {
        std::printf("ping: FAILED (%s)\n", e.what());
        bad = 1;
    }
    return bad;
}

// a peer that never shows up: the connect timeout turns into an exception
static int peer_never_joins()
{
    ::setenv("STDML_COLLECTIVE_CONNECT_TIMEOUT_MS", "300", 1);
    const pid_t pid = ::fork();
    if (pid == 0) {
        int rc = 1;
        try {
            peer p = peer::from_list(0, *parse_peer_list("127.0.0.1:10450,127.0.0.1:10451"), ring);
            session sess = p.join();  // the barrier dials rank 1, which does not exist
        } catch (const std::runtime_error &e) {
            rc = std::string(e.what()).find("could not reach") != std::string::npos ? 0 : 2;
        }
        ::_exit(rc);
    }
    int st = 0;
    ::waitpid(pid, &st, 0);
    const int bad = (WIFEXITED(st) && WEXITSTATUS(st) == 0) ? 0 : 1;
    if (bad) { std::printf("peer never joins: FAILED\n"); }
    return bad;
}

int main(int argc, char *argv[])
{
    const int np = argc > 1 ? std::atoi(argv[1]) : 4;
    const bool verbose = std::getenv("TEST_SHUTDOWN_VERBOSE") != nullptr;
    int bad = 0;
    const auto run = [&](const char *name, const std::function<int()> &f) {
        if (verbose) {
            std::printf("... %s\n", name);
            std::fflush(stdout);
        }
        bad += f();
    };
    run("clean shutdown", [&] { return clean_shutdown(np); });
    run("peer leaves", [&] { return peer_leaves(np, false); });
    run("peer leaves (polled tasks)", [&] { return peer_leaves(np, true); });
    run("peer stalls", [&] { return peer_stalls(np); });
    run("peer never joins", [&] { return peer_never_joins(); });
    run("peer dies before connecting", [&] { return peer_dies_before_connecting(); });
    run("member lost and recovered", [&] { return member_lost_and_recovered(np, false); });
    run("member lost and recovered (polled tasks)", [&] { return member_lost_and_recovered(np, true); });
    run("survivors disagree", [&] { return survivors_disagree(); });
    run("stray connections", [&] { return stray_connections(); });
    run("ping", [&] { return ping_peers(); });
    std::printf("test-shutdown np=%d: %s\n", np, bad == 0 ? "OK" : "FAILED");
    return bad == 0 ? 0 : 1;
}
