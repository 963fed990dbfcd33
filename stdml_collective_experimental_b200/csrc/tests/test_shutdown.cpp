// Clean teardown: many collectives, then an explicit stop; and failure
// detection on the host path: a rank that leaves before a collective makes the
// others throw (instead of blocking for ever) when
// STDML_COLLECTIVE_HOST_TIMEOUT_MS is set.
//   test_shutdown <np>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include <sys/wait.h>
#include <unistd.h>

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

// rank 1 exits without taking part; rank 0 must notice within the timeout
static int peer_leaves(int np)
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
                if (r == 1) { ::_exit(0); }  // gone between two steps
                float x = 1, y = 0;
                sess.all_reduce(&x, &y, 1, f32, sum, "after");
                rc = 4;  // must not succeed
            } catch (const std::runtime_error &e) {
                rc = std::string(e.what()).find("within 500 ms") != std::string::npos ? 0 : 5;
            }
            ::_exit(rc);
        }
        kids.push_back(pid);
    }
    int bad = 0;
    for (pid_t pid : kids) {
        int st = 0;
        ::waitpid(pid, &st, 0);
        if (!WIFEXITED(st) || WEXITSTATUS(st) != 0) { ++bad; }
    }
    ::unsetenv("STDML_COLLECTIVE_HOST_TIMEOUT_MS");
    if (bad != 0) { std::printf("peer leaves: FAILED (%d ranks)\n", bad); }
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
    const int bad = clean_shutdown(np) + peer_leaves(np) + peer_never_joins();
    std::printf("test-shutdown np=%d: %s\n", np, bad == 0 ? "OK" : "FAILED");
    return bad == 0 ? 0 : 1;
}
