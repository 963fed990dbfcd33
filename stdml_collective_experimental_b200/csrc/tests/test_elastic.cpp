// Elastic agreement under host-side fault injection (no launcher, no GPU):
//   * one rank's config provider is STALE for its first polls, so the members
//     disagree and resize() must keep polling until all see the same answer;
//   * one rank's provider fails (returns nothing) once;
//   * the removed rank learns `detached`, survivors get a new session (next
//     version) and keep working; a second resize to the same cluster is a no-op.
//   test_elastic
#include <cstdio>
#include <vector>

#include <sys/wait.h>
#include <unistd.h>

#include <stdml/collective>

using namespace stdml::collective;

static int rank_main(size_t rank, size_t np)
{
    peer p = peer::from_fork(rank, np);
    auto sess = p.join_elastic();
    const cluster_config old_cluster = sess->cluster();
    const cluster_config wanted = old_cluster.resize(np - 1);
    int polls = 0;
    auto provider = [&]() -> std::optional<cluster_config> {
        ++polls;
        if (rank == 1 && polls <= 3) { return old_cluster; }  // stale view
        if (rank == 0 && polls == 2) { return {}; }           // server hiccup
        return wanted;
    };
    int committed_version = -1;
    const resize_result r = p.resize(sess, provider, [&](cluster_config c, int v) {
        committed_version = v;
        if (!(c == wanted)) { committed_version = -100; }
    });
    if (!r.changed || committed_version != 1) { return 10; }
    if (polls < 4) { return 11; }  // everybody had to wait for the stale rank
    if (rank == np - 1) { return r.detached ? 0 : 12; }
    if (r.detached) { return 13; }
    if (sess->size() != np - 1 || sess->version() != 1 || sess->rank() != rank) { return 14; }
    if (sess->all_reduce(1) != static_cast<int>(np - 1)) { return 15; }
    // asking again for the membership we already have changes nothing
    const resize_result again = p.resize(sess, [&] { return std::optional<cluster_config>(wanted); });
    if (again.changed || again.detached || sess->version() != 1) { return 16; }
    std::vector<double> x(50000, 0.5), y(x.size());
    sess->all_reduce(x.data(), y.data(), x.size(), f64, sum, "after");
    return y[0] == 0.5 * (np - 1) ? 0 : 17;
}

int main()
{
    const size_t np = 3;
    std::vector<pid_t> kids;
    for (size_t r = 0; r < np; ++r) {
        const pid_t pid = ::fork();
        if (pid == 0) {
            int rc = 99;
            try {
                rc = rank_main(r, np);
            } catch (const std::exception &e) {
                std::fprintf(stderr, "rank %zu: %s\n", r, e.what());
            }
            ::_exit(rc);
        }
        kids.push_back(pid);
    }
    int bad = 0;
    for (size_t r = 0; r < np; ++r) {
        int st = 0;
        ::waitpid(kids[r], &st, 0);
        const int rc = WIFEXITED(st) ? WEXITSTATUS(st) : -1;
        if (rc != 0) {
            std::printf("rank %zu failed with %d\n", r, rc);
            ++bad;
        }
    }
    std::printf("test-elastic: %s\n", bad == 0 ? "OK" : "FAILED");
    return bad == 0 ? 0 : 1;
}
