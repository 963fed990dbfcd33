// The same-host rendezvous used while a device world is set up, checked
// without a GPU: full mesh among forked ranks, byte and descriptor exchange
// (a memfd stands in for an exported CUDA allocation), agreement, and a rank
// that never shows up (exception after the timeout, no descriptor left open).
//   test_rendezvous [np]
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include <dirent.h>
#include <sys/mman.h>
#include <sys/wait.h>
#include <unistd.h>

#include "../cuda/local_rendezvous.hpp"
#include "testing.hpp"

using stdml::collective::cuda::LocalRendezvous;

static int open_descriptors()
{
    int n = 0;
    if (DIR *d = ::opendir("/proc/self/fd")) {
        while (::readdir(d) != nullptr) { ++n; }
        ::closedir(d);
    }
    return n;
}

static int rank_main(const std::string &key, int r, int np)
{
    LocalRendezvous rdv(key, r, np, 20000);
    // bytes
    const int mine = 100 + r;
    std::vector<std::vector<char>> all;
    rdv.all_gather(&mine, sizeof(mine), all);
    for (int p = 0; p < np; ++p) {
        int v;
        std::memcpy(&v, all[p].data(), sizeof(v));
        CHECK(v == 100 + p);
    }
    // a contribution far larger than a socket buffer (every rank sends before it receives)
    {
        std::vector<unsigned char> big((3u << 20) + 7);
        for (size_t i = 0; i < big.size(); ++i) { big[i] = static_cast<unsigned char>(i * 31 + r); }
        rdv.all_gather(big.data(), big.size(), all);
        for (int p = 0; p < np; ++p) {
            CHECK(all[p].size() == big.size());
            bool same = true;
            for (size_t i = 0; i < big.size() && same; i += 4093) {
                same = static_cast<unsigned char>(all[p][i]) == static_cast<unsigned char>(i * 31 + p);
            }
            CHECK(same);
        }
        rdv.all_gather(nullptr, 0, all);  // nothing to say is fine too
    }
    // descriptors: everybody shares a page that names its owner
    const int mfd = ::memfd_create("rdv-test", MFD_CLOEXEC);
    REQUIRE(mfd >= 0);
    REQUIRE(::ftruncate(mfd, 4096) == 0);
    const std::string text = "page of rank " + std::to_string(r);
    REQUIRE(::pwrite(mfd, text.data(), text.size(), 0) == static_cast<ssize_t>(text.size()));
    const std::vector<int> fds = rdv.all_gather_fd(mfd);
    ::close(mfd);
    for (int p = 0; p < np; ++p) {
        if (p == r) {
            CHECK(fds[p] == -1);
            continue;
        }
        char buf[64] = {0};
        CHECK(::pread(fds[p], buf, sizeof(buf) - 1, 0) > 0);
        CHECK(std::string(buf) == "page of rank " + std::to_string(p));
        ::close(fds[p]);
    }
    // agreement is a logical AND, and a barrier
    CHECK(rdv.all_agree(true));
    CHECK(!rdv.all_agree(r != np - 1));
    // point to point
    if (r == 0) {
        for (int p = 1; p < np; ++p) { rdv.send_bytes(p, "hi", 2); }
    } else {
        char hi[2];
        rdv.recv_bytes(0, hi, 2);
        CHECK(hi[0] == 'h' && hi[1] == 'i');
    }
    rdv.barrier();
    return testing::failures();
}

int main(int argc, char *argv[])
{
    const int np = argc > 1 ? std::atoi(argv[1]) : 4;
    const std::string key = "test-" + std::to_string(::getpid());
    std::vector<pid_t> kids;
    for (int r = 0; r < np; ++r) {
        const pid_t pid = ::fork();
        if (pid == 0) {
            int rc = 1;
            try {
                rc = rank_main(key, r, np) == 0 ? 0 : 1;
            } catch (const std::exception &e) {
                std::printf("rank %d: %s\n", r, e.what());
            }
            ::_exit(rc);
        }
        kids.push_back(pid);
    }
    for (pid_t pid : kids) {
        int st = 0;
        ::waitpid(pid, &st, 0);
        CHECK(WIFEXITED(st) && WEXITSTATUS(st) == 0);
    }

    // a world of two whose other rank never comes: in time, with nothing left open
    const int before = open_descriptors();
    bool threw = false;
    try {
        LocalRendezvous lonely(key + "-lonely", 1, 2, 300);  // rank 1 dials rank 0
    } catch (const std::runtime_error &e) {
        threw = std::string(e.what()).find("did not show up") != std::string::npos;
    }
    CHECK(threw);
    threw = false;
    try {
        LocalRendezvous lonely(key + "-lonely", 0, 2, 300);  // rank 0 waits to be dialled
    } catch (const std::runtime_error &) {
        threw = true;
    }
    CHECK(threw);
    CHECK(open_descriptors() == before);
    // a world of one needs nobody
    LocalRendezvous alone(key + "-alone", 0, 1, 100);
    CHECK(alone.all_agree(true));
    return testing::result("test-rendezvous");
}
