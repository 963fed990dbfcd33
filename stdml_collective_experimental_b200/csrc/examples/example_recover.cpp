// Unplanned loss of a member: a training-style loop that survives it.
//
//   example_recover [np] [victim] [at_step]
//
// forks np ranks; rank `victim` dies at step `at_step`; the others catch
// peer_failure, call peer::recover(), agree on the step to resume from and
// finish as a world of np - 1.  (The reference handles planned resizes only
// and blocks for ever when a member dies.)
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <vector>

#include <sys/wait.h>
#include <unistd.h>

#include <stdml/collective>

using namespace stdml::collective;

int main(int argc, char *argv[])
{
    const int np = argc > 1 ? std::atoi(argv[1]) : 4;
    const int victim = argc > 2 ? std::atoi(argv[2]) : 1;
    const int at_step = argc > 3 ? std::atoi(argv[3]) : 3;
    const int steps = 8;
    std::vector<pid_t> kids;
    for (int r = 0; r < np; ++r) {
        const pid_t pid = ::fork();
        if (pid == 0) {
            peer p = peer::from_fork(r, np);
            std::unique_ptr<session> sess = p.join_elastic();
            std::vector<float> weights(1000, 0.0f), grad(1000), sum(1000);
            int64_t step = 0;
            while (step < steps) {
                if (r == victim && step == at_step) { ::_exit(0); }
                try {
                    std::fill(grad.begin(), grad.end(), 1.0f);
                    sess->all_reduce(grad.data(), sum.data(), grad.size(), f32, stdml::collective::sum,
                                     "grad");
                    for (size_t i = 0; i < weights.size(); ++i) { weights[i] += sum[i] / sess->size(); }
                    ++step;
                } catch (const peer_failure &e) {
                    std::printf("[%d] step %d: %s\n", r, int(step), e.what());
                    const peer_list dropped = p.recover(sess);
                    // a step that failed here may have finished elsewhere: take the
                    // furthest rank's progress and the first rank's weights
                    step = sess->all_reduce(step, max);
                    sess->broadcast(weights.data(), weights.data(), weights.size(), f32, "weights");
                    std::printf("[%d] carrying on as rank %d of %d without %s, from step %d\n", r,
                                int(sess->rank()), int(sess->size()), dropped[0].str().c_str(),
                                int(step));
                }
            }
            std::printf("[%d] done: %d members, version %d\n", r, int(sess->size()),
                        int(sess->version()));
            std::fflush(stdout);
            ::_exit(sess->size() == size_t(np - 1) ? 0 : 1);
        }
        kids.push_back(pid);
    }
    int bad = 0;
    for (pid_t pid : kids) {
        int st = 0;
        ::waitpid(pid, &st, 0);
        if (!WIFEXITED(st) || WEXITSTATUS(st) != 0) { ++bad; }
    }
    std::printf("example-recover: %s\n", bad == 0 ? "OK" : "FAILED");
    return bad == 0 ? 0 : 1;
}
