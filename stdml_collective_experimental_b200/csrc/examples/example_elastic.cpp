// Elastic data-parallel loop driven by a resize schedule:
//   stdml_collective_run -np 4 -w -builtin-config-port 0
//       example_elastic --max-step=12 3:2 6:3 9:4
// "3:2" = after step 3 resize to 2 workers.  Survivors keep running; joiners
// are started by the runner and catch up: the step counter by a max-all-reduce
// (as in the reference's examples/example-elastic.cpp:43-51) and the model
// state by a broadcast from rank 0 (which the reference leaves to the user).
#include <cstdio>
#include <cstdlib>
#include <map>
#include <vector>

#include <stdml/collective>

using namespace stdml::collective;

int main(int argc, char *argv[])
{
    int max_step = 10;
    std::map<int, int> schedule;
    for (int i = 1; i < argc; ++i) {
        int k, v;
        if (std::sscanf(argv[i], "--max-step=%d", &max_step) == 1) { continue; }
        if (std::sscanf(argv[i], "%d:%d", &k, &v) == 2) { schedule[k] = v; }
    }
    auto p = peer::from_env();
    auto sess = p.join_elastic();
    std::printf("[%s] joined: rank %zu of %zu, version %zu\n", p.self().str().c_str(),
                sess->rank(), sess->size(), sess->version());

    std::vector<float> weights(4096, 0.0f), grad(4096), sum_grad(4096);
    bool synced = false;
    for (int step = 0; step < max_step; ++step) {
        if (!synced) {
            // whoever is furthest ahead defines the step; rank 0 defines the state
            step = sess->all_reduce(step, max);
            sess->broadcast(weights.data(), weights.data(), weights.size(), f32, "state");
            synced = true;
            if (step >= max_step) { break; }
        }
        for (size_t i = 0; i < grad.size(); ++i) { grad[i] = float(step + 1); }
        sess->all_reduce(grad.data(), sum_grad.data(), grad.size(), f32, sum, "grad");
        for (size_t i = 0; i < weights.size(); ++i) { weights[i] += sum_grad[i] / sess->size(); }
        if (schedule.count(step) != 0) {
            const auto [changed, detached] = p.resize(sess, static_cast<size_t>(schedule[step]));
            if (detached) {
                std::printf("[%s] detached after step %d\n", p.self().str().c_str(), step);
                return 0;
            }
            if (changed) {
                std::printf("[%s] resized after step %d: rank %zu of %zu, version %zu\n",
                            p.self().str().c_str(), step, sess->rank(), sess->size(),
                            sess->version());
                synced = false;
            }
        }
    }
    // every step adds (step + 1) to every weight, whatever the membership was
    const float want = max_step * (max_step + 1) / 2.0f;
    const bool ok = weights[0] == want && weights.back() == want &&
                    sess->consistent(weights.data(), weights.size() * sizeof(float));
    std::printf("[%s] finished: rank %zu of %zu, weight %.1f (want %.1f) %s\n",
                p.self().str().c_str(), sess->rank(), sess->size(), weights[0], want,
                ok ? "OK" : "WRONG");
    return ok ? 0 : 1;
}
