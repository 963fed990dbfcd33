// The same loop written with elastic_state: progress and resize checks are
// handled by the state object; membership follows the config server, so a
// proposal can come from anywhere (here: rank 0 follows a schedule).
//   stdml_collective_run -np 2 -w -builtin-config-port 0
//       example_elastic_state --max-step=9 2:4 5:3
// --die=PORT:STEP makes the worker that listens on PORT die at STEP: the others
// catch peer_failure and carry on without it (elastic_state::recover).
#include <cstdio>
#include <cstdlib>
#include <map>
#include <vector>

#include <stdml/collective>

using namespace stdml::collective;

int main(int argc, char *argv[])
{
    int max_step = 10;
    int die_port = -1, die_step = -1;
    std::map<int, int> schedule;
    for (int i = 1; i < argc; ++i) {
        int k, v;
        if (std::sscanf(argv[i], "--max-step=%d", &max_step) == 1) { continue; }
        if (std::sscanf(argv[i], "--die=%d:%d", &die_port, &die_step) == 2) { continue; }
        if (std::sscanf(argv[i], "%d:%d", &k, &v) == 2) { schedule[k] = v; }
    }
    std::vector<float> weights(1024, 0.0f);
    elastic_state state(max_step);
    state.on_resize([&](session &s) {
        s.broadcast(weights.data(), weights.data(), weights.size(), f32, "state", nullptr,
                    state.state_root());
        std::printf("  resized: rank %zu of %zu\n", s.rank(), s.size());
    });
    while (!state.should_stop()) {
        try {
            const int step = static_cast<int>(static_cast<int64_t>(state));
            if (step == die_step && state.get_peer().self().port == die_port) {
                std::printf("  dying at step %d\n", step);
                std::fflush(stdout);
                std::_Exit(3);
            }
            session &sess = state.sess();
            std::vector<float> g(weights.size(), float(step + 1)), total(weights.size());
            sess.all_reduce(g.data(), total.data(), g.size(), f32, sum, "grad");
            for (size_t i = 0; i < weights.size(); ++i) { weights[i] += total[i] / sess.size(); }
            if (sess.rank() == 0 && schedule.count(step) != 0) {
                propose_new_size(sess.cluster(), static_cast<size_t>(schedule[step]));
            }
            ++state;
        } catch (const peer_failure &e) {
            const peer_list dropped = state.recover();
            std::printf("  lost %s, carrying on with %zu members\n", dropped[0].str().c_str(),
                        state.sess().size());
        }
    }
    if (state.detached()) {
        std::printf("detached\n");
        return 0;
    }
    const float want = max_step * (max_step + 1) / 2.0f;
    const bool ok = weights[0] == want;
    std::printf("finished at step %lld: weight %.1f (want %.1f) %s\n",
                static_cast<long long>(static_cast<int64_t>(state)), weights[0], want,
                ok ? "OK" : "WRONG");
    return ok ? 0 : 1;
}
