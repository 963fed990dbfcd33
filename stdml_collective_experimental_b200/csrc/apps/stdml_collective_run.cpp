// stdml_collective_run: start the workers of one host.
//
//   stdml_collective_run -np 4 [-strategy RING] [-w -builtin-config-port 9100]
//                        [-logdir logs] [-q] [-env NAME=VALUE]... prog [args...]
//
// -w keeps the runner listening for membership updates (elastic jobs); the
// built-in config server answers GET/PUT on http://127.0.0.1:<port>/config and
// its URL is handed to the workers as KUNGFU_CONFIG_SERVER.
#include <cstdio>

#include <stdml/bits/collective/runner.hpp>

int main(int argc, char *argv[])
{
    stdml::collective::runner_options opt;
    std::string error;
    if (!stdml::collective::parse_runner_args(argc, argv, opt, error)) {
        std::fprintf(stderr, "%s: %s\nusage: %s -np N [-strategy STAR|RING|BINARY_TREE|CLIQUE] [-w] "
                             "[-builtin-config-port P] [-config-server URL] [-logdir DIR] [-q] "
                             "[-runner-port P] [-port-range P] [-env K=V] [-spares N] "
                             "[-H ip:slots,ip:slots -self ip] prog [args...]\n",
                     argv[0], error.c_str(), argv[0]);
        return 2;
    }
    try {
        stdml::collective::runner r(opt);
        const int failed = r.run();
        return failed == 0 ? 0 : 1;
    } catch (const std::exception &e) {
        std::fprintf(stderr, "%s: %s\n", argv[0], e.what());
        return 1;
    }
}
