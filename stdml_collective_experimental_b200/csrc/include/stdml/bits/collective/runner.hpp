// The launcher side of a job: starts the worker processes of this host with
// the environment contract that peer::from_env() reads, serves the cluster
// configuration over HTTP (GET returns it, PUT proposes a new one), and, in
// watch mode, listens for the "update" messages that workers send after they
// have agreed on a new configuration and starts the workers that joined.
//
// The reference relies on KungFu's Go launcher `kungfu-run` for all of this
// (scripts/bin/stdml-collective-run:15-53); nothing in the reference repository
// implements it.  This is a native replacement with the same division of
// labour and the same wire formats (conn_control message "update" carrying
// {"Version":v,"Cluster":{"Runners":[...],"Workers":[...]}}).
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include <stdml/bits/collective/address.hpp>
#include <stdml/bits/collective/http.hpp>
#include <stdml/bits/collective/rchan.hpp>
#include <stdml/bits/collective/topology.hpp>

namespace stdml::collective
{
struct runner_options {
    size_t np = 1;
    peer_id self{(127u << 24) | 1u, 38080};  // this runner
    // -H ip:slots,ip:slots: the hosts of the job in rank order.  One runner per
    // host (same command line, its own -self ip) starts that host's workers; the
    // first np slots are used.  Empty: everything on `self`.
    std::vector<std::pair<uint32_t, size_t>> hosts;
    uint16_t worker_base_port = 10000;
    strategy strat = star;
    bool watch = false;              // elastic: keep serving updates
    int config_port = -1;            // >= 0: serve the configuration on this port (0: any)
    std::string config_server_url;   // external config server instead
    std::string logdir;              // per-worker <ip>.<port>.{stdout,stderr}.log
    bool quiet = false;
    // Elastic growth without the start-up cost of a worker: keep this many warm
    // standby processes (the same program, run up to its peer::from_env(), where
    // it waits for an identity on a pipe from this launcher).  A worker that joins
    // is then a standby that is told who it is, not a fresh process.
    size_t spares = 0;
    std::vector<std::string> command;  // program and arguments
    std::vector<std::pair<std::string, std::string>> extra_env;
};

class runner
{
  public:
    explicit runner(runner_options opt);
    ~runner();

    // starts the initial workers, serves until every worker has exited (and, in
    // watch mode, no newer configuration is pending); returns the number of
    // workers that failed
    int run();

    const cluster_config &cluster() const { return cluster_; }
    std::string config_url() const;

    // called by the control handler
    void on_update(size_t version, const cluster_config &next);

  private:
    struct impl;
    runner_options opt_;
    cluster_config cluster_;
    size_t version_ = 0;
    std::mutex mu_;
    std::map<uint64_t, int> pids_;  // worker hash -> pid
    struct standby {
        int pid;
        int fd;  // write end of its identity pipe
    };
    std::vector<standby> standbys_;
    int failed_ = 0;
    std::unique_ptr<http_server> http_;
    std::unique_ptr<rchan::conn_handler> handler_;
    std::unique_ptr<rchan::server> server_;
    std::string stored_config_;  // what the config server returns

    // the environment contract of one worker (what peer::from_env() reads)
    std::vector<std::pair<std::string, std::string>> identity(const peer_id &worker,
                                                              const cluster_config &cluster,
                                                              size_t version) const;
    void spawn(const peer_id &worker, const cluster_config &cluster, size_t version);
    void spawn_standby();
    // true: a standby took the identity and is now that worker
    bool hand_over(const peer_id &worker, const cluster_config &cluster, size_t version);
    void dismiss_standbys();
    void reap(bool block);
    void stop_workers();
};

// parses the command line of the stdml-collective-run program
bool parse_runner_args(int argc, char *argv[], runner_options &out, std::string &error);
}  // namespace stdml::collective
