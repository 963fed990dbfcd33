#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <thread>

#include <csignal>

#include <fcntl.h>
#include <sys/stat.h>
#include <sys/wait.h>
#include <unistd.h>

#include <stdml/bits/collective/json.hpp>
#include <stdml/bits/collective/log.hpp>
#include <stdml/bits/collective/peer.hpp>
#include <stdml/bits/collective/runner.hpp>

namespace stdml::collective
{
namespace
{
// set by SIGINT / SIGTERM: the run loop then stops the workers and leaves
volatile std::sig_atomic_t g_stop_signal = 0;

void on_stop_signal(int sig) { g_stop_signal = sig; }

class control_msg_handler final : public rchan::msg_handler
{
    runner *runner_;

  public:
    explicit control_msg_handler(runner *r) : runner_(r) {}

    bool operator()(const rchan::received_header &mh, rchan::message_reader *reader,
                    const peer_id &) override
    {
        std::string body(mh.len, '\0');
        if (!reader->read_body(body.data())) { return false; }
        if (mh.name != "update") { return true; }
        const auto v = json::parse(body);
        if (!v) { return true; }
        const json::value *ver = v->get("Version");
        const json::value *cl = v->get("Cluster");
        if (ver == nullptr || cl == nullptr) { return true; }
        const auto next = cluster_config::from_json(cl->dump());
        if (next) { runner_->on_update(static_cast<size_t>(ver->as_int()), *next); }
        return true;
    }
};

class control_conn_handler final : public rchan::conn_handler
{
    control_msg_handler h_;

  public:
    explicit control_conn_handler(runner *r) : h_(r) {}
    size_t operator()(std::unique_ptr<rchan::connection> conn) override
    {
        return handle_to_end(conn.get(), &h_);
    }
};
}  // namespace

runner::runner(runner_options opt) : opt_(std::move(opt))
{
    peer_list workers, runners;
    if (opt_.hosts.empty()) {
        for (size_t i = 0; i < opt_.np; ++i) {
            workers.push_back(
                peer_id{opt_.self.ipv4, static_cast<uint16_t>(opt_.worker_base_port + i)});
        }
        runners.push_back(opt_.self);
    } else {
        bool mine = false;
        size_t slots = 0;
        for (const auto &[ip, n] : opt_.hosts) {
            runners.push_back(peer_id{ip, opt_.self.port});
            for (size_t j = 0; j < n && workers.size() < opt_.np; ++j) {
                workers.push_back(peer_id{ip, static_cast<uint16_t>(opt_.worker_base_port + j)});
            }
            mine = mine || ip == opt_.self.ipv4;
            slots += n;
        }
        if (slots < opt_.np) { throw std::invalid_argument("runner: -H offers fewer slots than -np"); }
        if (!mine) { throw std::invalid_argument("runner: -self is not one of the hosts of -H"); }
        if (opt_.config_port == 0) {
            throw std::invalid_argument(
                "runner: with several hosts the config server needs a fixed -builtin-config-port");
        }
    }
    cluster_ = cluster_config(runners, workers);
    stored_config_ = cluster_.json();
}

runner::~runner()
{
    if (server_) { server_->stop(); }
    if (http_) { http_->stop(); }
}

std::string runner::config_url() const
{
    if (!opt_.config_server_url.empty()) { return opt_.config_server_url; }
    if (http_) { return "http://127.0.0.1:" + std::to_string(http_->port()) + "/config"; }
    if (!opt_.hosts.empty() && opt_.config_port > 0) {
        // served by the first host's runner
        return "http://" + peer_id{opt_.hosts[0].first, 0}.hostname() + ":" +
               std::to_string(opt_.config_port) + "/config";
    }
    return "";
}

std::vector<std::pair<std::string, std::string>> runner::identity(const peer_id &worker,
                                                                  const cluster_config &cluster,
                                                                  size_t version) const
{
    std::string peers;
    for (size_t i = 0; i < cluster.workers.size(); ++i) {
        peers += (i ? "," : "") + cluster.workers[i].str();
    }
    std::string runners;
    for (size_t i = 0; i < cluster.runners.size(); ++i) {
        runners += (i ? "," : "") + cluster.runners[i].str();
    }
    std::vector<std::pair<std::string, std::string>> env;
    env.emplace_back("KUNGFU_SELF_SPEC", worker.str());
    env.emplace_back("KUNGFU_INIT_PEERS", peers);
    env.emplace_back("KUNGFU_INIT_RUNNERS", runners);
    env.emplace_back("KUNGFU_INIT_CLUSTER_VERSION", std::to_string(version));
    env.emplace_back("KUNGFU_ALLREDUCE_STRATEGY", strategy_name(opt_.strat));
    const std::string url = config_url();
    if (!url.empty()) { env.emplace_back("KUNGFU_CONFIG_SERVER", url); }
    // a worker keeps its GPU for life: the index follows its port, not its rank
    env.emplace_back("STDML_COLLECTIVE_DEVICE_ID",
                     std::to_string(worker.port - opt_.worker_base_port));
    return env;
}

namespace
{
void redirect_output(const std::string &logdir, const std::string &name)
{
    if (logdir.empty()) { return; }
    ::mkdir(logdir.c_str(), 0755);
    const std::string base = logdir + "/" + name;
    const int out = ::open((base + ".stdout.log").c_str(), O_WRONLY | O_CREAT | O_APPEND, 0644);
    const int err = ::open((base + ".stderr.log").c_str(), O_WRONLY | O_CREAT | O_APPEND, 0644);
    if (out >= 0) { ::dup2(out, 1); }
    if (err >= 0) { ::dup2(err, 2); }
}

[[noreturn]] void exec_command(const std::vector<std::string> &command)
{
    std::vector<char *> argv;
    for (auto &a : command) { argv.push_back(const_cast<char *>(a.c_str())); }
    argv.push_back(nullptr);
    ::execvp(argv[0], argv.data());
    std::fprintf(stderr, "runner: cannot exec %s: %s\n", argv[0], std::strerror(errno));
    ::_exit(127);
}
}  // namespace

void runner::spawn(const peer_id &worker, const cluster_config &cluster, size_t version)
{
    const auto env = identity(worker, cluster, version);
    const pid_t pid = ::fork();
    if (pid < 0) { throw std::runtime_error("runner: fork failed"); }
    if (pid == 0) {
        // (no PR_SET_PDEATHSIG here: it fires when the forking THREAD ends, and
        // joiners are started from a short-lived connection thread)
        std::signal(SIGINT, SIG_DFL);
        std::signal(SIGTERM, SIG_DFL);
        std::signal(SIGPIPE, SIG_DFL);
        for (const auto &s : standbys_) { ::close(s.fd); }  // not this worker's to hold open
        for (const auto &kv : env) { ::setenv(kv.first.c_str(), kv.second.c_str(), 1); }
        for (const auto &kv : opt_.extra_env) { ::setenv(kv.first.c_str(), kv.second.c_str(), 1); }
        redirect_output(opt_.logdir, worker.hostname() + "." + std::to_string(worker.port));
        exec_command(opt_.command);
    }
    pids_[worker.hash()] = pid;
    if (!opt_.quiet) {
        log(PRINT) << "[runner] started worker" << worker.str() << "pid" << pid << "version"
                   << version;
    }
}

// A standby is the worker program without an identity: it runs up to its
// peer::from_env() (interpreter start, imports, model set-up), where it reads
// its identity from the pipe whose write end stays here.  End of file on that
// pipe (this launcher is done, or gone) makes it exit quietly.
void runner::spawn_standby()
{
    int fds[2];
    if (::pipe(fds) != 0) { return; }
    const pid_t pid = ::fork();
    if (pid < 0) {
        ::close(fds[0]);
        ::close(fds[1]);
        return;
    }
    if (pid == 0) {
        std::signal(SIGINT, SIG_DFL);
        std::signal(SIGTERM, SIG_DFL);
        std::signal(SIGPIPE, SIG_DFL);
        ::close(fds[1]);
        for (const auto &s : standbys_) { ::close(s.fd); }
        for (const char *name : {"KUNGFU_SELF_SPEC", "KUNGFU_INIT_PEERS", "KUNGFU_INIT_RUNNERS",
                                 "KUNGFU_INIT_CLUSTER_VERSION", "STDML_COLLECTIVE_DEVICE_ID"}) {
            ::unsetenv(name);
        }
        ::setenv("STDML_COLLECTIVE_STANDBY_FD", std::to_string(fds[0]).c_str(), 1);
        for (const auto &kv : opt_.extra_env) { ::setenv(kv.first.c_str(), kv.second.c_str(), 1); }
        redirect_output(opt_.logdir, "standby." + std::to_string(::getpid()));
        exec_command(opt_.command);
    }
    ::close(fds[0]);
    ::fcntl(fds[1], F_SETFD, FD_CLOEXEC);
    standbys_.push_back(standby{static_cast<int>(pid), fds[1]});
    if (!opt_.quiet) { log(PRINT) << "[runner] standby pid" << pid << "is warming up"; }
}

bool runner::hand_over(const peer_id &worker, const cluster_config &cluster, size_t version)
{
    while (!standbys_.empty()) {
        const standby s = standbys_.front();
        standbys_.erase(standbys_.begin());
        std::string block;
        for (const auto &kv : identity(worker, cluster, version)) {
            block += kv.first + "=" + kv.second + "\n";
        }
        block += "\n";
        size_t sent = 0;
        bool ok = true;
        while (sent < block.size()) {
            const ssize_t n = ::write(s.fd, block.data() + sent, block.size() - sent);
            if (n <= 0) {
                if (n < 0 && errno == EINTR) { continue; }
                ok = false;  // the standby is gone (EPIPE): try the next one
                break;
            }
            sent += static_cast<size_t>(n);
        }
        ::close(s.fd);
        if (!ok) { continue; }
        pids_[worker.hash()] = s.pid;
        if (!opt_.quiet) {
            log(PRINT) << "[runner] standby pid" << s.pid << "becomes worker" << worker.str()
                       << "version" << version;
        }
        return true;
    }
    return false;
}

// End of file on their pipes: standbys that were never needed exit by themselves.
void runner::dismiss_standbys()
{
    std::vector<standby> all;
    {
        std::lock_guard<std::mutex> lk(mu_);
        all.swap(standbys_);
    }
    for (const auto &s : all) { ::close(s.fd); }
    for (const auto &s : all) {
        bool gone = false;
        for (int waited_ms = 0; waited_ms < 3000 && !gone; waited_ms += 20) {
            gone = ::waitpid(s.pid, nullptr, WNOHANG) == s.pid;
            if (!gone) { std::this_thread::sleep_for(std::chrono::milliseconds(20)); }
        }
        if (!gone) {
            // still importing: it has not reached its read yet, do not wait for that
            ::kill(s.pid, SIGTERM);
            ::waitpid(s.pid, nullptr, 0);
        }
    }
}

void runner::reap(bool block)
{
    for (;;) {
        int status = 0;
        const pid_t pid = ::waitpid(-1, &status, block ? 0 : WNOHANG);
        if (pid <= 0) { return; }
        std::lock_guard<std::mutex> lk(mu_);
        bool was_standby = false;
        for (auto it = standbys_.begin(); it != standbys_.end(); ++it) {
            if (it->pid == pid) {  // died while warming up: no worker was lost
                ::close(it->fd);
                standbys_.erase(it);
                was_standby = true;
                break;
            }
        }
        if (was_standby) {
            if (!opt_.quiet) { log(PRINT) << "[runner] standby pid" << pid << "ended early"; }
            if (block) { return; }
            continue;
        }
        for (auto it = pids_.begin(); it != pids_.end(); ++it) {
            if (it->second == pid) {
                pids_.erase(it);
                break;
            }
        }
        if (!WIFEXITED(status) || WEXITSTATUS(status) != 0) {
            ++failed_;
            if (!opt_.quiet) { log(PRINT) << "[runner] worker pid" << pid << "failed"; }
        }
        if (block) { return; }
    }
}

// SIGTERM to every worker, a grace period, SIGKILL to what is left.
void runner::stop_workers()
{
    std::vector<int> pids;
    {
        std::lock_guard<std::mutex> lk(mu_);
        for (const auto &kv : pids_) { pids.push_back(kv.second); }
    }
    if (!opt_.quiet) { log(PRINT) << "[runner] signal" << int(g_stop_signal) << ": stopping" << pids.size() << "workers"; }
    for (int pid : pids) { ::kill(pid, SIGTERM); }
    for (int waited_ms = 0; waited_ms < 5000; waited_ms += 50) {
        reap(false);
        {
            std::lock_guard<std::mutex> lk(mu_);
            if (pids_.empty()) { break; }
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(50));
    }
    std::lock_guard<std::mutex> lk(mu_);
    for (const auto &kv : pids_) {
        ::kill(kv.second, SIGKILL);
        ::waitpid(kv.second, nullptr, 0);
        ++failed_;
    }
    pids_.clear();
    if (failed_ == 0) { failed_ = 1; }  // a job that was stopped did not succeed
}

void runner::on_update(size_t version, const cluster_config &next)
{
    std::lock_guard<std::mutex> lk(mu_);
    if (version <= version_) { return; }  // every surviving worker sends the same update
    version_ = version;
    const cluster_config old = cluster_;
    cluster_ = next;
    stored_config_ = next.json();
    if (!opt_.quiet) {
        log(PRINT) << "[runner] version" << version << ":" << old.workers.size() << "->"
                   << next.workers.size() << "workers";
    }
    for (const auto &w : next.workers) {
        if (w.ipv4 != opt_.self.ipv4) { continue; }  // another host's runner starts it
        if (old.workers.contains(w)) { continue; }
        const auto running = pids_.find(w.hash());
        if (running != pids_.end()) {
            // an earlier incarnation of this worker was removed and is on its
            // way out; its port is free only once it has exited
            int status = 0;
            if (::waitpid(running->second, &status, 0) == running->second &&
                (!WIFEXITED(status) || WEXITSTATUS(status) != 0)) {
                ++failed_;
            }
            pids_.erase(running);
        }
        if (!hand_over(w, next, version)) { spawn(w, next, version); }
    }
    while (opt_.watch && standbys_.size() < opt_.spares) { spawn_standby(); }
    // removed workers learn `detached` from their own resize() and exit by themselves
}

int runner::run()
{
    if (opt_.command.empty()) { throw std::invalid_argument("runner: no program given"); }
    const bool first_host = opt_.hosts.empty() || opt_.hosts[0].first == opt_.self.ipv4;
    if (opt_.config_port >= 0 && first_host) {
        http_ = std::make_unique<http_server>(
            static_cast<uint16_t>(opt_.config_port), [this](const http_server::request &rq) {
                http_response rs;
                rs.status = 200;
                std::lock_guard<std::mutex> lk(mu_);
                if (rq.method == "PUT" || rq.method == "POST") {
                    if (!cluster_config::from_json(rq.body)) {
                        rs.status = 400;
                        rs.body = "{\"error\":\"malformed cluster\"}";
                        return rs;
                    }
                    stored_config_ = rq.body;
                }
                rs.body = stored_config_;
                return rs;
            });
        http_->start();
    }
    if (opt_.watch) {
        handler_ = std::make_unique<control_conn_handler>(this);
        server_ = rchan::server::New(opt_.self, handler_.get());
        server_->start();
    }
    {
        std::lock_guard<std::mutex> lk(mu_);
        for (const auto &w : cluster_.workers) {
            if (w.ipv4 == opt_.self.ipv4) { spawn(w, cluster_, 0); }  // other hosts' runners start theirs
        }
        while (opt_.watch && standbys_.size() < opt_.spares) { spawn_standby(); }
    }
    // A runner of a several-host elastic job may have no worker of its own for a
    // while (its host was shrunk away) and must still be there when the job
    // grows back: it stays for as long as some worker of the current
    // configuration, on any host, answers a ping.
    const bool lingers = opt_.watch && !opt_.hosts.empty();
    int silent_checks = 0;
    std::signal(SIGINT, on_stop_signal);
    std::signal(SIGTERM, on_stop_signal);
    std::signal(SIGPIPE, SIG_IGN);  // a standby that died shows as EPIPE on its pipe
    for (;;) {
        if (g_stop_signal != 0) {
            stop_workers();
            break;
        }
        reap(false);
        bool idle;
        peer_list workers;
        {
            std::lock_guard<std::mutex> lk(mu_);
            idle = pids_.empty();
            workers = cluster_.workers;
        }
        if (!idle) {
            silent_checks = 0;
            std::this_thread::sleep_for(std::chrono::milliseconds(20));
            continue;
        }
        if (!lingers) { break; }
        bool alive = false;
        for (const auto &w : workers) {
            if (rchan::ping(w, opt_.self, 300) >= 0) {
                alive = true;
                break;
            }
        }
        silent_checks = alive ? 0 : silent_checks + 1;
        if (silent_checks >= 3) { break; }
        std::this_thread::sleep_for(std::chrono::milliseconds(500));
    }
    if (server_) { server_->stop(); }
    dismiss_standbys();
    if (http_) { http_->stop(); }
    return failed_;
}

bool parse_runner_args(int argc, char *argv[], runner_options &o, std::string &error)
{
    int i = 1;
    auto need = [&](const char *flag) -> const char * {
        if (i + 1 >= argc) {
            error = std::string("missing value for ") + flag;
            return nullptr;
        }
        return argv[++i];
    };
    for (; i < argc; ++i) {
        const std::string a = argv[i];
        if (a == "-np") {
            const char *v = need("-np");
            if (!v) { return false; }
            o.np = static_cast<size_t>(std::atoi(v));
        } else if (a == "-H") {  // ip:slots,ip:slots (kungfu-run's host list)
            const char *v = need("-H");
            if (!v) { return false; }
            std::string list = v;
            size_t at = 0;
            while (at <= list.size()) {
                const size_t comma = std::min(list.find(',', at), list.size());
                const std::string item = list.substr(at, comma - at);
                at = comma + 1;
                if (item.empty()) { continue; }
                const size_t colon = item.find(':');
                const auto ip = parse_peer_id(item.substr(0, colon) + ":1");
                const int slots = colon == std::string::npos ? 1 : std::atoi(item.c_str() + colon + 1);
                if (!ip || slots <= 0) {
                    error = "-H wants ip:slots[,ip:slots...]";
                    return false;
                }
                o.hosts.emplace_back(ip->ipv4, static_cast<size_t>(slots));
            }
        } else if (a == "-self") {
            const char *v = need("-self");
            if (!v) { return false; }
            const auto ip = parse_peer_id(std::string(v) + ":1");
            if (!ip) {
                error = "-self wants an IPv4 address";
                return false;
            }
            o.self.ipv4 = ip->ipv4;
        } else if (a == "-strategy") {
            const char *v = need("-strategy");
            if (!v) { return false; }
            o.strat = parse_kungfu_startegy(v);
        } else if (a == "-w") {
            o.watch = true;
        } else if (a == "-q") {
            o.quiet = true;
        } else if (a == "-spares") {
            const char *v = need("-spares");
            if (!v) { return false; }
            o.spares = static_cast<size_t>(std::max(0, std::atoi(v)));
        } else if (a == "-builtin-config-port") {
            const char *v = need("-builtin-config-port");
            if (!v) { return false; }
            o.config_port = std::atoi(v);
        } else if (a == "-config-server") {
            const char *v = need("-config-server");
            if (!v) { return false; }
            o.config_server_url = v;
        } else if (a == "-logdir") {
            const char *v = need("-logdir");
            if (!v) { return false; }
            o.logdir = v;
        } else if (a == "-runner-port") {
            const char *v = need("-runner-port");
            if (!v) { return false; }
            o.self.port = static_cast<uint16_t>(std::atoi(v));
        } else if (a == "-port-range") {
            const char *v = need("-port-range");
            if (!v) { return false; }
            o.worker_base_port = static_cast<uint16_t>(std::atoi(v));
        } else if (a == "-env") {
            const char *v = need("-env");
            if (!v) { return false; }
            const std::string kv = v;
            const size_t eq = kv.find('=');
            if (eq == std::string::npos) {
                error = "-env wants NAME=VALUE";
                return false;
            }
            o.extra_env.emplace_back(kv.substr(0, eq), kv.substr(eq + 1));
        } else if (a == "--") {
            ++i;
            break;
        } else if (!a.empty() && a[0] == '-') {
            error = "unknown flag " + a;
            return false;
        } else {
            break;
        }
    }
    for (; i < argc; ++i) { o.command.push_back(argv[i]); }
    if (o.hosts.size() == 1 && o.hosts[0].first == o.self.ipv4) { o.hosts.clear(); }
    if (o.np == 0) {
        error = "-np must be positive";
        return false;
    }
    if (o.command.empty()) {
        error = "no program given";
        return false;
    }
    return true;
}
}  // namespace stdml::collective
