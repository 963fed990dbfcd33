#include <chrono>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <stdexcept>
#include <thread>

#include <sys/wait.h>
#include <unistd.h>

#include <stdml/bits/collective/affinity.hpp>
#include <stdml/bits/collective/config.hpp>
#include <stdml/bits/collective/log.hpp>
#include <stdml/bits/collective/peer.hpp>
#include <stdml/bits/collective/stat.hpp>

namespace stdml::collective
{
namespace
{
// Routes messages of collective connections into the mailbox (eager) or the
// slotbox (rendezvous, flag wait_recv_buf); other connection types are drained.
class collective_msg_handler final : public rchan::msg_handler
{
    mailbox *mailbox_;
    slotbox *slotbox_;

  public:
    collective_msg_handler(mailbox *mb, slotbox *sb) : mailbox_(mb), slotbox_(sb) {}

    bool operator()(const rchan::received_header &mh, rchan::message_reader *reader,
                    const peer_id &src) override
    {
        if (mh.flags & rchan::message_header::wait_recv_buf) {
            bool ok = true;
            slotbox_->require(src, mh.name)->put(mh.len, [&](void *dst) {
                ok = reader->read_body(dst);
                return ok;
            });
            return ok;
        }
        buffer b = alloc_buffer(mh.len);
        if (!reader->read_body(b.data.get())) { return false; }
        mailbox_->require(src, mh.name)->put(std::move(b));
        return true;
    }
};

// Everything else is read and dropped, except the notice by which a member
// tells the others that it has given up on a session (liveness::abort_tag).
// Such notices travel on conn_control connections of their own, which are not
// counted as a sign of life: they are closed at once.
class drain_handler final : public rchan::msg_handler
{
    liveness *live_;

  public:
    explicit drain_handler(liveness *live) : live_(live) {}

    bool operator()(const rchan::received_header &mh, rchan::message_reader *reader,
                    const peer_id &) override
    {
        buffer b = alloc_buffer(mh.len);
        if (!reader->read_body(b.data.get())) { return false; }
        live_->note_abort(mh.name);
        return true;
    }
};

class peer_conn_handler final : public rchan::conn_handler
{
    collective_msg_handler collective_;
    drain_handler drain_;
    liveness *live_;

    // counts a data connection of a peer for as long as it is served
    struct presence {
        liveness *live;
        peer_id who;
        presence(liveness *l, const peer_id &p) : live(l), who(p) { live->connected(who); }
        ~presence() { live->disconnected(who); }
    };

  public:
    peer_conn_handler(mailbox *mb, slotbox *sb, liveness *live)
        : collective_(mb, sb), drain_(live), live_(live)
    {
    }

    size_t operator()(std::unique_ptr<rchan::connection> conn) override
    {
        switch (conn->type()) {
        case rchan::conn_collective:
        case rchan::conn_peer_to_peer:
        case rchan::conn_send:
        case rchan::conn_recv:
        case rchan::conn_mpi: {
            // the count drops only after everything read has been handed over
            presence here(live_, conn->src());
            return handle_to_end(conn.get(), &collective_);
        }
        default:  // conn_ping, conn_control from runners, user types: no data for a session
            return handle_to_end(conn.get(), &drain_);
        }
    }
};
}  // namespace

strategy parse_kungfu_startegy(const char *s)
{
    // an unset variable means star (the reference dereferences a null pointer here)
    if (s == nullptr) { return star; }
    std::string v(s);
    for (auto &c : v) { c = static_cast<char>(std::toupper(static_cast<unsigned char>(c))); }
    if (v == "BINARY_TREE" || v == "TREE") { return binary_tree; }
    if (v == "CLIQUE") { return clique; }
    return v == "RING" ? ring : star;
}

peer::peer(system_config config, size_t init_version, peer_id self, peer_list init_peers,
           peer_list init_runners, strategy init_strategy)
    : config_(std::move(config)), init_version_(init_version), self_(self),
      init_peers_(std::move(init_peers)), init_runners_(std::move(init_runners)),
      init_strategy_(init_strategy), mailbox_(new mailbox), slotbox_(new slotbox),
      liveness_(new liveness),
      handler_(new peer_conn_handler(mailbox_.get(), slotbox_.get(), liveness_.get())),
      client_pool_(new rchan::client_pool(self))
{
}

peer::peer(peer &&) noexcept = default;

peer::~peer() { stop(); }

peer peer::single()
{
    const peer_list ps = peer_list::gen(1);
    return peer(parse_system_config_from_env(), 0, ps[0], ps, {});
}

peer peer::from_list(size_t rank, peer_list peers, strategy s, size_t version, peer_list runners)
{
    if (rank >= peers.size()) { throw std::invalid_argument("peer: rank outside the peer list"); }
    const peer_id self = peers[rank];
    peer p(parse_system_config_from_env(), version, self, std::move(peers), std::move(runners), s);
    p.start();
    return p;
}

peer peer::from_kungfu_env()
{
    const auto self = parse_peer_id(safe_getenv("KUNGFU_SELF_SPEC"));
    const auto peers = parse_peer_list(safe_getenv("KUNGFU_INIT_PEERS"));
    const auto runners = parse_peer_list(safe_getenv("KUNGFU_INIT_RUNNERS"));
    if (!self || !peers || !runners) { return single(); }
    if (!peers->contains(*self)) {
        throw std::runtime_error("KUNGFU_SELF_SPEC " + self->str() +
                                 " is not listed in KUNGFU_INIT_PEERS");
    }
    const size_t version =
        static_cast<size_t>(parse_env_int("KUNGFU_INIT_CLUSTER_VERSION").value_or(0));
    peer p(parse_system_config_from_env(), version, *self, *peers, *runners,
           parse_kungfu_startegy(std::getenv("KUNGFU_ALLREDUCE_STRATEGY")));
    p.start();
    return p;
}

peer peer::from_ompi_env()
{
    const auto size = parse_env_int("OMPI_COMM_WORLD_SIZE");
    const auto rank = parse_env_int("OMPI_COMM_WORLD_RANK");
    if (!size || !rank || *size <= 0 || *rank < 0 || *rank >= *size) { return single(); }
    return from_fork(static_cast<size_t>(*rank), static_cast<size_t>(*size));
}

peer peer::from_torchrun_env()
{
    const auto size = parse_env_int("WORLD_SIZE");
    const auto rank = parse_env_int("RANK");
    if (!size || !rank || *size <= 0 || *rank < 0 || *rank >= *size) { return single(); }
    const uint16_t base =
        static_cast<uint16_t>(parse_env_int("STDML_COLLECTIVE_BASE_PORT").value_or(10000));
    peer_list ps;
    for (int64_t i = 0; i < *size; ++i) {
        ps.push_back(peer_id{(127u << 24) | 1u, static_cast<uint16_t>(base + i)});
    }
    return from_list(static_cast<size_t>(*rank), ps,
                     parse_kungfu_startegy(std::getenv("KUNGFU_ALLREDUCE_STRATEGY")));
}

// A warm standby (started by the launcher with -spares) has run its program up
// to here without an identity.  It waits for the launcher to write one into
// its pipe ("NAME=VALUE" lines, an empty line at the end), puts it into the
// environment and goes on as a worker that joins.  End of file instead means
// that it was never needed: the process ends quietly.
std::string standby_wait()
{
    const char *spec = std::getenv("STDML_COLLECTIVE_STANDBY_FD");
    if (spec == nullptr || *spec == '\0') { return ""; }
    const int fd = std::atoi(spec);
    ::unsetenv("STDML_COLLECTIVE_STANDBY_FD");
    std::string block;
    char buf[512];
    for (;;) {
        const ssize_t n = ::read(fd, buf, sizeof(buf));
        if (n < 0 && errno == EINTR) { continue; }
        if (n <= 0) { break; }
        block.append(buf, static_cast<size_t>(n));
        if (block.size() >= 2 && block.compare(block.size() - 2, 2, "\n\n") == 0) { break; }
    }
    ::close(fd);
    if (block.size() < 2 || block.compare(block.size() - 2, 2, "\n\n") != 0) {
        std::fflush(nullptr);
        ::_exit(0);  // dismissed
    }
    size_t at = 0;
    while (at < block.size()) {
        const size_t nl = block.find('\n', at);
        const std::string line = block.substr(at, nl - at);
        at = nl + 1;
        const size_t eq = line.find('=');
        if (eq == std::string::npos || eq == 0) { continue; }
        ::setenv(line.substr(0, eq).c_str(), line.substr(eq + 1).c_str(), 1);
    }
    return block;
}

peer peer::from_env()
{
    (void)standby_wait();
    if (std::getenv("KUNGFU_SELF_SPEC") != nullptr) { return from_kungfu_env(); }
    if (std::getenv("OMPI_COMM_WORLD_SIZE") != nullptr) { return from_ompi_env(); }
    if (std::getenv("WORLD_SIZE") != nullptr && std::getenv("RANK") != nullptr) {
        return from_torchrun_env();
    }
    return single();
}

peer peer::from_fork(size_t rank, size_t size)
{
    return from_list(rank, peer_list::gen(size),
                     parse_kungfu_startegy(std::getenv("KUNGFU_ALLREDUCE_STRATEGY")));
}

void peer::start()
{
    if (!server_) {
        server_ = rchan::server::New(self_, handler_.get());
        server_->start();
    }
}

void peer::stop()
{
    client_pool_.reset();
    if (server_) {
        server_->stop();
        server_.reset();
    }
}

double peer::ping(const peer_id &target, int timeout_ms) const
{
    return rchan::ping(target, self_, timeout_ms);
}

session peer::join()
{
    if (!client_pool_) { client_pool_.reset(new rchan::client_pool(self_)); }
    const size_t rank = init_peers_.rank(self_);
    session s(config_, init_version_, rank, init_peers_, init_runners_, mailbox_.get(),
              slotbox_.get(), client_pool_.get(), init_strategy_, liveness_.get());
    if (config_.use_affinity) { set_affinity(rank, init_peers_.size()); }
    return s;
}

std::unique_ptr<session> peer::join_elastic()
{
    if (!client_pool_) { client_pool_.reset(new rchan::client_pool(self_)); }
    const size_t rank = init_peers_.rank(self_);
    return std::make_unique<session>(config_, init_version_, rank, init_peers_, init_runners_,
                                     mailbox_.get(), slotbox_.get(), client_pool_.get(),
                                     init_strategy_, liveness_.get());
}

resize_result peer::resize(std::unique_ptr<session> &sess, const config_prodiver &get_config,
                           const config_committer &commit)
{
    using namespace std::chrono_literals;
    std::optional<cluster_config> next;
    for (int attempt = 0;; ++attempt) {
        next = get_config();
        // the proposal may reach ranks at different times: go on only when
        // every current member has read the same configuration
        const std::vector<std::byte> bytes = next ? next->bytes() : std::vector<std::byte>();
        if (sess->consistent(bytes.data(), bytes.size())) { break; }
        log() << "resize: members disagree on the new configuration, retrying";
        std::this_thread::sleep_for(attempt < 20 ? 50ms : 1000ms);
    }
    if (!next || *next == sess->cluster()) { return {false, false}; }
    const size_t new_version = sess->version() + 1;
    const bool detached = !next->workers.contains(self_);
    commit(*next, static_cast<int>(new_version));
    if (detached) { return {true, true}; }
    const peer_list removed = sess->peers() - next->workers;
    const strategy s = sess->get_strategy();
    sess.reset();  // releases device mappings of the old membership first
    client_pool_->reset_peers(removed);
    init_peers_ = next->workers;
    init_runners_ = next->runners;
    init_version_ = new_version;
    // a joiner may reuse the address of a member that left earlier: it starts
    // with a clean record instead of that member's "gone"
    liveness_->forget(next->workers);
    // the constructor's barrier admits the joiners (they dial until we answer)
    sess = std::make_unique<session>(config_, new_version, next->workers.rank(self_),
                                     next->workers, next->runners, mailbox_.get(),
                                     slotbox_.get(), client_pool_.get(), s, liveness_.get());
    return {true, false};
}

peer_list peer::recover(std::unique_ptr<session> &sess, int ping_timeout_ms)
{
    return recover(sess, ping_timeout_ms, [this, ping_timeout_ms](const peer_id &p) {
        return rchan::ping(p, self_, ping_timeout_ms) >= 0;
    });
}

// Survivors must build the new session from ONE member list.  Each starts from
// its own pings, which can differ (a member that is slow, a ping that races
// with a death), so the views are intersected until they stop changing: in
// round k every member sends its view (one byte per old member) to the members
// of that view and waits for theirs; a member whose view does not come in time
// is dropped; the next view is the intersection of everything received.  The
// exchange ends when a round changes nothing and every view received equalled
// one's own.  A member that finds itself outside a view it received leaves with
// peer_failure (the others go on without it).
peer_list peer::agree_on_survivors(const peer_list &old, peer_list alive, size_t new_version,
                                   int ping_timeout_ms)
{
    using namespace std::chrono;
    const size_t n = old.size();
    // members enter recover() at different times: the one that saw the failure
    // first, the others after its notice and their own pings of the dead
    const long long patience_ms =
        std::max<long long>(5000, 3ll * std::max(ping_timeout_ms, 1) * static_cast<long long>(n));
    auto *out = client_pool_->require(rchan::conn_collective);
    out->set_dial_patience_ms(std::max<long long>(1000, ping_timeout_ms));
    peer_list told;  // everyone a view has gone to: they also hear of being dropped
    for (int round = 0; round < static_cast<int>(n) + 2; ++round) {
        const std::string name = "stdml::recover::v" + std::to_string(new_version) +
                                 "::view" + std::to_string(round);
        std::vector<uint8_t> mine(n, 0);
        for (size_t i = 0; i < n; ++i) { mine[i] = alive.contains(old[i]) ? 1 : 0; }
        peer_list reachable;
        for (const auto &p : alive) {
            if (p == self_) {
                reachable.push_back(p);
                continue;
            }
            try {
                out->send(p, name.c_str(), mine.data(), mine.size(), 0);
                reachable.push_back(p);
            } catch (const std::exception &) {
                // it went between the ping and now
            }
            if (!told.contains(p)) { told.push_back(p); }
        }
        for (const auto &p : told) {
            if (alive.contains(p)) { continue; }
            try {  // best effort: lets a member that is alive but was dropped give up at once
                out->send(p, name.c_str(), mine.data(), mine.size(), 0);
            } catch (const std::exception &) {
            }
        }
        bool all_equal = reachable.size() == alive.size();
        std::vector<uint8_t> next = mine;
        peer_list heard;
        const auto deadline = steady_clock::now() + milliseconds(patience_ms);
        for (const auto &p : reachable) {
            if (p == self_) {
                heard.push_back(p);
                continue;
            }
            auto *box = mailbox_->require(p, name);
            std::optional<buffer> got;
            for (;;) {
                got = box->get_for(milliseconds(liveness::slice_ms));
                if (got || steady_clock::now() >= deadline) { break; }
            }
            if (!got || got->len != n) {
                all_equal = false;  // silent (or not speaking this protocol): not a member
                continue;
            }
            const auto *theirs = reinterpret_cast<const uint8_t *>(got->data.get());
            const size_t me = old.rank(self_);
            if (theirs[me] == 0) {
                throw peer_failure(p, "recover: member " + p.str() +
                                          " could not reach this rank and the survivors go on "
                                          "without it");
            }
            heard.push_back(p);
            for (size_t i = 0; i < n; ++i) {
                if (theirs[i] != mine[i]) { all_equal = false; }
                next[i] = next[i] && theirs[i];
            }
        }
        peer_list agreed;
        for (size_t i = 0; i < n; ++i) {
            if (next[i] && heard.contains(old[i])) { agreed.push_back(old[i]); }
        }
        const bool stable = all_equal && agreed.size() == alive.size();
        alive = agreed;
        if (stable) { break; }
    }
    out->set_dial_patience_ms(-1);
    return alive;
}

peer_list peer::recover(std::unique_ptr<session> &sess, int ping_timeout_ms,
                        const std::function<bool(const peer_id &)> &answers)
{
    sess->abort();
    const peer_list old = sess->peers();
    const peer_list runners = sess->runners();
    const strategy s = sess->get_strategy();
    const size_t new_version = sess->version() + 1;
    peer_list alive;
    for (const auto &p : old) {
        // a member that is itself recovering still answers: its server runs
        if (p == self_ || answers(p)) { alive.push_back(p); }
    }
    sess.reset();
    liveness_->forget(old);
    alive = agree_on_survivors(old, alive, new_version, ping_timeout_ms);
    const peer_list dropped = old - alive;
    client_pool_->reset_peers(dropped);
    init_peers_ = alive;
    init_version_ = new_version;
    if (alive.rank(self_) == 0) {
        // the wanted membership is now the surviving one: tell the config server
        // (else the next resize check would ask for the dead member again) and
        // the runners (which start and stop worker processes)
        const cluster_config next(runners, alive);
        try {
            const std::string url = safe_getenv("KUNGFU_CONFIG_SERVER");
            if (!url.empty() && !propose_cluster(url, next)) {
                log(WARN) << "recover: the config server at" << url << "refused the new membership";
            }
            commit_cluster_config(next, new_version);
        } catch (const std::exception &e) {
            log(WARN) << "recover: could not publish the new membership:" << e.what();
        }
    }
    // the constructor's barrier completes once every survivor has got here
    sess = std::make_unique<session>(config_, new_version, alive.rank(self_), alive, runners,
                                     mailbox_.get(), slotbox_.get(), client_pool_.get(), s,
                                     liveness_.get());
    // belt and braces: every member of the new session was built from the same list
    const std::vector<std::byte> view = cluster_config(runners, alive).bytes();
    if (!sess->consistent(view.data(), view.size())) {
        throw std::runtime_error("recover: the survivors built sessions from different member "
                                 "lists (version " + std::to_string(new_version) + ")");
    }
    return dropped;
}

resize_result peer::resize(std::unique_ptr<session> &sess, const config_prodiver &get_config)
{
    return resize(sess, get_config, [](cluster_config c, int v) {
        commit_cluster_config(c, static_cast<size_t>(v));
    });
}

resize_result peer::resize(std::unique_ptr<session> &sess)
{
    return resize(sess, [] { return get_cluster_config(); });
}

resize_result peer::resize(std::unique_ptr<session> &sess, size_t new_size)
{
    // one proposer is enough; everyone then converges on the server's answer
    if (sess->rank() == 0) { propose_new_size(sess->cluster(), new_size); }
    return resize(sess);
}

void prun(int n, const std::function<void(session &)> &g)
{
    std::vector<pid_t> kids;
    for (int i = 0; i < n; ++i) {
        const pid_t pid = ::fork();
        if (pid < 0) { throw std::runtime_error("prun: fork failed"); }
        if (pid == 0) {
            int rc = 0;
            try {
                peer p = peer::from_fork(static_cast<size_t>(i), static_cast<size_t>(n));
                session s = p.join();
                g(s);
            } catch (const std::exception &e) {
                std::fprintf(stderr, "prun: rank %d failed: %s\n", i, e.what());
                rc = 1;
            }
            // _exit skips static destructors, which is where a traced process
            // prints its events
            if (rchan::stat_enabled()) {
                rchan::stat_report(std::cout);
                rchan::stat_clear();
                std::cout.flush();
            }
            std::fflush(nullptr);
            ::_exit(rc);
        }
        kids.push_back(pid);
    }
    int failed = 0;
    for (const pid_t pid : kids) {
        int status = 0;
        ::waitpid(pid, &status, 0);
        if (!WIFEXITED(status) || WEXITSTATUS(status) != 0) { ++failed; }
    }
    if (failed > 0) { throw std::runtime_error("prun: " + std::to_string(failed) + " rank(s) failed"); }
}
}  // namespace stdml::collective
