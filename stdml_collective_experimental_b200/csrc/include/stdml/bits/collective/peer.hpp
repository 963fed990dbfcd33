// peer: the identity and lifetime of one process in the job.  Owns the
// mailbox / slotbox, the rchan server and the client pool; creates sessions.
// Same surface as the reference (include/stdml/bits/collective/peer.hpp:16-73).
#pragma once
#include <cstddef>
#include <functional>
#include <memory>
#include <optional>
#include <string>

#include <stdml/bits/collective/address.hpp>
#include <stdml/bits/collective/config.hpp>
#include <stdml/bits/collective/elastic.hpp>
#include <stdml/bits/collective/mailbox.hpp>
#include <stdml/bits/collective/rchan.hpp>
#include <stdml/bits/collective/session.hpp>

namespace stdml::collective
{
// Warm standby hand-over (launcher option -spares): when this process was started
// without an identity, waits for the launcher to provide one, exports it into
// the environment and returns it as "NAME=VALUE\n" lines; returns "" at once in
// every other process.  peer::from_env() calls it first; programs that read the
// environment themselves before that (a device index, say) call it earlier.
std::string standby_wait();

class peer
{
    system_config config_;
    size_t init_version_;
    peer_id self_;
    peer_list init_peers_;
    peer_list init_runners_;
    strategy init_strategy_;

    std::unique_ptr<mailbox> mailbox_;
    std::unique_ptr<slotbox> slotbox_;
    std::unique_ptr<liveness> liveness_;  // which peers still hold connections to us
    std::unique_ptr<rchan::conn_handler> handler_;
    // the client pool goes away before the server
    std::unique_ptr<rchan::server> server_;
    std::unique_ptr<rchan::client_pool> client_pool_;

    peer(system_config config, size_t init_version, peer_id self, peer_list init_peers,
         peer_list init_runners, strategy init_strategy = star);

  public:
    peer(peer &&) noexcept;
    ~peer();

    // one process, no network
    static peer single();
    // KUNGFU_SELF_SPEC, KUNGFU_INIT_PEERS, KUNGFU_INIT_RUNNERS,
    // KUNGFU_INIT_CLUSTER_VERSION, KUNGFU_ALLREDUCE_STRATEGY
    static peer from_kungfu_env();
    // OMPI_COMM_WORLD_SIZE / OMPI_COMM_WORLD_RANK -> 127.0.0.1:10000+rank, star
    static peer from_ompi_env();
    // RANK / WORLD_SIZE (torchrun) -> 127.0.0.1:(STDML_COLLECTIVE_BASE_PORT or 10000)+rank
    static peer from_torchrun_env();
    // KungFu, then OpenMPI, then torchrun variables, else single()
    static peer from_env();
    static peer from_fork(size_t rank, size_t size);
    // explicit membership
    static peer from_list(size_t rank, peer_list peers, strategy s = star, size_t version = 0,
                          peer_list runners = {});

    const system_config &config() const { return config_; }
    const peer_id &self() const { return self_; }
    size_t init_version() const { return init_version_; }
    strategy init_strategy() const { return init_strategy_; }
    rchan::client_pool *clients() const { return client_pool_.get(); }
    liveness *peers_alive() const { return liveness_.get(); }
    // Round trip of a conn_ping handshake to `target` in microseconds, or a
    // negative value if it does not answer within timeout_ms.
    double ping(const peer_id &target, int timeout_ms = 1000) const;

    void start();
    void stop();

    session join();
    std::unique_ptr<session> join_elastic();

    using config_prodiver = std::function<std::optional<cluster_config>()>;
    using config_provider = config_prodiver;
    using config_committer = std::function<void(cluster_config, int)>;

    // Agree with the current members on the configuration that `get_config`
    // returns (polling until all see the same one), commit it, and replace
    // `sess` by a session of the new membership.  Survivors keep their process
    // and connections; `detached` tells a removed rank to leave.
    resize_result resize(std::unique_ptr<session> &sess, const config_prodiver &get_config);
    // configuration from the config server ($KUNGFU_CONFIG_SERVER)
    resize_result resize(std::unique_ptr<session> &sess);
    // propose `new_size` to the config server first
    resize_result resize(std::unique_ptr<session> &sess, size_t new_size);
    resize_result resize(std::unique_ptr<session> &sess, const config_prodiver &get_config,
                         const config_committer &commit);

    // Unplanned loss of members (the reference has planned resizes only).
    // After a peer_failure every surviving member calls recover(): it gives up
    // on `sess` (telling the others), pings the old members, and replaces
    // `sess` by a session of those that answer, with the next version.  The
    // ranks of the survivors keep their order.  Returns the members that were
    // dropped.  As after a resize, the application re-synchronises its state
    // (progress by max-all-reduce, parameters by broadcast): a collective that
    // was in flight when the member died may have finished on some survivors
    // and not on others.
    // The survivors agree on one member list before any of them builds the new
    // session (their pings may have seen different things); a member that the
    // others could not reach gets peer_failure from its own recover().
    peer_list recover(std::unique_ptr<session> &sess, int ping_timeout_ms = 1000);
    // Same with the liveness probe supplied by the caller (`answers(p)`: does
    // old member p still answer?), for tests that make one rank's probe fail.
    peer_list recover(std::unique_ptr<session> &sess, int ping_timeout_ms,
                      const std::function<bool(const peer_id &)> &answers);

  private:
    peer_list agree_on_survivors(const peer_list &old, peer_list alive, size_t new_version,
                                 int ping_timeout_ms);

  public:
};

// fork n ranks on this host (ports 10000 + i), run g in each, wait for all
void prun(int n, const std::function<void(session &)> &g);

strategy parse_kungfu_startegy(const char *s);
}  // namespace stdml::collective
