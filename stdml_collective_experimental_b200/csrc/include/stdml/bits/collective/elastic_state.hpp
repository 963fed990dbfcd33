// elastic_state: training progress that survives membership changes.
//
//     elastic_state st(get_config, max_step);
//     while (!st.should_stop()) { train(st.sess()); ++st; }
//
// ++st checks for a new configuration after every step; after a resize the
// progress counter becomes the maximum over the new members, so joiners catch
// up with survivors.  Same surface as the reference
// (include/stdml/bits/collective/elastic_state.hpp:8-38,
// src/stdml/collective/elastic_state.cpp:24-67), plus a constructor that uses
// the config server named by KUNGFU_CONFIG_SERVER (the reference leaves that
// one as a TODO) and a hook that is called after every resize so that model
// state can be re-broadcast from rank 0.
#pragma once
#include <cstdint>
#include <functional>
#include <memory>
#include <optional>

#include <stdml/bits/collective/peer.hpp>

namespace stdml::collective
{
class elastic_state
{
    peer peer_;
    std::unique_ptr<session> sess_;
    std::optional<int64_t> max_progress_;
    int64_t progress_ = 0;
    bool synced_ = false;
    bool detached_ = false;
    bool needs_state_ = false;
    size_t state_root_ = 0;
    peer::config_prodiver get_config_;
    std::function<void(session &)> on_resize_;

    void sync();
    void check_resize();

  public:
    explicit elastic_state(peer::config_prodiver get_config,
                           std::optional<int64_t> max_progress = {});
    explicit elastic_state(std::optional<int64_t> max_progress = {});

    operator int64_t();
    void operator++();
    bool should_stop();
    bool detached() const { return detached_; }
    session &sess();
    peer &get_peer() { return peer_; }
    // After a peer_failure in the loop body (or in ++): carry on with the
    // members that still answer.  Progress becomes the maximum over them and
    // the resize hook runs, exactly as after a planned resize.  Returns the
    // members that were dropped.
    //     try { train(st.sess()); ++st; } catch (const peer_failure &) { st.recover(); }
    peer_list recover();
    // called on every member of a new session (survivors right after the
    // resize, joiners at their first use of the state), after the progress
    // counter has been synchronised
    void on_resize(std::function<void(session &)> f) { on_resize_ = std::move(f); }
    // the rank whose state the hook should broadcast: the lowest one that has
    // made the most progress (0 after a planned resize)
    size_t state_root() const { return state_root_; }
};
}  // namespace stdml::collective
