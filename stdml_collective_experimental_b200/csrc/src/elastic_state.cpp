#include <vector>

#include <stdml/bits/collective/elastic_state.hpp>
#include <stdml/bits/collective/log.hpp>

namespace stdml::collective
{
elastic_state::elastic_state(peer::config_prodiver get_config, std::optional<int64_t> max_progress)
    : peer_(peer::from_env()), sess_(peer_.join_elastic()), max_progress_(max_progress),
      get_config_(std::move(get_config))
{
    // a process that joins a running job has to receive the state as well
    needs_state_ = sess_->version() > 0;
}

elastic_state::elastic_state(std::optional<int64_t> max_progress)
    : elastic_state([] { return get_cluster_config(); }, max_progress)
{
}

void elastic_state::sync()
{
    if (!synced_) {
        const int64_t mine = progress_;
        progress_ = sess_->all_reduce(mine, max);
        synced_ = true;
        if (needs_state_) {
            needs_state_ = false;
            // the lowest rank that is as far as anyone holds the state to copy:
            // rank 0 after a planned resize, possibly another one after a loss
            // (the step in flight may have finished on some members only)
            std::vector<int64_t> all(sess_->size(), 0);
            sess_->all_gather(&mine, all.data(), 1, i64, "stdml::progress");
            state_root_ = 0;
            while (state_root_ + 1 < all.size() && all[state_root_] != progress_) { ++state_root_; }
            if (on_resize_) { on_resize_(*sess_); }
        }
    }
}

void elastic_state::check_resize()
{
    const resize_result r = peer_.resize(sess_, get_config_);
    if (r.detached) {
        detached_ = true;
        return;
    }
    if (r.changed) {
        synced_ = false;
        needs_state_ = true;
        sync();
    }
}

elastic_state::operator int64_t()
{
    sync();
    return progress_;
}

void elastic_state::operator++()
{
    sync();
    ++progress_;
    check_resize();
}

bool elastic_state::should_stop()
{
    if (detached_) { return true; }
    sync();
    return max_progress_.has_value() && progress_ >= *max_progress_;
}

peer_list elastic_state::recover()
{
    const peer_list dropped = peer_.recover(sess_);
    synced_ = false;
    needs_state_ = true;
    sync();
    return dropped;
}

session &elastic_state::sess() { return *sess_; }
}  // namespace stdml::collective
