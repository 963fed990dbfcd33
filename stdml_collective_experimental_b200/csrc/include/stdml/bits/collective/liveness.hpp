// Failure detection on the host path.  The reference has none: a peer that
// dies in the middle of a collective leaves the others blocked for ever in
// channel::get (include/stdml/bits/collective/channel.hpp:26-34 there) and
// conn_ping exists as an enumerator only (connection.hpp:14).
//
// Here every inbound connection is counted per source peer.  A peer that had
// connections and has none left has gone (its process ended or dropped us); a
// receiver waiting for a message from it is woken within one wait slice and
// throws peer_failure instead of waiting for a timeout, or for ever.  Messages
// that arrived before the connection closed are still delivered: the count
// drops only after the reader thread has handed over everything it read.
// A peer that never connected at all (it died before its first message to us)
// cannot be told from one that is still starting; for such a peer a receiver
// is as patient as a dialler (STDML_COLLECTIVE_CONNECT_TIMEOUT_MS) and then
// pings it about once a second: no answer means it has gone.
#pragma once
#include <atomic>
#include <cstdint>
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>

#include <stdml/bits/collective/address.hpp>

namespace stdml::collective
{
class liveness
{
    struct entry {
        int open = 0;
        bool seen = false;
    };
    mutable std::mutex mu_;
    std::map<uint64_t, entry> peers_;
    std::atomic<int> gone_{0};
    std::atomic<uint64_t> aborted_{0};  // 1 + the newest session version a member has given up on

  public:
    // name of the message a member sends to the others when it gives up on the
    // session of that version (so that ranks which wait for a live member that
    // will never answer give up too)
    static std::string abort_tag(size_t version) { return "stdml::abort::v" + std::to_string(version); }

    // handler side: returns true if `name` was an abort message
    bool note_abort(const std::string &name)
    {
        static const std::string prefix = "stdml::abort::v";
        if (name.compare(0, prefix.size(), prefix) != 0) { return false; }
        uint64_t v = 0;
        for (size_t i = prefix.size(); i < name.size(); ++i) {
            if (name[i] < '0' || name[i] > '9') { return false; }
            v = v * 10 + static_cast<uint64_t>(name[i] - '0');
        }
        uint64_t cur = aborted_.load();
        while (cur < v + 1 && !aborted_.compare_exchange_weak(cur, v + 1)) {}
        return true;
    }

    bool aborted(size_t version) const { return aborted_.load(std::memory_order_acquire) > version; }

    // how long a blocked receiver sleeps between two looks at this table
    static constexpr long long slice_ms = 100;

    void connected(const peer_id &p)
    {
        std::lock_guard<std::mutex> lk(mu_);
        entry &e = peers_[p.hash()];
        if (e.seen && e.open == 0) { gone_.fetch_sub(1, std::memory_order_relaxed); }
        e.seen = true;
        ++e.open;
    }

    void disconnected(const peer_id &p)
    {
        std::lock_guard<std::mutex> lk(mu_);
        entry &e = peers_[p.hash()];
        if (e.open > 0 && --e.open == 0) { gone_.fetch_add(1, std::memory_order_release); }
    }

    // cheap pre-check for polling loops
    bool any_gone() const { return gone_.load(std::memory_order_acquire) > 0; }

    bool gone(const peer_id &p) const
    {
        if (!any_gone()) { return false; }
        std::lock_guard<std::mutex> lk(mu_);
        const auto it = peers_.find(p.hash());
        return it != peers_.end() && it->second.seen && it->second.open == 0;
    }

    // has this peer ever opened a data connection to us?
    bool seen(const peer_id &p) const
    {
        std::lock_guard<std::mutex> lk(mu_);
        const auto it = peers_.find(p.hash());
        return it != peers_.end() && it->second.seen;
    }

    // a new membership starts with a clean record for these peers
    void forget(const peer_list &ps)
    {
        std::lock_guard<std::mutex> lk(mu_);
        for (const auto &p : ps) {
            const auto it = peers_.find(p.hash());
            if (it == peers_.end()) { continue; }
            if (it->second.seen && it->second.open == 0) {
                gone_.fetch_sub(1, std::memory_order_relaxed);
            }
            if (it->second.open == 0) {
                peers_.erase(it);
            }
        }
    }
};
}  // namespace stdml::collective
