// Peer identities and cluster membership.
//
// Same public surface and the same byte / JSON layouts as the reference
// (include/stdml/bits/collective/address.hpp:15-108,
// src/stdml/collective/address.cpp:160-250), so that configurations written by
// either implementation (or by a KungFu config server) are interchangeable:
//   bytes(): u32 #runners, u32 #workers, runners (6 B each), workers (6 B each)
//   json():  {"Runners":[{"IPv4":n,"Port":p},...],"Workers":[...]}
// Added here: cluster_config::from_json (the reference only declares it) and
// peer_list::contains.
#pragma once
#include <algorithm>
#include <cstddef>
#include <cstdint>
#include <optional>
#include <ostream>
#include <stdexcept>
#include <string>
#include <vector>

namespace stdml::collective
{
struct peer_id {
    uint32_t ipv4;  // a.b.c.d packed as (a << 24) | (b << 16) | (c << 8) | d
    uint16_t port;

    bool operator==(const peer_id &p) const { return ipv4 == p.ipv4 && port == p.port; }
    bool operator!=(const peer_id &p) const { return !(*this == p); }
    bool operator<(const peer_id &p) const
    {
        return ipv4 != p.ipv4 ? ipv4 < p.ipv4 : port < p.port;
    }

    std::string hostname() const;
    operator std::string() const;
    std::string str() const { return static_cast<std::string>(*this); }

    uint64_t hash() const { return (static_cast<uint64_t>(ipv4) << 32) | port; }
} __attribute__((packed));

static_assert(sizeof(peer_id) == 6, "peer_id is a packed 6-byte record");

std::ostream &operator<<(std::ostream &os, const peer_id &id);

// Thrown by sends to and receives from a peer that is known to have gone (its
// connections closed): see liveness.hpp.  The reference has no such error; a
// dead peer blocks the others for ever.
struct peer_failure : std::runtime_error {
    peer_id who;
    peer_failure(const peer_id &p, const std::string &what) : std::runtime_error(what), who(p) {}
};

class peer_list : public std::vector<peer_id>
{
    using base = std::vector<peer_id>;

  public:
    using base::base;
    using base::operator[];

    // sub-list by ranks
    template <typename I>
    peer_list operator[](const std::vector<I> &ranks) const
    {
        peer_list out;
        out.reserve(ranks.size());
        for (auto r : ranks) { out.push_back(base::operator[](static_cast<size_t>(r))); }
        return out;
    }

    // peers of *this that are not in `other`, order kept
    peer_list operator-(const peer_list &other) const;

    // 127.0.0.1:10000 ... 127.0.0.1:(10000 + n - 1)
    static peer_list gen(size_t n);

    // index of `id`, or size() when absent
    size_t rank(const peer_id &id) const
    {
        return static_cast<size_t>(std::find(begin(), end(), id) - begin());
    }

    bool contains(const peer_id &id) const { return rank(id) < size(); }
};

std::ostream &operator<<(std::ostream &os, const peer_list &ps);

std::optional<peer_id> parse_peer_id(const std::string &s);
// comma separated; empty string -> empty list; any malformed entry -> nullopt
std::optional<peer_list> parse_peer_list(const std::string &s);

struct cluster_config {
    peer_list runners;
    peer_list workers;

    cluster_config() = default;
    cluster_config(peer_list r, peer_list w) : runners(std::move(r)), workers(std::move(w)) {}

    bool operator==(const cluster_config &c) const
    {
        return runners == c.runners && workers == c.workers;
    }
    bool operator!=(const cluster_config &c) const { return !(*this == c); }

    // Shrink: keep the first new_size workers.  Grow: add workers on the runner
    // host with the fewest workers, on the lowest unused port above that
    // host's lowest worker port (10000 when the host has none).  Without
    // runners a cluster cannot grow and is returned unchanged.
    cluster_config resize(size_t new_size) const;

    std::vector<std::byte> bytes() const;
    static std::optional<cluster_config> from(const std::vector<std::byte> &bs);

    std::string json() const;
    static std::optional<cluster_config> from_json(const std::string &js);
};

std::ostream &operator<<(std::ostream &os, const cluster_config &c);

// KUNGFU_INIT_RUNNERS / KUNGFU_INIT_PEERS
cluster_config get_init_cluster_config_from_env();
}  // namespace stdml::collective
