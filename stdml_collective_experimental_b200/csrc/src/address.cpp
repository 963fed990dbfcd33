#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <set>
#include <sstream>

#include <stdml/bits/collective/address.hpp>
#include <stdml/bits/collective/json.hpp>

namespace stdml::collective
{
std::string peer_id::hostname() const
{
    char buf[32];
    std::snprintf(buf, sizeof(buf), "%u.%u.%u.%u", (ipv4 >> 24) & 0xffu, (ipv4 >> 16) & 0xffu,
                  (ipv4 >> 8) & 0xffu, ipv4 & 0xffu);
    return buf;
}

peer_id::operator std::string() const { return hostname() + ":" + std::to_string(port); }

std::ostream &operator<<(std::ostream &os, const peer_id &id) { return os << id.str(); }

std::ostream &operator<<(std::ostream &os, const peer_list &ps)
{
    os << "[";
    for (size_t i = 0; i < ps.size(); ++i) { os << (i ? ", " : "") << ps[i]; }
    return os << "]";
}

peer_list peer_list::operator-(const peer_list &other) const
{
    const std::set<peer_id> gone(other.begin(), other.end());
    peer_list rest;
    for (const auto &p : *this) {
        if (gone.count(p) == 0) { rest.push_back(p); }
    }
    return rest;
}

peer_list peer_list::gen(size_t n)
{
    peer_list ps;
    ps.reserve(n);
    for (size_t i = 0; i < n; ++i) {
        ps.push_back(peer_id{(127u << 24) | 1u, static_cast<uint16_t>(10000 + i)});
    }
    return ps;
}

std::optional<peer_id> parse_peer_id(const std::string &s)
{
    unsigned a, b, c, d, p;
    char tail;
    if (std::sscanf(s.c_str(), "%u.%u.%u.%u:%u%c", &a, &b, &c, &d, &p, &tail) != 5) { return {}; }
    if (a > 255 || b > 255 || c > 255 || d > 255 || p > 65535) { return {}; }
    return peer_id{(a << 24) | (b << 16) | (c << 8) | d, static_cast<uint16_t>(p)};
}

std::optional<peer_list> parse_peer_list(const std::string &s)
{
    peer_list ps;
    std::istringstream in(s);
    std::string item;
    while (std::getline(in, item, ',')) {
        if (item.empty()) { continue; }
        const auto id = parse_peer_id(item);
        if (!id) { return {}; }
        ps.push_back(*id);
    }
    return ps;
}

cluster_config cluster_config::resize(size_t new_size) const
{
    cluster_config next(runners, workers);
    if (new_size <= workers.size()) {
        next.workers.resize(new_size);
        return next;
    }
    if (runners.empty()) { return next; }
    std::map<uint32_t, std::set<uint16_t>> ports;  // host -> worker ports in use
    uint16_t base = workers.empty() ? 10000 : workers.front().port;
    for (const auto &w : workers) {
        ports[w.ipv4].insert(w.port);
        base = std::min(base, w.port);
    }
    while (next.workers.size() < new_size) {
        // least loaded runner host; the first such runner wins ties
        const peer_id *host = &runners.front();
        for (const auto &r : runners) {
            if (ports[r.ipv4].size() < ports[host->ipv4].size()) { host = &r; }
        }
        auto &used = ports[host->ipv4];
        // a host without workers starts at the lowest port of the job (its port range)
        uint16_t port = used.empty() ? base : static_cast<uint16_t>(*used.begin() + 1);
        while (used.count(port) != 0) { ++port; }
        used.insert(port);
        next.workers.push_back(peer_id{host->ipv4, port});
    }
    return next;
}

std::vector<std::byte> cluster_config::bytes() const
{
    const uint32_t nr = static_cast<uint32_t>(runners.size());
    const uint32_t nw = static_cast<uint32_t>(workers.size());
    std::vector<std::byte> out(8 + sizeof(peer_id) * (nr + nw));
    std::byte *p = out.data();
    std::memcpy(p, &nr, 4);
    std::memcpy(p + 4, &nw, 4);
    if (nr) { std::memcpy(p + 8, runners.data(), sizeof(peer_id) * nr); }
    if (nw) { std::memcpy(p + 8 + sizeof(peer_id) * nr, workers.data(), sizeof(peer_id) * nw); }
    return out;
}

std::optional<cluster_config> cluster_config::from(const std::vector<std::byte> &bs)
{
    if (bs.size() < 8) { return {}; }
    uint32_t nr, nw;
    std::memcpy(&nr, bs.data(), 4);
    std::memcpy(&nw, bs.data() + 4, 4);
    if (8 + sizeof(peer_id) * (static_cast<size_t>(nr) + nw) != bs.size()) { return {}; }
    cluster_config c;
    c.runners.resize(nr);
    c.workers.resize(nw);
    if (nr) { std::memcpy(c.runners.data(), bs.data() + 8, sizeof(peer_id) * nr); }
    if (nw) {
        std::memcpy(c.workers.data(), bs.data() + 8 + sizeof(peer_id) * nr, sizeof(peer_id) * nw);
    }
    return c;
}

namespace
{
json::value peers_to_json(const peer_list &ps)
{
    json::value arr = json::value::array();
    for (const auto &p : ps) {
        arr.push(json::value::object({{"IPv4", json::value::integer(p.ipv4)},
                                      {"Port", json::value::integer(p.port)}}));
    }
    return arr;
}

bool peers_from_json(const json::value *arr, peer_list &out)
{
    if (arr == nullptr) { return false; }
    if (arr->is_null()) { return true; }  // Go encodes an empty slice as null
    if (arr->type() != json::value::array_k) { return false; }
    for (const auto &item : arr->items()) {
        const json::value *ip = item.get("IPv4");
        const json::value *port = item.get("Port");
        if (ip == nullptr || port == nullptr || ip->type() != json::value::number_k ||
            port->type() != json::value::number_k) {
            return false;
        }
        const int64_t a = ip->as_int(), p = port->as_int();
        if (a < 0 || a > 0xffffffffll || p < 0 || p > 65535) { return false; }
        out.push_back(peer_id{static_cast<uint32_t>(a), static_cast<uint16_t>(p)});
    }
    return true;
}
}  // namespace

std::string cluster_config::json() const
{
    return json::value::object({{"Runners", peers_to_json(runners)},
                                {"Workers", peers_to_json(workers)}})
        .dump();
}

std::optional<cluster_config> cluster_config::from_json(const std::string &js)
{
    const auto v = json::parse(js);
    if (!v || v->type() != json::value::object_k) { return {}; }
    cluster_config c;
    if (!peers_from_json(v->get("Runners"), c.runners)) { return {}; }
    if (!peers_from_json(v->get("Workers"), c.workers)) { return {}; }
    return c;
}

std::ostream &operator<<(std::ostream &os, const cluster_config &c)
{
    return os << "runners: " << c.runners << ", workers: " << c.workers;
}

cluster_config get_init_cluster_config_from_env()
{
    auto read = [](const char *name) {
        const char *v = std::getenv(name);
        return parse_peer_list(v == nullptr ? "" : v).value_or(peer_list());
    };
    return cluster_config(read("KUNGFU_INIT_RUNNERS"), read("KUNGFU_INIT_PEERS"));
}
}  // namespace stdml::collective
