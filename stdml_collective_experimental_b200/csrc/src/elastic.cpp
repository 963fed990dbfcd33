#include <stdml/bits/collective/config.hpp>
#include <stdml/bits/collective/elastic.hpp>
#include <stdml/bits/collective/http.hpp>
#include <stdml/bits/collective/json.hpp>
#include <stdml/bits/collective/log.hpp>
#include <stdml/bits/collective/rchan.hpp>

namespace stdml::collective
{
std::optional<cluster_config> get_cluster_config(const std::string &url)
{
    const auto rs = http_get(url);
    if (!rs || rs->status != 200) { return {}; }
    return cluster_config::from_json(rs->body);
}

std::optional<cluster_config> get_cluster_config()
{
    const std::string url = safe_getenv("KUNGFU_CONFIG_SERVER");
    if (url.empty()) { return {}; }
    return get_cluster_config(url);
}

bool propose_cluster(const std::string &url, const cluster_config &next)
{
    const auto rs = http_put(url, next.json());
    return rs && rs->status == 200;
}

void propose_new_size(const cluster_config &old_cluster, size_t new_size)
{
    const std::string url = safe_getenv("KUNGFU_CONFIG_SERVER");
    if (url.empty()) {
        log(WARN) << "propose_new_size: KUNGFU_CONFIG_SERVER is not set";
        return;
    }
    if (!propose_cluster(url, old_cluster.resize(new_size))) {
        log(WARN) << "propose_new_size: the config server at" << url << "refused the proposal";
    }
}

void commit_cluster_config(const cluster_config &config, size_t new_version)
{
    if (config.runners.empty()) { return; }
    json::value msg = json::value::object();
    msg.set("Version", json::value::integer(static_cast<int64_t>(new_version)));
    msg.set("Cluster", json::parse(config.json()).value_or(json::value()));
    const std::string body = msg.dump();
    auto cl = rchan::client::New(peer_id{0, 0}, rchan::conn_control);
    for (const auto &runner : config.runners) {
        try {
            cl->send(runner, "update", body.data(), body.size(), 0);
        } catch (const std::exception &e) {
            log(WARN) << "commit_cluster_config: runner" << runner.str() << "unreachable:" << e.what();
        }
    }
}
}  // namespace stdml::collective
