// Elastic membership control: read the wanted cluster from a config server,
// propose a new size, announce a committed configuration to the runners.
// Same entry points as the reference (include/stdml/bits/collective/elastic.hpp:14-18).
// There the reader needs a Go shim (src/stdml/collective/elastic/elastic.go) and
// the whole feature is a build option; here it is always built and native:
// HTTP GET/PUT with a JSON body {"Runners":[...],"Workers":[...]} against
// KUNGFU_CONFIG_SERVER (this package ships a matching server, see http.hpp).
#pragma once
#include <cstddef>
#include <optional>
#include <string>

#include <stdml/bits/collective/address.hpp>

namespace stdml::collective
{
struct resize_result {
    bool changed;
    bool detached;
};

// GET $KUNGFU_CONFIG_SERVER; nullopt when unset, unreachable or malformed
std::optional<cluster_config> get_cluster_config();
std::optional<cluster_config> get_cluster_config(const std::string &url);

// PUT old_cluster.resize(new_size) to $KUNGFU_CONFIG_SERVER
void propose_new_size(const cluster_config &old_cluster, size_t new_size);
bool propose_cluster(const std::string &url, const cluster_config &next);

// send {"Version":v,"Cluster":{...}} as message "update" on conn_control to
// every runner of `config` (runners start and stop worker processes)
void commit_cluster_config(const cluster_config &config, size_t new_version);
}  // namespace stdml::collective
