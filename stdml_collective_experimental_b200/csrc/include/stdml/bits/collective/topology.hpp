// Communication graphs of the host (TCP) collectives and the strategy names of
// the public API.  Same surface as the reference
// (include/stdml/bits/collective/topology.hpp:10-93): graph, graph_builder,
// graph_pair, graph_pair_list, strategy {star, ring}, make_graph_pair_list.
//
// On the device path the strategies name algorithm families instead of wires
// (NVSwitch gives every GPU the same bandwidth to every peer): star -> every
// rank reads all peers (one-shot), ring -> reduce-scatter + all-gather
// (two-shot); both are upgraded to in-switch reduction (NVLS) when available.
#pragma once
#include <cstddef>
#include <ostream>
#include <set>
#include <utility>
#include <vector>

namespace stdml::collective
{
class graph
{
    std::vector<bool> self_loop_;
    std::vector<std::vector<size_t>> nexts_, prevs_;

  public:
    graph() = default;
    graph(std::vector<bool> self_loop, std::vector<std::vector<size_t>> nexts,
          std::vector<std::vector<size_t>> prevs)
        : self_loop_(std::move(self_loop)), nexts_(std::move(nexts)), prevs_(std::move(prevs))
    {
    }

    size_t size() const { return self_loop_.size(); }
    bool self_loop(size_t i) const { return self_loop_[i]; }
    const std::vector<size_t> &nexts(size_t i) const { return nexts_[i]; }
    const std::vector<size_t> &prevs(size_t i) const { return prevs_[i]; }
};

std::ostream &operator<<(std::ostream &os, const graph &g);

class graph_builder
{
    size_t n_;
    std::set<std::pair<size_t, size_t>> edges_;

  public:
    explicit graph_builder(size_t n) : n_(n) {}

    // false if the edge exists already, is a self edge, or is out of range
    bool add_edge(size_t i, size_t j);

    // reverse: flip every edge; add_self_loops: mark every vertex
    graph build(bool reverse = false, bool add_self_loops = false) const;
};

struct graph_pair {
    graph reduce_graph;     // data flows towards the root, accumulating
    graph broadcast_graph;  // the result flows back out
};

struct graph_pair_list {
    std::vector<graph_pair> pairs;

    std::pair<const graph *, const graph *> choose(size_t i) const
    {
        const graph_pair &p = pairs[i % pairs.size()];
        return {&p.reduce_graph, &p.broadcast_graph};
    }
};

enum strategy {
    star,
    ring,
    binary_tree,  // the reference lists it and leaves it commented out (topology.hpp:85-89 there)
    clique,       // one star per rank; KungFu's name for it (the reference has no such strategy)
};

// star rooted at `root`: edges root -> i
graph_builder start_broadcast_graph_builder(size_t n, size_t root);

// star: one pair rooted at 0.  ring: n pairs; pair r reduces along
// (r+1) -> (r+2) -> ... -> r and broadcasts along r -> r+1 -> ... -> r+n-1.
// binary_tree: n pairs; pair r is a complete binary tree over the ranks renumbered
// from r (rank (r + k) % n is node k, whose parent is node (k - 1) / 2): log2(n)
// hops instead of the ring's n - 1, two children per node instead of the star's
// n - 1 at the root.  clique: n pairs; pair r is the star rooted at r, so the
// chunks of a tensor (and the tensors of a set) spread their roots over all
// ranks: two hops like the star, the ring's even load per rank.
graph_pair_list make_graph_pair_list(strategy s, size_t n);

const char *strategy_name(strategy s);
}  // namespace stdml::collective
