#include <algorithm>

#include <stdml/bits/collective/topology.hpp>

namespace stdml::collective
{
std::ostream &operator<<(std::ostream &os, const graph &g)
{
    for (size_t i = 0; i < g.size(); ++i) {
        os << i << (g.self_loop(i) ? "*" : "") << " ->";
        for (size_t j : g.nexts(i)) { os << " " << j; }
        os << "\n";
    }
    return os;
}

bool graph_builder::add_edge(size_t i, size_t j)
{
    if (i == j || i >= n_ || j >= n_) { return false; }
    return edges_.insert({i, j}).second;
}

graph graph_builder::build(bool reverse, bool add_self_loops) const
{
    std::vector<std::vector<size_t>> nexts(n_), prevs(n_);
    for (const auto &[a, b] : edges_) {  // std::set iterates sorted -> sorted adjacency
        const size_t from = reverse ? b : a, to = reverse ? a : b;
        nexts[from].push_back(to);
        prevs[to].push_back(from);
    }
    for (auto &v : nexts) { std::sort(v.begin(), v.end()); }
    for (auto &v : prevs) { std::sort(v.begin(), v.end()); }
    return graph(std::vector<bool>(n_, add_self_loops), std::move(nexts), std::move(prevs));
}

graph_builder start_broadcast_graph_builder(size_t n, size_t root)
{
    graph_builder b(n);
    for (size_t i = 0; i < n; ++i) { b.add_edge(root, i); }
    return b;
}

namespace
{
graph_pair star_pair(size_t n, size_t root)
{
    const graph_builder b = start_broadcast_graph_builder(n, root);
    return graph_pair{b.build(true, true), b.build(false, false)};
}

graph_pair ring_pair(size_t n, size_t root)
{
    graph_builder reduce(n), bcast(n);
    for (size_t k = 1; k < n; ++k) {
        reduce.add_edge((root + k) % n, (root + k + 1) % n);  // ends at root
        bcast.add_edge((root + k - 1) % n, (root + k) % n);   // starts at root
    }
    return graph_pair{reduce.build(false, true), bcast.build(false, false)};
}
graph_pair tree_pair(size_t n, size_t root)
{
    graph_builder bcast(n);
    for (size_t k = 1; k < n; ++k) { bcast.add_edge((root + (k - 1) / 2) % n, (root + k) % n); }
    return graph_pair{bcast.build(true, true), bcast.build(false, false)};
}
}  // namespace

graph_pair_list make_graph_pair_list(strategy s, size_t n)
{
    graph_pair_list l;
    if (s == ring && n > 1) {
        for (size_t r = 0; r < n; ++r) { l.pairs.push_back(ring_pair(n, r)); }
    } else if (s == binary_tree && n > 1) {
        for (size_t r = 0; r < n; ++r) { l.pairs.push_back(tree_pair(n, r)); }
    } else if (s == clique && n > 1) {
        for (size_t r = 0; r < n; ++r) { l.pairs.push_back(star_pair(n, r)); }
    } else {
        l.pairs.push_back(star_pair(n, 0));
    }
    return l;
}

const char *strategy_name(strategy s)
{
    return s == ring ? "RING" : s == binary_tree ? "BINARY_TREE" : s == clique ? "CLIQUE" : "STAR";
}
}  // namespace stdml::collective
