// Offset allocator of the symmetric heap.
#pragma once
#include <algorithm>
#include <cstddef>
#include <iterator>
#include <map>
#include <new>
#include <stdexcept>

namespace stdml::collective::cuda
{
inline size_t heap_round_up(size_t x, size_t m) { return (x + m - 1) / m * m; }

// First-fit free-list allocator over [base, base + size).  Deterministic, so
// ranks that make the same calls get the same offsets.
class OffsetHeap
{
    std::map<size_t, size_t> free_;  // offset -> length
    std::map<size_t, size_t> used_;

  public:
    void reset(size_t base, size_t size)
    {
        free_.clear();
        used_.clear();
        if (size > 0) { free_[base] = size; }
    }

    size_t alloc(size_t bytes)
    {
        bytes = heap_round_up(std::max<size_t>(bytes, 1), 256);
        for (auto it = free_.begin(); it != free_.end(); ++it) {
            if (it->second >= bytes) {
                const size_t off = it->first;
                const size_t rest = it->second - bytes;
                free_.erase(it);
                if (rest > 0) { free_[off + bytes] = rest; }
                used_[off] = bytes;
                return off;
            }
        }
        throw std::bad_alloc();
    }

    void release(size_t off)
    {
        auto it = used_.find(off);
        if (it == used_.end()) { throw std::invalid_argument("release: unknown arena offset"); }
        size_t len = it->second;
        used_.erase(it);
        auto next = free_.lower_bound(off);
        if (next != free_.end() && off + len == next->first) {
            len += next->second;
            next = free_.erase(next);
        }
        if (next != free_.begin()) {
            auto prev = std::prev(next);
            if (prev->first + prev->second == off) {
                prev->second += len;
                return;
            }
        }
        free_[off] = len;
    }
};

}  // namespace stdml::collective::cuda
