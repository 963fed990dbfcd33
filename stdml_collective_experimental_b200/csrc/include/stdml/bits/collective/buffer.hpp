// Host-side message buffers and the `workspace` descriptor of one collective
// operand.  Same public surface as the reference
// (include/stdml/bits/collective/buffer.hpp:49-187): alloc_buffer,
// even_partition, workspace::{slice, split, forward}, workspace_state.
// Differences: a zero-length workspace is defined (no chunks), and chunking is
// by a byte limit so callers do not repeat the arithmetic.
#pragma once
#include <algorithm>
#include <cstddef>
#include <cstring>
#include <memory>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include <stdml/bits/collective/dtype.hpp>

namespace stdml::collective
{
struct buffer {
    std::unique_ptr<char[]> data;
    size_t len = 0;
};

inline buffer alloc_buffer(size_t len)
{
    buffer b;
    b.data.reset(new char[len > 0 ? len : 1]);
    b.len = len;
    return b;
}

// Appends fixed-width fields into one contiguous block (message headers).
class byte_buffer
{
    std::vector<char> bytes_;

  public:
    explicit byte_buffer(size_t reserve = 0) { bytes_.reserve(reserve); }

    template <typename T>
    byte_buffer &put(const T &x)
    {
        const char *p = reinterpret_cast<const char *>(&x);
        bytes_.insert(bytes_.end(), p, p + sizeof(T));
        return *this;
    }

    byte_buffer &put_bytes(const void *data, size_t n)
    {
        const char *p = static_cast<const char *>(data);
        bytes_.insert(bytes_.end(), p, p + n);
        return *this;
    }

    const char *data() const { return bytes_.data(); }
    size_t size() const { return bytes_.size(); }
};

// [begin, end) of part i when n items are cut into k parts whose sizes differ
// by at most one (the first n % k parts are the longer ones).
inline std::pair<size_t, size_t> even_part(size_t n, size_t k, size_t i)
{
    const size_t q = n / k, r = n % k;
    const size_t begin = q * i + std::min(i, r);
    return {begin, begin + q + (i < r ? 1 : 0)};
}

inline std::vector<std::pair<size_t, size_t>> even_partition(size_t n, size_t k)
{
    std::vector<std::pair<size_t, size_t>> parts;
    parts.reserve(k);
    for (size_t i = 0; i < k; ++i) { parts.push_back(even_part(n, k, i)); }
    return parts;
}

struct workspace {
    const void *send = nullptr;
    void *recv = nullptr;
    size_t count = 0;
    dtype dt = f32;
    reduce_op op = sum;
    std::string name;

    size_t bytes() const { return count * dtype_size(dt); }

    // Elements [i, j); the chunk name is what the peers match messages by.
    workspace slice(size_t i, size_t j) const
    {
        const size_t es = dtype_size(dt);
        workspace w;
        w.send = static_cast<const char *>(send) + i * es;
        w.recv = static_cast<char *>(recv) + i * es;
        w.count = j - i;
        w.dt = dt;
        w.op = op;
        w.name = "part::" + name + "[" + std::to_string(i) + ":" + std::to_string(j) + "]";
        return w;
    }

    std::vector<workspace> split(size_t k) const
    {
        std::vector<workspace> parts;
        if (k == 0 || count == 0) { return parts; }
        k = std::min(k, count);
        parts.reserve(k);
        for (size_t i = 0; i < k; ++i) {
            const auto [b, e] = even_part(count, k, i);
            parts.push_back(slice(b, e));
        }
        return parts;
    }

    // Chunks of at most `chunk_bytes` (0 chunks for an empty workspace).
    std::vector<workspace> split_by_bytes(size_t chunk_bytes) const
    {
        const size_t total = bytes();
        if (total == 0) { return {}; }
        return split((total + chunk_bytes - 1) / chunk_bytes);
    }

    void forward() const
    {
        if (send != recv && count > 0) { std::memcpy(recv, send, bytes()); }
    }
};

// Accumulation state of one workspace while messages for it arrive
// concurrently.  Until something has been accumulated the running value is
// `send`; afterwards it lives in `recv`.
class workspace_state
{
    const workspace *w_;
    std::mutex mu_;
    size_t received_ = 0;

  public:
    explicit workspace_state(const workspace *w) : w_(w) {}

    const workspace *operator->() const { return w_; }

    size_t received() const { return received_; }

    const void *effective_data() const { return received_ > 0 ? w_->recv : w_->send; }

    // recv = data op running value
    void add_to(const void *data)
    {
        std::lock_guard<std::mutex> lk(mu_);
        reduce(w_->recv, data, effective_data(), w_->count, w_->dt, w_->op);
        ++received_;
    }

    // a full value was written straight into recv (broadcast phase)
    void replaced()
    {
        std::lock_guard<std::mutex> lk(mu_);
        ++received_;
    }

    void forward() const { w_->forward(); }
};
}  // namespace stdml::collective
