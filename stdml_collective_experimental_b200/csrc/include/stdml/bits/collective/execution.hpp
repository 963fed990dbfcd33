// fmap(policy, f, xs): apply f to every element of xs under an execution
// policy -- one thread per item (par), in order (seq), or on a thread_pool.
// Counterpart of include/stdml/bits/collective/execution.hpp:55-90.
#pragma once
#include <exception>
#include <mutex>
#include <thread>
#include <vector>

#include <stdml/bits/collective/thread_pool.hpp>

namespace stdml::collective
{
struct parallel_policy {
};
struct sequenced_policy {
};
inline constexpr parallel_policy par{};
inline constexpr sequenced_policy seq{};

template <typename F, typename L>
void fmap(sequenced_policy, const F &f, const L &xs)
{
    for (const auto &x : xs) { f(x); }
}

// a thread per item; the caller runs the first item itself
template <typename F, typename L>
void fmap(parallel_policy, const F &f, const L &xs)
{
    std::vector<std::thread> ths;
    std::mutex err_mu;
    std::exception_ptr err;
    auto keep = [&err_mu, &err] {
        std::lock_guard<std::mutex> lk(err_mu);
        if (!err) { err = std::current_exception(); }
    };
    auto it = xs.begin();
    if (it == xs.end()) { return; }
    const auto first = it++;
    for (; it != xs.end(); ++it) {
        ths.emplace_back([&f, &keep, it] {
            try {
                f(*it);
            } catch (...) {
                keep();
            }
        });
    }
    try {
        f(*first);
    } catch (...) {
        keep();
    }
    for (auto &t : ths) { t.join(); }
    if (err) { std::rethrow_exception(err); }
}

// on a pool; a null pool means a thread per item
template <typename F, typename L>
void fmap(sync::thread_pool *pool, const F &f, const L &xs)
{
    if (pool == nullptr) {
        fmap(par, f, xs);
        return;
    }
    std::vector<sync::thread_pool::task> fs;
    for (const auto &x : xs) {
        fs.emplace_back([&f, &x] { f(x); });
    }
    pool->par(std::move(fs));
}
}  // namespace stdml::collective
