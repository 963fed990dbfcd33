#include <memory>
#include <mutex>
#include <stdexcept>

#include <stdml/bits/collective/algorithm.hpp>
#include <stdml/bits/collective/peer.hpp>

namespace stdml::collective
{
namespace
{
std::mutex g_mu;
std::unique_ptr<peer> g_peer;
std::unique_ptr<session> g_sess;
}  // namespace

void init()
{
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_sess) { return; }
    g_peer = std::make_unique<peer>(peer::from_env());
    g_sess = g_peer->join_elastic();
}

void finalize()
{
    std::lock_guard<std::mutex> lk(g_mu);
    g_sess.reset();
    g_peer.reset();
}

session &default_session()
{
    init();
    return *g_sess;
}

resize_result resize(size_t new_size)
{
    init();
    return g_peer->resize(g_sess, new_size);
}

void all_reduce(const void *input, void *output, size_t count, dtype dt, reduce_op op)
{
    default_session().all_reduce(input, output, count, dt, op);
}

void reduce(const void *input, void *output, size_t count, dtype dt, reduce_op op)
{
    default_session().reduce(input, output, count, dt, op);
}

void all_gather(const void *input, void *output, size_t count, dtype dt)
{
    default_session().all_gather(input, output, count, dt);
}

void gather(const void *input, void *output, size_t count, dtype dt)
{
    default_session().gather(input, output, count, dt);
}

void broadcast(const void *input, void *output, size_t count, dtype dt)
{
    default_session().broadcast(input, output, count, dt);
}
}  // namespace stdml::collective
