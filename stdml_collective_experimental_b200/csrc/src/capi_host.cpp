// C ABI of the host runtime (loaded from Python with ctypes).
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <string>

#include <stdml/bits/collective/dtype.hpp>

namespace sc = stdml::collective;

extern "C" {
const char *stdmlc_version() { return "0.1.0"; }

int stdmlc_dtype_size(int dt)
{
    return static_cast<int>(sc::dtype_size_nothrow(static_cast<sc::dtype>(dt)));
}

// out[i] = in[0][i] op ... op in[n-1][i], rank-ascending; the CPU oracle of the
// device kernels.  Returns 0, or 2 for an undefined (dtype, op) pair.
int stdmlc_reduce_many(void *out, const void *const *in, unsigned long long n,
                       unsigned long long count, int dt, int op, double scale)
{
    try {
        sc::reduce_many(out, in, n, count, static_cast<sc::dtype>(dt),
                        static_cast<sc::reduce_op>(op), scale);
        return 0;
    } catch (const std::exception &) {
        return 2;
    }
}

int stdmlc_reduce(void *x, const void *y, const void *z, unsigned long long count, int dt, int op)
{
    try {
        sc::reduce(x, y, z, count, static_cast<sc::dtype>(dt), static_cast<sc::reduce_op>(op));
        return 0;
    } catch (const std::exception &) {
        return 2;
    }
}
}

// ------------------------------------------------------------ peer / session
#include <memory>
#include <optional>
#include <vector>

#include <stdml/bits/collective/peer.hpp>
#include <stdml/bits/collective/stat.hpp>

namespace stdml::collective::cuda
{
void set_last_error(const std::string &msg);  // cuda/capi_cuda.cpp
}

namespace
{
template <typename F>
int host_guarded(F f)
{
    try {
        f();
        return 0;
    } catch (const std::invalid_argument &e) {
        sc::cuda::set_last_error(e.what());
        return 2;
    } catch (const sc::peer_failure &e) {
        sc::cuda::set_last_error(e.what());
        return 5;
    } catch (const std::exception &e) {
        sc::cuda::set_last_error(e.what());
        return 1;
    } catch (...) {  // nothing may unwind through the C boundary
        sc::cuda::set_last_error("unknown C++ exception");
        return 1;
    }
}

struct session_box {
    std::unique_ptr<sc::session> s;
};

sc::peer *PP(void *h)
{
    if (h == nullptr) { throw std::invalid_argument("null peer handle"); }
    return static_cast<sc::peer *>(h);
}

sc::session &SS(void *h)
{
    auto *box = static_cast<session_box *>(h);
    if (box == nullptr || !box->s) { throw std::invalid_argument("null or closed session handle"); }
    return *box->s;
}
}  // namespace

extern "C" {
// Warm standby hand-over: copies the identity ("NAME=VALUE\n" lines) into buf and
// returns its length; 0 when this process is not a standby (the usual case).
long long stdmlc_standby_wait(char *buf, unsigned long long cap)
{
    try {
        const std::string block = sc::standby_wait();
        if (buf != nullptr && cap > 0) {
            const size_t n = std::min<size_t>(block.size(), static_cast<size_t>(cap) - 1);
            std::memcpy(buf, block.data(), n);
            buf[n] = '\0';
        }
        return static_cast<long long>(block.size());
    } catch (...) {
        return -1;
    }
}

int stdmlc_peer_from_env(void **out)
{
    *out = nullptr;
    return host_guarded([&] { *out = new sc::peer(sc::peer::from_env()); });
}

int stdmlc_peer_create(void **out, int rank, const char *peers_csv, int strategy,
                       unsigned long long version, const char *runners_csv)
{
    *out = nullptr;
    return host_guarded([&] {
        const auto peers = sc::parse_peer_list(peers_csv ? peers_csv : "");
        const auto runners = sc::parse_peer_list(runners_csv ? runners_csv : "");
        if (!peers || !runners || peers->empty()) {
            throw std::invalid_argument("peer: malformed peer list");
        }
        *out = new sc::peer(sc::peer::from_list(static_cast<size_t>(rank), *peers,
                                                strategy == 1 ? sc::ring : strategy == 2 ? sc::binary_tree : strategy == 3 ? sc::clique : sc::star, version,
                                                *runners));
    });
}

int stdmlc_peer_destroy(void *p)
{
    return host_guarded([&] { delete static_cast<sc::peer *>(p); });  // null is a no-op
}

int stdmlc_peer_self(void *p, char *buf, unsigned long long size)
{
    return host_guarded([&] {
        const std::string s = PP(p)->self().str();
        std::snprintf(buf, size, "%s", s.c_str());
    });
}

// round trip of one conn_ping handshake in microseconds; negative: no answer
int stdmlc_peer_ping(void *p, const char *target, int timeout_ms, double *us)
{
    *us = -1;
    return host_guarded([&] {
        const auto id = sc::parse_peer_id(target);
        if (!id) { throw std::invalid_argument(std::string("ping: bad address ") + target); }
        *us = PP(p)->ping(*id, timeout_ms);
    });
}

int stdmlc_peer_join(void *p, void **sess)
{
    *sess = nullptr;
    return host_guarded([&] {
        auto box = std::make_unique<session_box>();
        box->s = PP(p)->join_elastic();
        *sess = box.release();
    });
}

// *out = a session of the listed ranks (null handle if this rank is not listed);
// it shares the parent's connections and must be destroyed before the peer
int stdmlc_session_subgroup(void *s, const unsigned long long *ranks, unsigned long long n,
                            const char *scope, void **out)
{
    *out = nullptr;
    return host_guarded([&] {
        std::vector<size_t> rs(ranks, ranks + n);
        auto sub = SS(s).subgroup(rs, scope ? scope : "");
        if (sub) {
            auto box = std::make_unique<session_box>();
            box->s = std::move(sub);
            *out = box.release();
        }
    });
}

int stdmlc_session_destroy(void *s)
{
    return host_guarded([&] { delete static_cast<session_box *>(s); });
}

// what: 0 rank, 1 size, 2 version, 3 strategy (0 star, 1 ring, 2 binary tree)
int stdmlc_session_info(void *s, int what, unsigned long long *out)
{
    return host_guarded([&] {
        sc::session &ss = SS(s);
        switch (what) {
        case 0:
            *out = ss.rank();
            break;
        case 1:
            *out = ss.size();
            break;
        case 2:
            *out = ss.version();
            break;
        case 3:
            *out = ss.get_strategy() == sc::ring ? 1 : ss.get_strategy() == sc::binary_tree ? 2 : ss.get_strategy() == sc::clique ? 3 : 0;
            break;
        default:
            throw std::invalid_argument("session_info: unknown item");
        }
    });
}

int stdmlc_session_cluster_json(void *s, char *buf, unsigned long long size)
{
    return host_guarded([&] {
        const std::string js = SS(s).cluster().json();
        if (js.size() + 1 > size) { throw std::invalid_argument("cluster_json: buffer too small"); }
        std::snprintf(buf, size, "%s", js.c_str());
    });
}

int stdmlc_session_all_reduce(void *s, const void *in, void *out, unsigned long long count, int dt,
                              int op, const char *name, void *stream)
{
    return host_guarded([&] {
        SS(s).all_reduce(in, out, count, static_cast<sc::dtype>(dt), static_cast<sc::reduce_op>(op),
                         name ? name : "", stream);
    });
}

int stdmlc_session_reduce(void *s, const void *in, void *out, unsigned long long count, int dt,
                          int op, const char *name, void *stream)
{
    return host_guarded([&] {
        SS(s).reduce(in, out, count, static_cast<sc::dtype>(dt), static_cast<sc::reduce_op>(op),
                     name ? name : "", stream);
    });
}

int stdmlc_session_group_all_reduce(void *s, unsigned long long n, const void *const *ins,
                                    void *const *outs, const unsigned long long *counts, int dt,
                                    int op, const char *const *names, double scale, void *stream)
{
    return host_guarded([&] {
        std::vector<sc::workspace> ws(n);
        for (size_t i = 0; i < n; ++i) {
            ws[i].send = ins[i];
            ws[i].recv = outs[i];
            ws[i].count = counts[i];
            ws[i].dt = static_cast<sc::dtype>(dt);
            ws[i].op = static_cast<sc::reduce_op>(op);
            ws[i].name = names != nullptr && names[i] != nullptr ? names[i]
                                                                 : "tensor:" + std::to_string(i);
        }
        SS(s).group_all_reduce(ws, scale, stream);
    });
}

int stdmlc_session_all_gather(void *s, const void *in, void *out, unsigned long long count, int dt,
                              const char *name, void *stream)
{
    return host_guarded([&] {
        SS(s).all_gather(in, out, count, static_cast<sc::dtype>(dt), name ? name : "", stream);
    });
}

int stdmlc_session_reduce_to(void *s, const void *in, void *out, unsigned long long count, int dt,
                             int op, int root, const char *name, void *stream)
{
    return host_guarded([&] {
        if (root < 0) { throw std::invalid_argument("reduce: negative root"); }
        SS(s).reduce(in, out, count, static_cast<sc::dtype>(dt), static_cast<sc::reduce_op>(op),
                     name ? name : "", stream, static_cast<size_t>(root));
    });
}

int stdmlc_session_gather_to(void *s, const void *in, void *out, unsigned long long count, int dt,
                             int root, const char *name)
{
    return host_guarded([&] {
        if (root < 0) { throw std::invalid_argument("gather: negative root"); }
        SS(s).gather(in, out, count, static_cast<sc::dtype>(dt), name ? name : "",
                     static_cast<size_t>(root));
    });
}

int stdmlc_session_gather(void *s, const void *in, void *out, unsigned long long count, int dt,
                          const char *name)
{
    return host_guarded(
        [&] { SS(s).gather(in, out, count, static_cast<sc::dtype>(dt), name ? name : ""); });
}

int stdmlc_session_broadcast(void *s, const void *in, void *out, unsigned long long count, int dt,
                             const char *name, void *stream)
{
    return host_guarded([&] {
        SS(s).broadcast(in, out, count, static_cast<sc::dtype>(dt), name ? name : "", stream);
    });
}

int stdmlc_session_broadcast_from(void *s, const void *in, void *out, unsigned long long count,
                                  int dt, int root, const char *name, void *stream)
{
    return host_guarded([&] {
        if (root < 0) { throw std::invalid_argument("broadcast: negative root"); }
        SS(s).broadcast(in, out, count, static_cast<sc::dtype>(dt), name ? name : "", stream,
                        static_cast<size_t>(root));
    });
}

int stdmlc_session_reduce_scatter(void *s, const void *in, void *out, unsigned long long count,
                                  int dt, int op, const char *name, void *stream)
{
    return host_guarded([&] {
        SS(s).reduce_scatter(in, out, count, static_cast<sc::dtype>(dt),
                             static_cast<sc::reduce_op>(op), name ? name : "", stream);
    });
}

int stdmlc_session_all_to_all(void *s, const void *in, void *out, unsigned long long count, int dt,
                              const char *name, void *stream)
{
    return host_guarded([&] {
        SS(s).all_to_all(in, out, count, static_cast<sc::dtype>(dt), name ? name : "", stream);
    });
}

int stdmlc_session_send(void *s, const void *in, unsigned long long count, int dt, int target,
                        const char *name)
{
    return host_guarded([&] {
        SS(s).send(in, count, static_cast<sc::dtype>(dt), static_cast<size_t>(target),
                   name ? name : "");
    });
}

int stdmlc_session_recv(void *s, void *out, unsigned long long count, int dt, int target,
                        const char *name)
{
    return host_guarded([&] {
        SS(s).recv(out, count, static_cast<sc::dtype>(dt), static_cast<size_t>(target),
                   name ? name : "");
    });
}

int stdmlc_session_symm_alloc(void *s, unsigned long long bytes, void **out)
{
    *out = nullptr;
    return host_guarded([&] { *out = SS(s).symm_alloc(bytes); });
}

int stdmlc_session_symm_free(void *s, void *p)
{
    return host_guarded([&] { SS(s).symm_free(p); });
}

int stdmlc_session_device_setup_ms(void *s, double *out4)
{
    return host_guarded([&] { SS(s).device_setup_ms(out4); });
}

int stdmlc_session_device_set_knob(void *s, const char *name, long long value)
{
    return host_guarded([&] { SS(s).device_set_knob(name ? name : "", value); });
}

int stdmlc_session_device_drop_registrations(void *s)
{
    return host_guarded([&] { SS(s).device_drop_registrations(); });
}

int stdmlc_session_device_launches(void *s, unsigned long long *out)
{
    return host_guarded([&] { *out = SS(s).device_launches(); });
}

int stdmlc_session_barrier(void *s)
{
    return host_guarded([&] { SS(s).barrier(); });
}

int stdmlc_session_consistent(void *s, const void *data, unsigned long long size, int *same)
{
    return host_guarded([&] { *same = SS(s).consistent(data, size) ? 1 : 0; });
}

// new_size >= 0: propose it to the config server first; < 0: follow the server.
// cluster_json != NULL: use this configuration instead of the config server.
int stdmlc_peer_resize(void *p, void *sess, long long new_size, const char *cluster_json,
                       int *changed, int *detached)
{
    return host_guarded([&] {
        auto *peer = PP(p);
        auto *box = static_cast<session_box *>(sess);
        sc::resize_result r{false, false};
        if (cluster_json != nullptr) {
            const auto cfg = sc::cluster_config::from_json(cluster_json);
            if (!cfg) { throw std::invalid_argument("resize: malformed cluster JSON"); }
            r = peer->resize(box->s, [cfg] { return std::optional<sc::cluster_config>(*cfg); });
        } else if (new_size >= 0) {
            r = peer->resize(box->s, static_cast<size_t>(new_size));
        } else {
            r = peer->resize(box->s);
        }
        *changed = r.changed ? 1 : 0;
        *detached = r.detached ? 1 : 0;
    });
}

// After STDMLC_ERR_PEER: every survivor calls this; `sess` becomes a session of
// the members that still answer.  *dropped = how many members were left out.
int stdmlc_peer_recover(void *p, void *sess, int ping_timeout_ms, int *dropped)
{
    *dropped = 0;
    return host_guarded([&] {
        auto *box = static_cast<session_box *>(sess);
        *dropped = static_cast<int>(
            PP(p)->recover(box->s, ping_timeout_ms).size());
    });
}

int stdmlc_cluster_resize_json(const char *cluster_json, unsigned long long new_size, char *buf,
                               unsigned long long size)
{
    return host_guarded([&] {
        const auto cfg = sc::cluster_config::from_json(cluster_json);
        if (!cfg) { throw std::invalid_argument("malformed cluster JSON"); }
        const std::string js = cfg->resize(new_size).json();
        if (js.size() + 1 > size) { throw std::invalid_argument("buffer too small"); }
        std::snprintf(buf, size, "%s", js.c_str());
    });
}

void stdmlc_trace_enable(int on)
{
    if (on) {
        sc::rchan::stat_enable();
    } else {
        sc::rchan::stat_disable();
    }
}

int stdmlc_trace_write(const char *path)
{
    return sc::rchan::stat_write_chrome_trace(path) ? 0 : 1;
}
}

// ------------------------------------------------------------ async interface
extern "C" {
int stdmlc_session_all_reduce_async(void *s, const void *in, void *out, unsigned long long count,
                                    int dt, int op, const char *name, void *stream, void **task)
{
    *task = nullptr;
    return host_guarded([&] {
        *task = SS(s)
                    .async_all_reduce(in, out, count, static_cast<sc::dtype>(dt),
                                      static_cast<sc::reduce_op>(op), name ? name : "", stream)
                    .release();
    });
}

// send / recv that return a task (see session::async_send): device buffers are
// enqueued behind `stream` and run beside the collectives
int stdmlc_session_send_async(void *s, const void *in, unsigned long long count, int dt, int target,
                              const char *name, void *stream, void **task)
{
    *task = nullptr;
    return host_guarded([&] {
        *task = SS(s)
                    .async_send(in, count, static_cast<sc::dtype>(dt), static_cast<size_t>(target),
                                name ? name : "", stream)
                    .release();
    });
}

int stdmlc_session_recv_async(void *s, void *out, unsigned long long count, int dt, int source,
                              const char *name, void *stream, void **task)
{
    *task = nullptr;
    return host_guarded([&] {
        *task = SS(s)
                    .async_recv(out, count, static_cast<sc::dtype>(dt), static_cast<size_t>(source),
                                name ? name : "", stream)
                    .release();
    });
}

int stdmlc_task_poll(void *task, int *finished)
{
    return host_guarded([&] {
        auto *t = static_cast<sc::task *>(task);
        t->poll();
        *finished = t->finished() ? 1 : 0;
    });
}

int stdmlc_task_finish(void *task)
{
    return host_guarded([&] { static_cast<sc::task *>(task)->finish(); });
}

int stdmlc_task_destroy(void *task)
{
    return host_guarded([&] { delete static_cast<sc::task *>(task); });
}
}
