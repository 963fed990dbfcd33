// session: the collective front-end.  One session = one fixed membership
// (version, rank, peers).  Construction is collective and ends with a barrier.
//
// Same calls as the reference (include/stdml/bits/collective/session.hpp:25-178)
// -- all_reduce, group_all_reduce, all_gather, broadcast (root 0), send, recv,
// consistent -- plus reduce / gather to root 0 (the reference only declares
// them, include/stdml/bits/collective/algorithm.hpp:16-18) and a public
// barrier.  Every call accepts host pointers (TCP path: star / ring graphs,
// 1 MiB chunks) and CUDA device pointers (NVLink path: fused sm_100a kernels;
// all ranks on one box, one GPU per rank); the two kinds are told apart by
// asking the CUDA runtime.  Device calls are enqueued on `stream` (the legacy
// default stream when null) and return without waiting for the GPU.
//
// Messages are matched by (source peer, name): concurrent operations between
// the same peers need distinct names, operations with one name are FIFO.
#pragma once
#include <cstddef>
#include <cstdint>
#include <atomic>
#include <chrono>
#include <future>
#include <iterator>
#include <memory>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include <stdml/bits/collective/address.hpp>
#include <stdml/bits/collective/buffer.hpp>
#include <stdml/bits/collective/config.hpp>
#include <stdml/bits/collective/dtype.hpp>
#include <stdml/bits/collective/liveness.hpp>
#include <stdml/bits/collective/mailbox.hpp>
#include <stdml/bits/collective/rchan.hpp>
#include <stdml/bits/collective/task.hpp>
#include <stdml/bits/collective/thread_pool.hpp>
#include <stdml/bits/collective/topology.hpp>

namespace stdml::collective
{
namespace cuda
{
class DeviceSession;
class NcclP2P;
}

class session
{
    std::unique_ptr<sync::thread_pool> pool_;
    std::unique_ptr<runtime> async_runtime_;
    std::unique_ptr<cuda::DeviceSession> device_;
    bool device_tried_ = false;
    std::shared_ptr<std::mutex> device_mu_ = std::make_shared<std::mutex>();  // guards device_'s creation
    std::unique_ptr<cuda::NcclP2P> p2p_;  // device send / recv, created by the first such call
    cuda::NcclP2P *p2p();
    int spin_polls_ = 0;  // looks at a mailbox before a receiver sleeps (see session.cpp)
    bool established_ = false;  // the constructor's barrier has completed
    // Two-level execution for members on several hosts (built on first use,
    // collectively): the ranks of this host, and one leader per host.
    struct levels {
        std::unique_ptr<session> local;    // same address, in rank order; its rank 0 leads
        std::unique_ptr<session> leaders;  // null on ranks that do not lead
    };
    std::unique_ptr<levels> levels_;
    bool spans_hosts() const;
    levels &two_levels();
    void all_reduce_two_level(const workspace &w, bool device, void *stream, double scale = 1.0);
    // how long a first connection is retried once the session is established
    static constexpr long long established_patience_ms = 1000;

    const std::string scope_;  // names the sub-group among its parent's messages ("" = the whole group)
    const system_config config_;
    const size_t version_;
    const size_t rank_;
    const peer_list peers_;
    const peer_list runners_;
    const strategy strategy_;

    graph_pair_list all_reduce_topo_;

    void run_chunk(const workspace &w, const graph *reduce_g, const graph *bcast_g);
    task *chunk_task(const workspace &w, const graph *reduce_g, const graph *bcast_g);
    cuda::DeviceSession *device();  // collective on first use
    bool on_device(const void *a, const void *b) const;

    // Every blocking receive of the host path goes through these: they sleep in
    // slices, throw peer_failure as soon as the source is known to have gone,
    // and std::runtime_error after config().host_timeout_ms (0: no limit).
    buffer take_eager(size_t src, const std::string &tag, const char *what);
    void take_into(size_t src, const std::string &tag, void *dst, size_t cap, const char *what);
    void finish_pending(slot::pending &p, size_t src, const std::string &tag, const char *what);
    bool source_gone(size_t src, long long waited_ms) const;
    struct poll_watch {
        std::chrono::steady_clock::time_point start{}, asked{};
        unsigned polls = 0;
    };
    bool polled_source_gone(const peer_id &who, poll_watch &w) const;
    void ensure_usable(const char *what);
    enum class failure { gone, late, other };
    [[noreturn]] void give_up(failure why, const peer_id &who, const char *what,
                              const std::string &tag);
    // set by the first receive that fails; every other blocked receive of this
    // session then gives up within one slice (the message streams of a session
    // that lost a peer no longer line up, so there is nothing to wait for)
    std::shared_ptr<std::atomic<bool>> broken_ = std::make_shared<std::atomic<bool>>(false);

  public:
    static constexpr size_t chunk_bytes = 1u << 20;
    // group_all_reduce(futures): device tensors are fused in buckets of about this size
    static constexpr size_t group_bucket_bytes = 64u << 20;
    static constexpr size_t tiny_chunk_bytes = 512u << 10;  // handled without helper threads (measured: star, 4 ranks, 64 KB +80 %, 400 KB +45 %; 1 MB chunks -15 %)

    mailbox *mailbox_;                 // owned by peer
    slotbox *slotbox_;                 // owned by peer
    rchan::client_pool *client_pool_;  // owned by peer
    liveness *liveness_;               // owned by peer; may be null (no failure detection)

    session(system_config config, size_t version, size_t rank, peer_list peers, peer_list runners,
            mailbox *eager_box, slotbox *posted_box, rchan::client_pool *client_pool,
            strategy s = star, liveness *live = nullptr, std::string scope = "");
    ~session();

    session(const session &) = delete;
    session(session &&) noexcept;

    size_t rank() const { return rank_; }
    size_t size() const { return peers_.size(); }
    const peer_list &peers() const { return peers_; }
    const peer_list &runners() const { return runners_; }
    sync::thread_pool *pool() const { return pool_.get(); }
    runtime *async_rt() const { return async_runtime_.get(); }
    cluster_config cluster() const { return cluster_config(runners_, peers_); }
    size_t version() const { return version_; }
    const std::string &scope() const { return scope_; }
    // A session of a subset of the members, in the order given (the counterpart of
    // a communicator split; the reference has one group only).  Collective among
    // the listed ranks, which all pass the same list and the same `scope`, a name
    // that is unique among the sub-groups alive at the same time; other ranks
    // need not call it and get null.  It shares this session's connections and
    // must not outlive the peer.
    std::unique_ptr<session> subgroup(const std::vector<size_t> &ranks, const std::string &scope);
    strategy get_strategy() const { return strategy_; }
    const system_config &config() const { return config_; }

    void barrier();

    // Device memory in this session's symmetric heap (collective: every rank makes
    // the same calls in the same order; the heap belongs to this membership and
    // goes with it on a resize).  Collectives on such buffers are zero-copy: no
    // staging, one launch.  Size of the heap: STDML_COLLECTIVE_HEAP_MB.
    void *symm_alloc(size_t bytes);
    void symm_free(void *p);

    // Milliseconds the device world of this membership took to set up (zeros
    // before the first device call): rendezvous among the ranks, own arena,
    // peers' arenas, NVLS multicast.
    void device_setup_ms(double out[4]) const;

    // A named tuning knob of the device plane, the same value on every rank
    // (e.g. "register_min_bytes": collectives on ordinary device buffers of at
    // least that size map the buffers' allocations on every peer and run on
    // them in place; a group of separately allocated tensors is then one
    // launch).  device_drop_registrations() is collective and unmaps what
    // registered calls mapped; buffers used that way must stay allocated until then.
    void device_set_knob(const std::string &name, long long value);
    void device_drop_registrations();

    // Kernels this session has launched on the device so far (0 before its first
    // device call): lets callers and tests see how many launches a call cost.
    unsigned long long device_launches() const;

    // true once a receive of this session has failed or a member has told us
    // that it gave up: the session is of no further use (see peer::recover)
    bool given_up() const;
    // gives up on this session and tells the other members
    void abort() noexcept;

    void all_reduce(const workspace &w, void *stream = nullptr);
    // Blocks until every tensor is reduced (device tensors: until every launch
    // is enqueued on the default stream).  Tensors may become ready in any order
    // and in different orders on different ranks.  Device tensors are reduced by
    // fused launches over buckets of consecutive tensors (same dtype and
    // operator, about group_bucket_bytes each), issued from the calling thread in
    // list order; host tensors run on worker threads in list order.
    void group_all_reduce(std::vector<std::future<workspace>> ws);
    // Same for tensors that are ready now; on device pointers this is ONE fused
    // launch per staging slot, with `scale` applied in the kernel.
    void group_all_reduce(const std::vector<workspace> &ws, double scale = 1.0,
                          void *stream = nullptr);

    void all_reduce(const void *input, void *output, size_t count, dtype dt, reduce_op op,
                    std::string name = "", void *stream = nullptr);
    // The async interface: starts the operation and returns a task to poll()
    // (or finish()).  Host buffers: the chunk graph as a polled task tree, no
    // thread blocks; device buffers: the kernels are enqueued at once and the
    // task finishes when the GPU has run them.  The buffers must stay alive
    // until the task has finished.
    std::unique_ptr<task> async_all_reduce(const void *input, void *output, size_t count,
                                           dtype dt, reduce_op op, std::string name = "",
                                           void *stream = nullptr);
    // only `root` receives the result (output may be null elsewhere)
    void reduce(const void *input, void *output, size_t count, dtype dt, reduce_op op,
                std::string name = "", void *stream = nullptr, size_t root = 0);
    void all_gather(const void *input, void *output, size_t count, dtype dt,
                    std::string name = "", void *stream = nullptr);
    void gather(const void *input, void *output, size_t count, dtype dt, std::string name = "",
                size_t root = 0);
    // From rank `root` (the reference fixes root 0: session.cpp:49-62 there).
    // Root 0 follows the session's broadcast graph; any other root sends to
    // every member directly.
    void broadcast(const void *input, void *output, size_t count, dtype dt,
                   std::string name = "", void *stream = nullptr, size_t root = 0);
    // Beyond the reference.  reduce_scatter: input holds size() blocks of `count`
    // elements; rank r receives block r reduced over all ranks (folded in rank
    // order).  all_to_all: block q of the input goes to rank q, block q of the
    // output comes from rank q.  Device buffers are staged through host memory.
    void reduce_scatter(const void *input, void *output, size_t count, dtype dt, reduce_op op,
                        std::string name = "", void *stream = nullptr);
    void all_to_all(const void *input, void *output, size_t count, dtype dt,
                    std::string name = "", void *stream = nullptr);
    // Host buffers: the rendezvous message of the TCP path.  Device buffers: NCCL
    // send / recv on a stream of this session's own (libnccl is opened at run
    // time; the two ranks of a pair build a communicator of two on first use).
    // Both return when the buffer may be reused (send) or holds the data (recv);
    // as with MPI, two ranks that send to each other first and receive second
    // may wait for each other for ever: order the calls, or use the async forms.
    void recv(void *output, size_t count, dtype dt, size_t target, std::string name = "");
    void send(const void *input, size_t count, dtype dt, size_t target, std::string name = "");
    // Device buffers: the transfer is enqueued behind the work that `stream`
    // holds now and runs beside the collectives; the task finishes when the GPU
    // has done it.  Host buffers: the call blocks as above and returns a
    // finished task.
    std::unique_ptr<task> async_send(const void *input, size_t count, dtype dt, size_t target,
                                     std::string name = "", void *stream = nullptr);
    std::unique_ptr<task> async_recv(void *output, size_t count, dtype dt, size_t target,
                                     std::string name = "", void *stream = nullptr);

    bool consistent(const void *ptr, size_t size);

    // ------------------------------------------------------- typed overloads
    template <typename R>
    void all_reduce(const R *in, R *out, const size_t count, const std::string &name = "")
    {
        all_reduce(in, out, count, type<R>(), sum, name);
    }

    template <typename R>
    void all_reduce(const R *in, R *out, const size_t count, reduce_op op,
                    const std::string &name = "")
    {
        all_reduce(in, out, count, type<R>(), op, name);
    }

    template <typename R>
    void all_reduce(const R *begin1, const R *end1, R *begin2)
    {
        all_reduce(begin1, begin2, static_cast<size_t>(std::distance(begin1, end1)), type<R>(),
                   sum, "");
    }

    template <typename R>
    void all_reduce(const R *begin1, const R *end1, R *begin2, const std::string &name)
    {
        all_reduce(begin1, begin2, static_cast<size_t>(std::distance(begin1, end1)), type<R>(),
                   sum, name);
    }

    template <typename R>
    void all_reduce(const R *begin1, const R *end1, R *begin2, reduce_op op,
                    const std::string &name = "")
    {
        all_reduce(begin1, begin2, static_cast<size_t>(std::distance(begin1, end1)), type<R>(),
                   op, name);
    }

    template <typename T>
    T all_reduce(const T &x, reduce_op op = sum)
    {
        T y;
        all_reduce(&x, &y, 1, type<T>(), op, "");
        return y;
    }

    template <typename R>
    void all_gather(const R *input, R *output, const size_t count, const std::string &name = "")
    {
        all_gather(input, output, count, type<R>(), name);
    }

    template <typename T>
    bool consistent(const T &x)
    {
        return consistent(&x, sizeof(T));
    }

    template <typename R>
    void broadcast(const R *begin1, const R *end1, R *begin2)
    {
        broadcast(begin1, begin2, static_cast<size_t>(std::distance(begin1, end1)), type<R>());
    }

    template <typename T>
    T broadcast(const T &x)
    {
        T y;
        broadcast(reinterpret_cast<const int8_t *>(&x), reinterpret_cast<int8_t *>(&y), sizeof(T),
                  i8);
        return y;
    }
};

// Which graph pair (ring root) serves a chunk: sum of squared character codes
// of its name, as the reference hashes it (src/stdml/collective/session.cpp:142-149),
// so both implementations spread chunks over roots identically.
size_t name_based_hash(const std::string &name);

std::vector<std::pair<workspace, std::pair<const graph *, const graph *>>>
split_work(const workspace &w, const graph_pair_list &gps, size_t chunk_size);
}  // namespace stdml::collective
