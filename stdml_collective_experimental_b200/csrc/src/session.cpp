#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <cstdlib>
#include <cstring>
#include <numeric>
#include <stdexcept>
#include <thread>

#include <sched.h>

#include <stdml/bits/collective/device.hpp>
#include <stdml/bits/collective/execution.hpp>
#include <stdml/bits/collective/log.hpp>
#include <stdml/bits/collective/session.hpp>
#include <stdml/bits/collective/stat.hpp>

#include "../cuda/device_session.hpp"
#include "../cuda/nccl_p2p.hpp"

namespace stdml::collective
{
using rchan::conn_collective;
using rchan::message_header;

size_t name_based_hash(const std::string &name)
{
    size_t h = 0;
    for (const unsigned char c : name) { h += static_cast<size_t>(c) * c; }
    return h;
}

std::vector<std::pair<workspace, std::pair<const graph *, const graph *>>>
split_work(const workspace &w, const graph_pair_list &gps, size_t chunk_size)
{
    std::vector<std::pair<workspace, std::pair<const graph *, const graph *>>> out;
    for (auto &part : w.split_by_bytes(chunk_size)) {
        const auto gs = gps.choose(name_based_hash(part.name));
        out.emplace_back(std::move(part), gs);
    }
    return out;
}

namespace
{
int default_spin_polls(const peer_list &peers, const peer_id &self);

// STDML_COLLECTIVE_ALGO: auto | oneshot | twoshot | nvls | nvls_oneshot
int forced_algo(const system_config &c)
{
    if (c.device_algo == "oneshot") { return cuda::kAlgoOneShot; }
    if (c.device_algo == "twoshot") { return cuda::kAlgoTwoShot; }
    if (c.device_algo == "nvls") { return cuda::kAlgoNvls; }
    if (c.device_algo == "nvls_oneshot") { return cuda::kAlgoNvlsOneShot; }
    return -1;
}
}  // namespace

session::session(system_config config, size_t version, size_t rank, peer_list peers,
                 peer_list runners, mailbox *eager_box, slotbox *posted_box,
                 rchan::client_pool *client_pool, strategy s, liveness *live, std::string scope)
    : scope_(std::move(scope)), config_(std::move(config)), version_(version), rank_(rank), peers_(std::move(peers)),
      runners_(std::move(runners)), strategy_(s),
      all_reduce_topo_(make_graph_pair_list(s, peers_.size())), mailbox_(eager_box),
      slotbox_(posted_box), client_pool_(client_pool), liveness_(live)
{
    if (rank_ >= peers_.size()) { throw std::invalid_argument("session: rank outside the peer list"); }
    if (config_.thread_pool_size > 0 &&
        (config_.rt == rt_thread_pool || config_.rt == rt_go)) {
        pool_ = sync::thread_pool::make(config_.thread_pool_size);
    }
    async_runtime_.reset(runtime::New(8));
    spin_polls_ = default_spin_polls(peers_, peers_[rank_]);
    // members may still be starting: first connections are retried patiently
    client_pool_->set_dial_patience_ms(-1);
    barrier();
    // every member has answered, so each has a listening server from now on: a
    // connection that is refused means a dead peer, not a late one
    established_ = true;
    client_pool_->set_dial_patience_ms(established_patience_ms);
    // built now, by one thread, rather than by whichever worker gets there first
    if (scope_.empty() && peers_.size() > 1 && spans_hosts()) { two_levels(); }
}

session::~session() = default;
session::session(session &&) noexcept = default;

std::unique_ptr<session> session::subgroup(const std::vector<size_t> &ranks,
                                           const std::string &scope)
{
    if (scope.empty()) { throw std::invalid_argument("subgroup: a scope name is needed"); }
    peer_list members;
    size_t me = ranks.size();
    for (size_t i = 0; i < ranks.size(); ++i) {
        if (ranks[i] >= peers_.size()) { throw std::out_of_range("subgroup: no such rank"); }
        for (size_t j = 0; j < i; ++j) {
            if (ranks[j] == ranks[i]) { throw std::invalid_argument("subgroup: rank listed twice"); }
        }
        if (ranks[i] == rank_) { me = i; }
        members.push_back(peers_[ranks[i]]);
    }
    if (me == ranks.size()) { return nullptr; }  // not a member: nothing to take part in
    const std::string full = scope_.empty() ? scope : scope_ + "/" + scope;
    return std::make_unique<session>(config_, version_, me, members, runners_, mailbox_, slotbox_,
                                     client_pool_, strategy_, liveness_, full);
}

void session::barrier()
{
    uint32_t one = 1, all = 0;
    all_reduce(&one, &all, 1, u32, sum, "stdml::barrier::v" + std::to_string(version_));
}

// ---------------------------------------------------------------- host path
namespace
{
std::string versioned(const session &s, const std::string &name)
{
    // keeps messages of an old membership from matching operations of a new one,
    // and those of a sub-group from matching the whole group's
    std::string out = s.version() == 0 ? name : name + "@v" + std::to_string(s.version());
    if (!s.scope().empty()) { out += "#" + s.scope(); }
    return out;
}
}  // namespace

// The polled tasks' form of source_gone(): looks at the clock once in a while.
bool session::polled_source_gone(const peer_id &who, poll_watch &w) const
{
    using clock = std::chrono::steady_clock;
    if (liveness_ == nullptr) { return false; }
    if (liveness_->gone(who)) { return true; }
    if ((++w.polls & 1023u) != 0) { return false; }
    const auto now = clock::now();
    if (w.start == clock::time_point()) {
        w.start = w.asked = now;
        return false;
    }
    const auto ms = [](clock::duration d) {
        return std::chrono::duration_cast<std::chrono::milliseconds>(d).count();
    };
    const long long patience =
        established_ ? established_patience_ms / 2 : rchan::connect_timeout_ms();
    if (patience > 0 && ms(now - w.start) >= patience && ms(now - w.asked) >= 1000 &&
        !liveness_->seen(who)) {
        w.asked = now;
        return rchan::ping(who, peers_[rank_], 1000) < 0;
    }
    return false;
}

namespace
{
// How many times a receiver looks for its message before it goes to sleep.
// Meeting a message awake saves a wake-up per hop (measured on 4 ranks, 4 KB
// tensors: ring +35 %, star +30 %), but only while every rank has cores to
// spare: on 8 ranks sharing 8 cores the same spin cost a factor of three.  So
// the default spins only when this process may run on at least two cores per
// rank of this host.  STDML_COLLECTIVE_SPIN_POLLS overrides (0: never spin).
int default_spin_polls(const peer_list &peers, const peer_id &self)
{
    if (const auto v = parse_env_int("STDML_COLLECTIVE_SPIN_POLLS"); v && *v >= 0) {
        return static_cast<int>(*v);
    }
    size_t local = 0;
    for (const auto &p : peers) { local += p.ipv4 == self.ipv4 ? 1 : 0; }
    cpu_set_t set;
    CPU_ZERO(&set);
    const size_t cores = ::sched_getaffinity(0, sizeof(set), &set) == 0
                             ? static_cast<size_t>(CPU_COUNT(&set))
                             : std::thread::hardware_concurrency();
    return cores >= 2 * std::max<size_t>(local, 1) ? 10000 : 0;
}

// Spinning is for a thread that is the only receiver of its process: a single
// small operation on the calling thread.  Lanes of a chunked tensor and the
// workers of a fused group keep several receivers waiting at once (all of them
// spinning costs more than it saves: measured), so they sleep at once.
thread_local int tl_spin_polls = 0;
thread_local bool tl_in_group = false;

struct spin_scope {
    int saved;
    explicit spin_scope(int polls) : saved(tl_spin_polls) { tl_spin_polls = tl_in_group ? 0 : polls; }
    ~spin_scope() { tl_spin_polls = saved; }
};

inline void cpu_relax()
{
#if defined(__x86_64__) || defined(__i386__)
    __builtin_ia32_pause();
#else
    std::this_thread::yield();
#endif
}
}  // namespace

bool session::source_gone(size_t src, long long waited_ms) const
{
    if (liveness_ == nullptr) { return false; }
    if (liveness_->gone(peers_[src])) { return true; }
    // never heard of it (no message of it has come our way yet): ask it about once
    // a second, at once in a session whose members have all been seen alive, after
    // a dialler's patience while they may still be starting
    const long long patience =
        established_ ? established_patience_ms / 2 : rchan::connect_timeout_ms();
    if (patience > 0 && waited_ms >= patience &&
        (waited_ms / liveness::slice_ms) % 10 == 0 && !liveness_->seen(peers_[src])) {
        return rchan::ping(peers_[src], peers_[rank_], 1000) < 0;
    }
    return false;
}

void session::ensure_usable(const char *what)
{
    if (given_up()) { give_up(failure::other, peers_[rank_], what, "(not started)"); }
}

bool session::given_up() const
{
    return broken_->load() || (liveness_ != nullptr && liveness_->aborted(version_));
}

// The first failure of a session tells the other members (an empty message
// named liveness::abort_tag(version)): a member that waits for this rank, which
// is alive but will never answer, gives up as well.  Members that are known to
// be dead, or do not accept a connection within half a second, are skipped.
void session::abort() noexcept
{
    if (broken_->exchange(true) || liveness_ == nullptr) { return; }
    try {
        const std::string tag = liveness::abort_tag(version_);
        for (size_t r = 0; r < peers_.size(); ++r) {
            if (r == rank_ || liveness_->gone(peers_[r])) { continue; }
            try {
                // a connection of its own, made with a deadline: the pooled ones are
                // dialled with a starter's patience, which a dying member does not deserve
                auto c = rchan::connection::dial_once(peers_[r], rchan::conn_control, peers_[rank_], 500);
                if (c) { c->send(tag.c_str(), nullptr, 0, 0); }
            } catch (const std::exception &) {
                // that member has gone too
            }
        }
    } catch (const std::exception &) {
    }
}

void session::give_up(failure why, const peer_id &who, const char *what, const std::string &tag)
{
    const long long limit = config_.host_timeout_ms;
    switch (why) {
    case failure::gone:
        abort();
        throw peer_failure(who, std::string(what) + " '" + tag + "': peer " + who.str() +
                                    " has gone (its connections closed, or it never connected "
                                    "and does not answer)");
    case failure::late:
        abort();
        throw std::runtime_error(std::string(what) + " '" + tag + "': nothing from peer " +
                                 who.str() + " within " + std::to_string(limit) +
                                 " ms (peer failed or left?)");
    default:
        break;
    }
    abort();
    throw peer_failure(who, std::string(what) + " '" + tag +
                                "': given up, this session has lost a member (another receive "
                                "failed, or a member told us so)");
}

buffer session::take_eager(size_t src, const std::string &tag, const char *what)
{
    auto *box = mailbox_->require(peers_[src], tag);
    // a message that is about to arrive is cheaper to meet spinning than asleep
    for (int spin = 0; spin < tl_spin_polls; ++spin) {
        if (auto got = box->try_get()) { return std::move(*got); }
        cpu_relax();
    }
    const long long limit = config_.host_timeout_ms;
    long long waited = 0;
    for (;;) {
        const long long slice =
            limit > 0 ? std::min(liveness::slice_ms, limit - waited) : liveness::slice_ms;
        if (auto got = box->get_for(std::chrono::milliseconds(slice))) { return std::move(*got); }
        waited += slice;
        if (source_gone(src, waited)) {
            // what it sent before it went has been handed over by now
            if (auto got = box->try_get()) { return std::move(*got); }
            give_up(failure::gone, peers_[src], what, tag);
        }
        if (limit > 0 && waited >= limit) { give_up(failure::late, peers_[src], what, tag); }
        if (given_up()) { give_up(failure::other, peers_[src], what, tag); }
    }
}

void session::finish_pending(slot::pending &p, size_t src, const std::string &tag, const char *what)
{
    for (int spin = 0; spin < tl_spin_polls && p.ready() < 0; ++spin) { cpu_relax(); }
    const long long limit = config_.host_timeout_ms;
    long long waited = 0;
    for (;;) {
        const long long slice =
            limit > 0 ? std::min(liveness::slice_ms, limit - waited) : liveness::slice_ms;
        int rc = p.wait(slice);
        if (rc < 0) {
            waited += slice;
            const bool gone = source_gone(src, waited);
            const bool late = limit > 0 && waited >= limit;
            if (!gone && !late && !given_up()) { continue; }
            if (p.cancel()) {
                give_up(gone ? failure::gone : late ? failure::late : failure::other, peers_[src],
                        what, tag);
            }
            rc = p.wait(0);  // it was delivered while we were giving up
        }
        if (rc == 0) {
            throw std::length_error(std::string(what) + ": the message from peer " +
                                    peers_[src].str() + " is longer than the posted buffer");
        }
        return;
    }
}

void session::take_into(size_t src, const std::string &tag, void *dst, size_t cap,
                        const char *what)
{
    slot::pending p = slotbox_->require(peers_[src], tag)->post_pending(dst, cap);
    finish_pending(p, src, tag, what);
}

void session::run_chunk(const workspace &w, const graph *rg, const graph *bg)
{
    workspace_state st(&w);
    const std::string name = versioned(*this, w.name);
    const size_t bytes = w.bytes();
    rchan::client *out = client_pool_->require(conn_collective);

    auto recv_reduce = [&](size_t src) {
        buffer b = take_eager(src, name, "all_reduce");
        if (b.len != bytes) {
            throw std::runtime_error("all_reduce: peer " + peers_[src].str() + " sent " +
                                     std::to_string(b.len) + " bytes for '" + w.name +
                                     "', expected " + std::to_string(bytes));
        }
        st.add_to(b.data.get());
    };
    auto send_partial = [&](size_t dst) {
        out->send(peers_[dst], name.c_str(), st.effective_data(), bytes, 0);
    };
    auto recv_result = [&](size_t src) {
        take_into(src, name, w.recv, bytes, "all_reduce");
        st.replaced();
    };
    auto send_result = [&](size_t dst) {
        out->send(peers_[dst], name.c_str(), w.recv, bytes, message_header::wait_recv_buf);
    };

    // Below a full chunk the messages fit the socket buffers, so sends do not
    // block, and starting a thread per neighbour costs more than copying in
    // turn; everything runs on the calling thread, in order.
    const bool tiny = bytes <= tiny_chunk_bytes;
    // reduce graph: accumulate what the predecessors send, pass the partial on
    if (tiny) {
        fmap(seq, recv_reduce, rg->prevs(rank_));
        fmap(seq, send_partial, rg->nexts(rank_));
    } else if (pool_) {
        fmap(pool_.get(), recv_reduce, rg->prevs(rank_));
        fmap(pool_.get(), send_partial, rg->nexts(rank_));
    } else {
        fmap(par, recv_reduce, rg->prevs(rank_));
        fmap(par, send_partial, rg->nexts(rank_));
    }
    // broadcast graph: the root already holds the result
    if (bg->prevs(rank_).empty()) {
        if (st.received() == 0) { st.forward(); }
    } else {
        fmap(seq, recv_result, bg->prevs(rank_));
    }
    if (tiny) {
        fmap(seq, send_result, bg->nexts(rank_));
    } else if (pool_) {
        fmap(pool_.get(), send_result, bg->nexts(rank_));
    } else {
        fmap(par, send_result, bg->nexts(rank_));
    }
}

// The same chunk as a polled task tree (rt_async): nothing in it blocks.
task *session::chunk_task(const workspace &w, const graph *rg, const graph *bg)
{
    struct shared {
        workspace w;
        workspace_state st;
        std::string name;
        explicit shared(const workspace &x) : w(x), st(&w) {}
    };
    auto sh = std::make_shared<shared>(w);
    sh->name = versioned(*this, w.name);
    const size_t bytes = w.bytes();
    rchan::client *out = client_pool_->require(conn_collective);

    task_builder recv1, send1, recv2, send2;
    for (size_t src : rg->prevs(rank_)) {
        auto *box = mailbox_->require(peers_[src], sh->name);
        auto got = std::make_shared<buffer>();
        auto watch = std::make_shared<poll_watch>();
        const peer_id who = peers_[src];
        recv1 << new poll_task(
            [this, box, got, watch, who, sh] {
                auto b = box->try_get();
                if (!b && polled_source_gone(who, *watch)) {
                    b = box->try_get();  // sent before it went
                    if (!b) { give_up(failure::gone, who, "all_reduce", sh->name); }
                }
                if (!b) {
                    if (given_up()) { give_up(failure::other, who, "all_reduce", sh->name); }
                    return false;
                }
                *got = std::move(*b);
                return true;
            },
            [sh, got, bytes] {
                if (got->len != bytes) { throw std::runtime_error("all_reduce: size mismatch"); }
                sh->st.add_to(got->data.get());
            });
    }
    for (size_t dst : rg->nexts(rank_)) {
        const peer_id target = peers_[dst];
        send1 << new simple_task([sh, out, target, bytes] {
            out->send(target, sh->name.c_str(), sh->st.effective_data(), bytes, 0);
        });
    }
    if (bg->prevs(rank_).empty()) {
        recv2 << new simple_task([sh] {
            if (sh->st.received() == 0) { sh->st.forward(); }
        });
    } else {
        for (size_t src : bg->prevs(rank_)) {
            auto *sl = slotbox_->require(peers_[src], sh->name);
            // withdrawn with the task if the tree is abandoned (another task threw):
            // nothing may be written into the user's buffer after all_reduce has returned
            struct posted {
                slot::pending p;
                ~posted()
                {
                    if (p && !p.settled()) { p.cancel(); }
                }
            };
            auto pend = std::make_shared<posted>();
            auto watch = std::make_shared<poll_watch>();
            const peer_id who = peers_[src];
            recv2 << new poll_task([this, sl, sh, pend, bytes, watch, who] {
                // the destination is posted on the first poll, i.e. after the
                // reduce phase is over and recv no longer holds partial sums
                if (!pend->p) { pend->p = sl->post_pending(sh->w.recv, bytes); }
                int rc = pend->p.ready();
                if (rc < 0) {
                    const bool gone = polled_source_gone(who, *watch);
                    if (!gone && !given_up()) { return false; }
                    if (pend->p.cancel()) {
                        give_up(gone ? failure::gone : failure::other, who, "all_reduce", sh->name);
                    }
                    rc = pend->p.wait(0);
                }
                if (rc == 0) { throw std::length_error("all_reduce: the result did not fit"); }
                return true;
            });
        }
    }
    for (size_t dst : bg->nexts(rank_)) {
        const peer_id target = peers_[dst];
        send2 << new simple_task([sh, out, target, bytes] {
            out->send(target, sh->name.c_str(), sh->w.recv, bytes, message_header::wait_recv_buf);
        });
    }
    task_builder steps;
    steps << recv1.par();
    steps << send1.par();
    steps << recv2.seq();
    steps << send2.par();
    return steps.seq();
}

void session::all_reduce(const workspace &w, void *stream)
{
    STDML_COLLECTIVE_PROFILE_RATE("all_reduce", w.bytes());
    if (!reduce_supported(w.dt, w.op)) {
        throw std::invalid_argument(std::string("all_reduce: ") + reduce_op_name(w.op) +
                                    " is not defined for " + dtype_name(w.dt));
    }
    if (w.count == 0) { return; }
    ensure_usable("all_reduce");
    const bool dev = on_device(w.send, w.recv);
    if (scope_.empty() && peers_.size() > 1 && (dev || config_.hierarchical) && spans_hosts()) {
        all_reduce_two_level(w, dev, stream);
        return;
    }
    if (dev) {
        const void *in[1] = {w.send};
        void *out[1] = {w.recv};
        device()->all_reduce(in, out, w.count, w.dt, w.op, 1.0, forced_algo(config_), stream);
        return;
    }
    if (peers_.size() == 1) {
        w.forward();
        return;
    }
    const auto work = split_work(w, all_reduce_topo_, chunk_bytes);
    if (config_.rt == rt_async || config_.rt == rt_coro) {
        std::vector<std::unique_ptr<task>> ts;
        for (const auto &[part, gs] : work) {
            ts.emplace_back(chunk_task(part, gs.first, gs.second));
        }
        std::unique_ptr<task> all(task::par(std::move(ts), async_runtime_.get()));
        all->finish();
        return;
    }
    // Chunks are independent (distinct names, spread over the ring roots), so a
    // few of them are kept in flight; every rank starts them in the same order,
    // which keeps the pipeline free of deadlocks (see group_all_reduce).  The
    // reference runs the chunks of one tensor strictly one after another
    // (src/stdml/collective/run_graph_pair_list_multi_thread.cpp:93-95).
    // measured on 4 ranks: ring 4 -> 8 +8 %, star 1 -> 2 +33 %; the tree spreads its roots like the ring
    size_t lanes = strategy_ == star ? 2 : 8;
    if (const auto v = parse_env_int("STDML_COLLECTIVE_CHUNK_LANES"); v && *v > 0) {
        lanes = static_cast<size_t>(*v);
    }
    lanes = std::min(lanes, work.size());
    if (lanes <= 1) {
        spin_scope spin(spin_polls_);
        for (const auto &[part, gs] : work) { run_chunk(part, gs.first, gs.second); }
        return;
    }
    std::atomic<size_t> next{0};
    std::mutex err_mu;
    std::exception_ptr err;
    auto lane = [&] {
        for (;;) {
            const size_t i = next.fetch_add(1);
            if (i >= work.size()) { return; }
            try {
                run_chunk(work[i].first, work[i].second.first, work[i].second.second);
            } catch (...) {
                std::lock_guard<std::mutex> lk(err_mu);
                if (!err) { err = std::current_exception(); }
            }
        }
    };
    std::vector<std::thread> ths;
    for (size_t t = 1; t < lanes; ++t) { ths.emplace_back(lane); }
    lane();
    for (auto &t : ths) { t.join(); }
    if (err) { std::rethrow_exception(err); }
}

bool session::spans_hosts() const
{
    for (const auto &p : peers_) {
        if (p.ipv4 != peers_[0].ipv4) { return true; }
    }
    return false;
}

session::levels &session::two_levels()
{
    if (levels_) { return *levels_; }
    auto lv = std::make_unique<levels>();
    std::vector<size_t> local, leaders;
    for (size_t r = 0; r < peers_.size(); ++r) {
        if (peers_[r].ipv4 == peers_[rank_].ipv4) { local.push_back(r); }
        bool first_of_host = true;
        for (size_t q = 0; q < r; ++q) { first_of_host = first_of_host && peers_[q].ipv4 != peers_[r].ipv4; }
        if (first_of_host) { leaders.push_back(r); }
    }
    lv->local = subgroup(local, "host-" + peers_[rank_].hostname());
    lv->leaders = subgroup(leaders, "leaders");  // null unless this rank leads its host
    log() << "two-level all_reduce:" << local.size() << "ranks on this host," << leaders.size()
          << "hosts" << (lv->leaders ? "(leader)" : "");
    levels_ = std::move(lv);
    return *levels_;
}

// Reduce inside each host, all-reduce among one leader per host, broadcast
// inside each host: the links between hosts carry one flow per host instead of
// one per rank.  Device buffers take this path whenever the members span hosts:
// the two inner stages run on the host's GPUs over NVLink, the leaders' stage
// goes through host memory and the network.
void session::all_reduce_two_level(const workspace &w, bool device, void *stream, double scale)
{
    levels &lv = two_levels();
    const std::string name = "2l::" + w.name;
    lv.local->reduce(w.send, w.recv, w.count, w.dt, w.op, name, stream, 0);
    if (lv.leaders) {
        if (device) {
            std::vector<char> host(w.bytes());
            cuda::copy_device_to_host(host.data(), w.recv, host.size(), stream);
            lv.leaders->all_reduce(host.data(), host.data(), w.count, w.dt, w.op, name);
            if (scale != 1.0) { scale_in_place(host.data(), w.count, w.dt, scale); }
            cuda::copy_host_to_device(w.recv, host.data(), host.size(), stream);
        } else {
            lv.leaders->all_reduce(w.recv, w.recv, w.count, w.dt, w.op, name);
            if (scale != 1.0) { scale_in_place(w.recv, w.count, w.dt, scale); }
        }
    }
    lv.local->broadcast(w.recv, w.recv, w.count, w.dt, name, stream, 0);
}

void session::all_reduce(const void *input, void *output, size_t count, dtype dt, reduce_op op,
                         std::string name, void *stream)
{
    workspace w;
    w.send = input;
    w.recv = output;
    w.count = count;
    w.dt = dt;
    w.op = op;
    w.name = std::move(name);
    all_reduce(w, stream);
}

std::unique_ptr<task> session::async_all_reduce(const void *input, void *output, size_t count,
                                                dtype dt, reduce_op op, std::string name,
                                                void *stream)
{
    if (!reduce_supported(dt, op)) {
        throw std::invalid_argument("async_all_reduce: undefined dtype/op pair");
    }
    workspace w;
    w.send = input;
    w.recv = output;
    w.count = count;
    w.dt = dt;
    w.op = op;
    w.name = std::move(name);
    if (count == 0) { return std::make_unique<noop_task>(); }
    if (on_device(input, output)) {
        all_reduce(w, stream);  // enqueues and returns
        return std::make_unique<event_task>(stream);
    }
    if (peers_.size() == 1) {
        w.forward();
        return std::make_unique<noop_task>();
    }
    std::vector<std::unique_ptr<task>> ts;
    for (const auto &[part, gs] : split_work(w, all_reduce_topo_, chunk_bytes)) {
        ts.emplace_back(chunk_task(part, gs.first, gs.second));
    }
    return std::unique_ptr<task>(task::par(std::move(ts)));
}

void session::group_all_reduce(const std::vector<workspace> &ws, double scale, void *stream)
{
    if (ws.empty()) { return; }
    bool dev = true, same = true;
    for (const auto &w : ws) {
        dev = dev && on_device(w.send, w.recv);
        same = same && w.dt == ws[0].dt && w.op == ws[0].op;
    }
    if (dev && scope_.empty() && peers_.size() > 1 && spans_hosts()) {
        // members on several hosts: tensor by tensor through the two-level path
        // (the fused kernel needs one NVLink domain)
        for (const auto &w : ws) {
            if (w.count == 0) { continue; }
            if (!reduce_supported(w.dt, w.op)) { throw std::invalid_argument("group_all_reduce: undefined dtype/op"); }
            ensure_usable("group_all_reduce");
            all_reduce_two_level(w, true, stream, scale);
        }
        return;
    }
    if (dev && same) {
        std::vector<const void *> ins;
        std::vector<void *> outs;
        std::vector<size_t> counts;
        for (const auto &w : ws) {
            ins.push_back(w.send);
            outs.push_back(w.recv);
            counts.push_back(w.count);
        }
        device()->group_all_reduce(ws.size(), ins.data(), outs.data(), counts.data(), ws[0].dt,
                                   ws[0].op, -1, scale, forced_algo(config_), stream);
        return;
    }
    std::vector<std::future<workspace>> fs;
    for (const auto &w : ws) {
        std::promise<workspace> p;
        p.set_value(w);
        fs.push_back(p.get_future());
    }
    group_all_reduce(std::move(fs));
    if (scale != 1.0) {
        for (const auto &w : ws) { scale_in_place(w.recv, w.count, w.dt, scale); }
    }
}

void session::group_all_reduce(std::vector<std::future<workspace>> fs)
{
    // ONE thread (the caller's) takes the futures in submission order, which is
    // the same on every rank (futures are positional), whatever order they
    // resolve in.
    //   * Host tensors go, in that order, to a small set of workers.  The
    //     earliest unfinished tensor is therefore always being worked on by every
    //     rank, so the group cannot deadlock (the reference runs each tensor on
    //     an ad-hoc pool of 76 threads as it becomes ready, which deadlocks for
    //     larger sets: src/stdml/collective/session.cpp:83-97).
    //   * Device tensors are collected into buckets and every bucket is ONE
    //     fused launch, issued by this thread only.  A bucket ends where the
    //     dtype or the operator changes, where a host tensor comes in between,
    //     and once it holds group_bucket_bytes: all of these depend on the list
    //     alone, never on when a future resolved, so every rank cuts the same
    //     buckets and the kernels of different ranks pair up.
    const size_t n = fs.size();
    if (n == 0) { return; }
    size_t workers = 8;
    if (pool_) {
        const size_t fan = std::max<size_t>(1, peers_.size() - 1);
        workers = std::max<size_t>(1, std::min<size_t>(8, pool_->size() / fan));
    }
    workers = std::min(workers, n);

    std::mutex mu;
    std::condition_variable cv;
    std::deque<workspace> host_q;
    bool closed = false;
    std::atomic<bool> failed{false};
    std::exception_ptr err;
    auto note_error = [&] {
        failed.store(true);
        std::lock_guard<std::mutex> lk(mu);
        if (!err) { err = std::current_exception(); }
    };
    auto work = [&] {
        struct in_group {
            bool saved = tl_in_group;
            in_group() { tl_in_group = true; }
            ~in_group() { tl_in_group = saved; }
        } mark;
        for (;;) {
            workspace w;
            {
                std::unique_lock<std::mutex> lk(mu);
                cv.wait(lk, [&] { return closed || !host_q.empty(); });
                if (host_q.empty()) { return; }
                w = host_q.front();
                host_q.pop_front();
            }
            try {
                if (!failed.load()) { all_reduce(w); }
            } catch (...) {
                note_error();
            }
        }
    };
    std::vector<std::thread> ths;  // started when the first host tensor shows up

    std::vector<workspace> bucket;
    size_t bucket_bytes = 0;
    auto flush = [&] {
        if (bucket.empty()) { return; }
        std::vector<workspace> b;
        b.swap(bucket);
        bucket_bytes = 0;
        if (!failed.load()) { group_all_reduce(b, 1.0, nullptr); }
    };
    for (size_t i = 0; i < n; ++i) {
        try {
            const workspace w = fs[i].get();
            if (failed.load() || w.count == 0) { continue; }
            if (on_device(w.send, w.recv)) {
                if (!bucket.empty() && (bucket[0].dt != w.dt || bucket[0].op != w.op)) { flush(); }
                bucket.push_back(w);
                bucket_bytes += w.count * dtype_size(w.dt);
                if (bucket_bytes >= group_bucket_bytes) { flush(); }
            } else {
                flush();
                if (ths.empty()) {
                    for (size_t t = 0; t < workers; ++t) { ths.emplace_back(work); }
                }
                {
                    std::lock_guard<std::mutex> lk(mu);
                    host_q.push_back(w);
                }
                cv.notify_one();
            }
        } catch (...) {
            note_error();
        }
    }
    try {
        flush();
    } catch (...) {
        note_error();
    }
    {
        std::lock_guard<std::mutex> lk(mu);
        closed = true;
    }
    cv.notify_all();
    for (auto &t : ths) { t.join(); }
    if (err) { std::rethrow_exception(err); }
}

void session::reduce(const void *input, void *output, size_t count, dtype dt, reduce_op op,
                     std::string name, void *stream, size_t root)
{
    if (count == 0) { return; }
    if (!reduce_supported(dt, op)) { throw std::invalid_argument("reduce: undefined dtype/op"); }
    if (root >= peers_.size()) { throw std::out_of_range("reduce: no such root"); }
    ensure_usable("reduce");
    if (on_device(input, output != nullptr ? output : input)) {
        if (scope_.empty() && spans_hosts()) {
            // members on several hosts: through host memory and the network
            const size_t nbytes = count * dtype_size(dt);
            std::vector<char> a(nbytes), b(rank_ == root ? nbytes : 0);
            cuda::copy_device_to_host(a.data(), input, nbytes, stream);
            reduce(a.data(), rank_ == root ? b.data() : nullptr, count, dt, op, "dev::" + name,
                   nullptr, root);
            if (rank_ == root) { cuda::copy_host_to_device(output, b.data(), nbytes, stream); }
            return;
        }
        const void *in[1] = {input};
        void *out[1] = {output};
        device()->reduce(in, out, count, dt, op, static_cast<int>(root), 1.0, stream);
        return;
    }
    // the root gathers the operands and folds them in rank order, left to right
    const size_t bytes = count * dtype_size(dt);
    const std::string tag = versioned(*this, "stdml::reduce::" + name);
    if (rank_ != root) {
        client_pool_->require(conn_collective)->send(peers_[root], tag.c_str(), input, bytes, 0);
        return;
    }
    bool started = false;  // output holds the fold of the ranks before r
    std::vector<char> mine;
    if (output == input && root != 0) {
        // in place on a root that is not first: keep the own operand aside
        mine.assign(static_cast<const char *>(input), static_cast<const char *>(input) + bytes);
    }
    for (size_t r = 0; r < peers_.size(); ++r) {
        const void *operand;
        buffer b;
        if (r == root) {
            operand = mine.empty() ? input : mine.data();
        } else {
            b = take_eager(r, tag, "reduce");
            if (b.len != bytes) { throw std::runtime_error("reduce: size mismatch"); }
            operand = b.data.get();
        }
        if (!started) {
            if (output != operand) { std::memcpy(output, operand, bytes); }
            started = true;
        } else {
            stdml::collective::reduce(output, output, operand, count, dt, op);
        }
    }
}

void session::all_gather(const void *input, void *output, size_t count, dtype dt,
                         std::string name, void *stream)
{
    if (count == 0) { return; }
    if (on_device(input, output)) {
        if (scope_.empty() && spans_hosts()) {
            // members on several hosts: through host memory and the network
            const size_t nbytes = count * dtype_size(dt);
            std::vector<char> a(nbytes), all(nbytes * peers_.size());
            cuda::copy_device_to_host(a.data(), input, nbytes, stream);
            all_gather(a.data(), all.data(), count, dt, "dev::" + name, nullptr);
            cuda::copy_host_to_device(output, all.data(), all.size(), stream);
            return;
        }
        const void *in[1] = {input};
        void *out[1] = {output};
        device()->all_gather(in, out, count, dt, stream);
        return;
    }
    const size_t bytes = count * dtype_size(dt);
    ensure_usable("all_gather");
    const std::string tag = versioned(*this, "stdml::all_gather::" + name);
    char *out = static_cast<char *>(output);
    // post every destination first, then send: the bodies land in place
    std::vector<std::pair<size_t, slot::pending>> waits;
    for (size_t r = 0; r < peers_.size(); ++r) {
        if (r == rank_) { continue; }
        waits.emplace_back(r, slotbox_->require(peers_[r], tag)->post_pending(out + r * bytes, bytes));
    }
    std::memmove(out + rank_ * bytes, input, bytes);
    std::vector<size_t> others;
    for (size_t r = 1; r < peers_.size(); ++r) { others.push_back((rank_ + r) % peers_.size()); }
    rchan::client *cl = client_pool_->require(conn_collective);
    auto send_to = [&](size_t r) {
        cl->send(peers_[r], tag.c_str(), input, bytes, message_header::wait_recv_buf);
    };
    std::exception_ptr first;
    try {
        if (pool_) {
            fmap(pool_.get(), send_to, others);
        } else {
            fmap(par, send_to, others);
        }
    } catch (...) {
        first = std::current_exception();  // the posted destinations are withdrawn below
    }
    for (auto &[r, p] : waits) {
        if (first) {
            p.cancel();  // nothing may be written into `output` after we have thrown
            continue;
        }
        try {
            finish_pending(p, r, tag, "all_gather");
        } catch (...) {
            first = std::current_exception();
        }
    }
    if (first) { std::rethrow_exception(first); }
}

void session::gather(const void *input, void *output, size_t count, dtype dt, std::string name,
                     size_t root)
{
    if (count == 0) { return; }
    if (root >= peers_.size()) { throw std::out_of_range("gather: no such root"); }
    ensure_usable("gather");
    const size_t bytes = count * dtype_size(dt);
    const std::string tag = versioned(*this, "stdml::gather::" + name);
    if (rank_ != root) {
        client_pool_->require(conn_collective)
            ->send(peers_[root], tag.c_str(), input, bytes, message_header::wait_recv_buf);
        return;
    }
    char *out = static_cast<char *>(output);
    std::memmove(out + root * bytes, input, bytes);
    for (size_t r = 0; r < peers_.size(); ++r) {
        if (r != root) { take_into(r, tag, out + r * bytes, bytes, "gather"); }
    }
}

void session::broadcast(const void *input, void *output, size_t count, dtype dt,
                        std::string name, void *stream, size_t root)
{
    if (count == 0) { return; }
    if (root >= peers_.size()) { throw std::out_of_range("broadcast: no such root"); }
    if (on_device(input, output)) {
        if (scope_.empty() && spans_hosts()) {
            // members on several hosts: through host memory and the network
            const size_t nbytes = count * dtype_size(dt);
            std::vector<char> a(nbytes);
            if (rank_ == root) { cuda::copy_device_to_host(a.data(), input, nbytes, stream); }
            broadcast(a.data(), a.data(), count, dt, "dev::" + name, nullptr, root);
            cuda::copy_host_to_device(output, a.data(), nbytes, stream);
            return;
        }
        const void *in[1] = {input};
        void *out[1] = {output};
        device()->broadcast(in, out, count, dt, static_cast<int>(root), stream);
        return;
    }
    if (root != 0) {
        ensure_usable("broadcast");
        const size_t nbytes = count * dtype_size(dt);
        const std::string rtag =
            versioned(*this, "stdml::broadcast::r" + std::to_string(root) + "::" + name);
        if (rank_ != root) {
            take_into(root, rtag, output, nbytes, "broadcast");
            return;
        }
        if (output != input) { std::memcpy(output, input, nbytes); }
        std::vector<size_t> others;
        for (size_t r = 0; r < peers_.size(); ++r) {
            if (r != root) { others.push_back(r); }
        }
        rchan::client *cl = client_pool_->require(conn_collective);
        fmap(par, [&](size_t r) {
            cl->send(peers_[r], rtag.c_str(), output, nbytes, message_header::wait_recv_buf);
        }, others);
        return;
    }
    const size_t bytes = count * dtype_size(dt);
    ensure_usable("broadcast");
    const std::string tag = versioned(*this, "stdml::broadcast::" + name);
    const graph &g = all_reduce_topo_.pairs[0].broadcast_graph;  // rooted at rank 0
    if (g.prevs(rank_).empty()) {
        if (output != input) { std::memcpy(output, input, bytes); }
    } else {
        for (size_t src : g.prevs(rank_)) {
            take_into(src, tag, output, bytes, "broadcast");
        }
    }
    rchan::client *cl = client_pool_->require(conn_collective);
    auto send_to = [&](size_t r) {
        cl->send(peers_[r], tag.c_str(), output, bytes, message_header::wait_recv_buf);
    };
    fmap(par, send_to, g.nexts(rank_));
}

void session::reduce_scatter(const void *input, void *output, size_t count, dtype dt,
                             reduce_op op, std::string name, void *stream)
{
    if (count == 0) { return; }
    if (!reduce_supported(dt, op)) { throw std::invalid_argument("reduce_scatter: undefined dtype/op"); }
    ensure_usable("reduce_scatter");
    const size_t bytes = count * dtype_size(dt), n = peers_.size();
    if (on_device(input, output)) {
        std::vector<char> a(bytes * n), b(bytes);
        cuda::copy_device_to_host(a.data(), input, a.size(), stream);
        reduce_scatter(a.data(), b.data(), count, dt, op, "dev::" + name, nullptr);
        cuda::copy_host_to_device(output, b.data(), bytes, stream);
        return;
    }
    // one rooted reduce per block; a rank only sends (eagerly) for the blocks of
    // others, so going through the blocks in order cannot deadlock
    const char *in = static_cast<const char *>(input);
    std::vector<char> own;
    if (output == static_cast<const void *>(in + rank_ * bytes) || output == input) {
        own.assign(in + rank_ * bytes, in + (rank_ + 1) * bytes);  // output overlaps the input
    }
    for (size_t q = 0; q < n; ++q) {
        const void *block = (q == rank_ && !own.empty()) ? own.data() : in + q * bytes;
        reduce(block, q == rank_ ? output : nullptr, count, dt, op,
               "rs" + std::to_string(q) + "::" + name, nullptr, q);
    }
}

void session::all_to_all(const void *input, void *output, size_t count, dtype dt,
                         std::string name, void *stream)
{
    if (count == 0) { return; }
    ensure_usable("all_to_all");
    const size_t bytes = count * dtype_size(dt), n = peers_.size();
    if (on_device(input, output)) {
        std::vector<char> a(bytes * n), b(bytes * n);
        cuda::copy_device_to_host(a.data(), input, a.size(), stream);
        all_to_all(a.data(), b.data(), count, dt, "dev::" + name, nullptr);
        cuda::copy_host_to_device(output, b.data(), b.size(), stream);
        return;
    }
    if (input == output) { throw std::invalid_argument("all_to_all: in place is not supported"); }
    const std::string tag = versioned(*this, "stdml::all_to_all::" + name);
    const char *in = static_cast<const char *>(input);
    char *out = static_cast<char *>(output);
    // post every destination first, then send: the bodies land in place
    std::vector<std::pair<size_t, slot::pending>> waits;
    for (size_t r = 0; r < n; ++r) {
        if (r != rank_) {
            waits.emplace_back(r, slotbox_->require(peers_[r], tag)->post_pending(out + r * bytes, bytes));
        }
    }
    std::memcpy(out + rank_ * bytes, in + rank_ * bytes, bytes);
    std::vector<size_t> others;
    for (size_t k = 1; k < n; ++k) { others.push_back((rank_ + k) % n); }
    rchan::client *cl = client_pool_->require(conn_collective);
    std::exception_ptr first;
    try {
        fmap(par, [&](size_t r) {
            cl->send(peers_[r], tag.c_str(), in + r * bytes, bytes, message_header::wait_recv_buf);
        }, others);
    } catch (...) {
        first = std::current_exception();
    }
    for (auto &[r, p] : waits) {
        if (first) {
            p.cancel();  // nothing may be written into `output` after we have thrown
            continue;
        }
        try {
            finish_pending(p, r, tag, "all_to_all");
        } catch (...) {
            first = std::current_exception();
        }
    }
    if (first) { std::rethrow_exception(first); }
}

cuda::NcclP2P *session::p2p()
{
    std::lock_guard<std::mutex> lk(*device_mu_);
    if (p2p_) { return p2p_.get(); }
    int local = 0;
    for (size_t r = 0; r < rank_; ++r) {
        if (peers_[r].ipv4 == peers_[rank_].ipv4) { ++local; }
    }
    if (const auto v = parse_env_int("STDML_COLLECTIVE_DEVICE_ID")) {
        local = static_cast<int>(*v);
    } else if (const auto l = parse_env_int("LOCAL_RANK")) {
        local = static_cast<int>(*l);
    }
    const int ndev = cuda::cuda_device_count();
    if (ndev <= 0) { throw std::runtime_error("device send/recv needs a CUDA device"); }
    // the communicator id of a pair travels as an ordinary host message
    auto exchange = [this](int peer, bool i_send, void *id, size_t size) {
        if (i_send) {
            send(id, size, u8, static_cast<size_t>(peer), "stdml::nccl::id");
        } else {
            recv(id, size, u8, static_cast<size_t>(peer), "stdml::nccl::id");
        }
    };
    p2p_ = std::make_unique<cuda::NcclP2P>(static_cast<int>(rank_), local % ndev, exchange);
    return p2p_.get();
}

std::unique_ptr<task> session::async_send(const void *input, size_t count, dtype dt, size_t target,
                                          std::string name, void *stream)
{
    if (target >= peers_.size()) { throw std::out_of_range("send: no such rank"); }
    if (count > 0 && cuda::pointer_kind(input) == 1) {
        ensure_usable("send");
        cuda::NcclP2P *p = p2p();
        p->send(input, count, static_cast<int>(dt), static_cast<int>(target), stream, nullptr);
        return std::make_unique<event_task>(p->stream());
    }
    send(input, count, dt, target, std::move(name));
    return std::make_unique<noop_task>();
}

std::unique_ptr<task> session::async_recv(void *output, size_t count, dtype dt, size_t target,
                                          std::string name, void *stream)
{
    if (target >= peers_.size()) { throw std::out_of_range("recv: no such rank"); }
    if (count > 0 && cuda::pointer_kind(output) == 1) {
        ensure_usable("recv");
        cuda::NcclP2P *p = p2p();
        p->recv(output, count, static_cast<int>(dt), static_cast<int>(target), stream, nullptr);
        return std::make_unique<event_task>(p->stream());
    }
    recv(output, count, dt, target, std::move(name));
    return std::make_unique<noop_task>();
}

void session::send(const void *input, size_t count, dtype dt, size_t target, std::string name)
{
    if (target >= peers_.size()) { throw std::out_of_range("send: no such rank"); }
    if (count > 0 && cuda::pointer_kind(input) == 1) {
        // a device address means nothing to a socket: NCCL moves it, and the call
        // returns when the GPU has sent it
        async_send(input, count, dt, target, std::move(name), nullptr)->finish();
        return;
    }
    const std::string tag = versioned(*this, "stdml::p2p::" + name);
    client_pool_->require(conn_collective)
        ->send(peers_[target], tag.c_str(), input, count * dtype_size(dt),
               message_header::wait_recv_buf);
}

void session::recv(void *output, size_t count, dtype dt, size_t target, std::string name)
{
    if (target >= peers_.size()) { throw std::out_of_range("recv: no such rank"); }
    ensure_usable("recv");
    if (count > 0 && cuda::pointer_kind(output) == 1) {
        async_recv(output, count, dt, target, std::move(name), nullptr)->finish();
        return;
    }
    const std::string tag = versioned(*this, "stdml::p2p::" + name);
    take_into(target, tag, output, count * dtype_size(dt), "recv");
}

bool session::consistent(const void *ptr, size_t size)
{
    // everyone holds the same bytes iff min == max for the length and, given
    // equal lengths, for every byte
    const uint64_t n = size;
    uint64_t lo = 0, hi = 0;
    all_reduce(&n, &lo, 1, u64, min, "stdml::consistent::len::min");
    all_reduce(&n, &hi, 1, u64, max, "stdml::consistent::len::max");
    if (lo != hi) { return false; }
    if (size == 0) { return true; }
    std::vector<uint8_t> a(size), b(size);
    all_reduce(ptr, a.data(), size, u8, min, "stdml::consistent::min");
    all_reduce(ptr, b.data(), size, u8, max, "stdml::consistent::max");
    return a == b;
}

// -------------------------------------------------------------- device path

bool session::on_device(const void *a, const void *b) const
{
    const int ka = cuda::pointer_kind(a), kb = cuda::pointer_kind(b);
    if (ka != kb) {
        throw std::invalid_argument(
            "collective: input and output must both be host or both be device memory");
    }
    return ka == 1;
}

void *session::symm_alloc(size_t bytes)
{
    cuda::DeviceWorld &w = device()->world();
    return w.ptr(w.rank(), w.alloc(bytes));
}

void session::symm_free(void *p)
{
    cuda::DeviceWorld &w = device()->world();
    const size_t off = w.offset_of(p, 0);
    if (off == SIZE_MAX) { throw std::invalid_argument("symm_free: not a symmetric buffer"); }
    w.release(off);
}

void session::device_setup_ms(double out[4]) const
{
    std::lock_guard<std::mutex> lk(*device_mu_);
    for (int i = 0; i < 4; ++i) { out[i] = 0.0; }
    if (device_) { device_->world().setup_ms(out); }
}

void session::device_set_knob(const std::string &name, long long value)
{
    device()->set_knob(name, value);
}

void session::device_drop_registrations()
{
    device()->drop_registrations();
}

unsigned long long session::device_launches() const
{
    std::lock_guard<std::mutex> lk(*device_mu_);
    return device_ ? device_->launches() : 0ull;
}

cuda::DeviceSession *session::device()
{
    // several threads of one rank may reach their first device call together
    std::lock_guard<std::mutex> lk(*device_mu_);
    if (device_) { return device_.get(); }
    if (device_tried_) { throw std::runtime_error("device collectives are unavailable"); }
    device_tried_ = true;
    cuda::DeviceWorldOptions o;
    o.rank = static_cast<int>(rank_);
    o.world = static_cast<int>(peers_.size());
    // one GPU per rank on this host: the rank's position among the peers that
    // share its address, unless STDML_COLLECTIVE_DEVICE_ID / LOCAL_RANK says otherwise
    int local = 0;
    for (size_t r = 0; r < rank_; ++r) {
        if (peers_[r].ipv4 == peers_[rank_].ipv4) { ++local; }
    }
    if (const auto v = parse_env_int("STDML_COLLECTIVE_DEVICE_ID")) {
        local = static_cast<int>(*v);
    } else if (const auto l = parse_env_int("LOCAL_RANK")) {
        local = static_cast<int>(*l);
    }
    const int ndev = cuda::cuda_device_count();
    if (ndev <= 0) { throw std::runtime_error("device collectives need a CUDA device"); }
    o.device = local % ndev;
    for (const auto &p : peers_) {
        if (p.ipv4 != peers_[0].ipv4) {
            throw std::runtime_error(
                "device collectives need all ranks on one box (one NVLink domain)");
        }
    }
    o.key = peers_[0].str() + ".v" + std::to_string(version_) + (scope_.empty() ? "" : "#" + scope_);
    if (const auto v = parse_env_int("STDML_COLLECTIVE_HEAP_MB")) {
        o.heap_bytes = static_cast<size_t>(*v) << 20;
    }
    if (const auto v = parse_env_int("STDML_COLLECTIVE_STAGING_MB")) {
        o.staging_bytes = static_cast<size_t>(*v) << 20;
    }
    o.enable_nvls = config_.use_nvls;
    o.wait_timeout_ms = static_cast<unsigned long long>(config_.timeout_ms);
    const std::string backend = safe_getenv("STDML_COLLECTIVE_SYMM");
    if (!backend.empty()) { o.backend = backend; }
    device_ = std::make_unique<cuda::DeviceSession>(cuda::DeviceWorld::create(o));
    return device_.get();
}
}  // namespace stdml::collective
