#include "device_session.hpp"

#include <algorithm>
#include <cstdlib>
#include <cstring>

#include <cuda_runtime.h>

namespace stdml::collective::cuda
{
namespace
{
constexpr size_t kElemSize[12] = {1, 2, 4, 8, 1, 2, 4, 8, 2, 2, 4, 8};

size_t elem_size(int dt)
{
    if (dt < 0 || dt >= 12) { throw std::invalid_argument("device session: bad dtype"); }
    return kElemSize[dt];
}

void rt_check(cudaError_t e, const char *what)
{
    if (e != cudaSuccess) {
        throw std::runtime_error(std::string("CUDA runtime: ") + what + ": " +
                                 cudaGetErrorString(e));
    }
}

// Inside a stream capture the two staging slots do not alternate across
// replays (a graph with an odd number of staged calls would reuse one slot back
// to back), so captured staged calls end with a barrier, which makes any reuse
// of the slot safe.
bool capturing(void *stream)
{
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(static_cast<cudaStream_t>(stream), &st) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    return st != cudaStreamCaptureStatusNone;
}

void launch_check(int rc, const char *what)
{
    if (rc != 0) {
        throw std::runtime_error(std::string("device session: launch of ") + what + " failed: " +
                                 cudaGetErrorString(static_cast<cudaError_t>(rc)));
    }
}
}  // namespace

DeviceSession::DeviceSession(std::unique_ptr<DeviceWorld> world) : world_(std::move(world))
{
    if (const char *e = std::getenv("STDML_COLLECTIVE_PIPELINE_MIN_BYTES")) {
        pipeline_min_bytes_ = static_cast<size_t>(std::atoll(e));
    }
    if (const char *e = std::getenv("STDML_COLLECTIVE_REGISTER_MIN_BYTES")) {
        const long long v = std::atoll(e);
        register_min_bytes_ = v < 0 ? SIZE_MAX : static_cast<size_t>(v);
    }
    if (const char *e = std::getenv("STDML_COLLECTIVE_PIPELINE_CHUNK_BYTES")) {
        pipeline_chunk_bytes_ = std::max<size_t>(1u << 16, static_cast<size_t>(std::atoll(e)));
    }
}

DeviceSession::~DeviceSession()
{
    (void)cudaDeviceSynchronize();
    if (pack_stream_ != nullptr) {
        (void)cudaStreamDestroy(static_cast<cudaStream_t>(pack_stream_));
        (void)cudaStreamDestroy(static_cast<cudaStream_t>(unpack_stream_));
        (void)cudaEventDestroy(static_cast<cudaEvent_t>(entry_ev_));
        for (int i = 0; i < 2; ++i) {
            (void)cudaEventDestroy(static_cast<cudaEvent_t>(packed_ev_[i]));
            (void)cudaEventDestroy(static_cast<cudaEvent_t>(reduced_ev_[i]));
            (void)cudaEventDestroy(static_cast<cudaEvent_t>(unpacked_ev_[i]));
        }
    }
    for (void *p : table_mem_) { (void)cudaFree(p); }
    table_mem_.clear();
    forget_peer_plans();
    if (order_ev_ != nullptr) { (void)cudaEventDestroy(static_cast<cudaEvent_t>(order_ev_)); }
    (void)cudaGetLastError();
}

void DeviceSession::set_knob(const std::string &name, long long value)
{
    std::lock_guard<std::recursive_mutex> lk(mu_);
    if (name == "register_min_bytes") {
        register_min_bytes_ = value < 0 ? SIZE_MAX : static_cast<size_t>(value);
        return;
    }
    if (name == "register_verify") {
        register_verify_ = value != 0;
        return;
    }
    if (name == "chunk_push_blocks") {
        chunk_push_blocks_ = static_cast<int>(std::max<long long>(1, std::min<long long>(kMaxBlocks, value)));
        return;
    }
    if (name == "chunk_unpack_blocks") {
        chunk_unpack_blocks_ = static_cast<int>(std::max<long long>(0, std::min<long long>(kMaxBlocks, value)));
        return;
    }
    if (name == "pipeline_min_bytes") {
        pipeline_min_bytes_ = value < 0 ? SIZE_MAX : static_cast<size_t>(value);
        return;
    }
    world_->set_knob(name, value);
}

void DeviceSession::drop_registrations()
{
    std::lock_guard<std::recursive_mutex> lk(mu_);
    world_->drop_registrations();  // waits for the device first
    forget_peer_plans();           // their tables hold addresses of the mappings just closed
}

void DeviceSession::forget_peer_plans()
{
    for (auto &kv : peer_plans_) {
        if (kv.second.dev != nullptr) { (void)cudaFree(kv.second.dev); }
    }
    peer_plans_.clear();
}

// Registered (zero-copy on user memory) execution applies to real multi-GPU
// worlds, outside stream capture (the handle exchange is host work), from the
// configured size up.
bool DeviceSession::registered_path(size_t bytes, void *stream) const
{
    return world_->world() > 1 && world_->vranks() == 1 && bytes >= register_min_bytes_ &&
           !capturing(stream);
}

namespace
{
bool all_aligned16(void *const *p, int n, bool allow_null = false)
{
    for (int i = 0; i < n; ++i) {
        if (p[i] == nullptr && allow_null) { continue; }
        if (p[i] == nullptr || reinterpret_cast<uintptr_t>(p[i]) % 16 != 0) { return false; }
    }
    return true;
}
}  // namespace

void DeviceSession::order_after_previous(void *stream)
{
    if (have_last_stream_ && last_stream_ != stream && !capturing(stream) &&
        !capturing(last_stream_)) {
        if (order_ev_ == nullptr) {
            cudaEvent_t e;
            rt_check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate");
            order_ev_ = e;
        }
        // the previous stream may have been destroyed by its owner since (then all of
        // its work has been submitted and completed or abandoned): nothing to wait for
        if (cudaEventRecord(static_cast<cudaEvent_t>(order_ev_),
                            static_cast<cudaStream_t>(last_stream_)) == cudaSuccess) {
            rt_check(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream),
                                         static_cast<cudaEvent_t>(order_ev_), 0),
                     "cudaStreamWaitEvent");
        } else {
            (void)cudaGetLastError();
        }
    }
    last_stream_ = stream;
    have_last_stream_ = true;
}

void DeviceSession::check()
{
    std::lock_guard<std::recursive_mutex> lk(mu_);
    const DeviceStatus s = world_->poll_status();
    if (s.code == kStatusBadArgs) {
        throw std::invalid_argument("device collective refused its launch arguments (in-kernel "
                                    "debug checks): rank " + std::to_string(s.rank) + " block " +
                                    std::to_string(s.block) + "; nothing was read or written; "
                                    "call recover() on every rank");
    }
    if (s.code != 0) {
        throw DeviceTimeout("device collective gave up: rank " + std::to_string(s.rank) +
                                " block " + std::to_string(s.block) + " waited for rank " +
                                std::to_string(s.peer) + " (barrier " + std::to_string(s.phase) +
                                ", want " + std::to_string(s.want) + ", have " +
                                std::to_string(s.have) + "); call recover() on every rank",
                            s);
    }
}

void DeviceSession::launch_ar(AllReduceCall &c, void *stream)
{
    launch_check(world_->all_reduce(c, stream), "all_reduce");
    ++launches_;
}

void DeviceSession::ensure_pipeline()
{
    if (pack_stream_ != nullptr) { return; }
    cudaStream_t a, b;
    rt_check(cudaStreamCreateWithFlags(&a, cudaStreamNonBlocking), "cudaStreamCreate");
    rt_check(cudaStreamCreateWithFlags(&b, cudaStreamNonBlocking), "cudaStreamCreate");
    pack_stream_ = a;
    unpack_stream_ = b;
    auto make = [](void *&slot) {
        cudaEvent_t e;
        rt_check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate");
        slot = e;
    };
    make(entry_ev_);
    for (int i = 0; i < 2; ++i) {
        make(packed_ev_[i]);
        make(reduced_ev_[i]);
        make(unpacked_ev_[i]);
    }
}

void DeviceSession::run_pipelined(std::vector<AllReduceCall> &calls, void *stream)
{
    ensure_pipeline();
    cudaStream_t main_s = static_cast<cudaStream_t>(stream);
    cudaStream_t pack_s = static_cast<cudaStream_t>(pack_stream_);
    cudaStream_t unpack_s = static_cast<cudaStream_t>(unpack_stream_);
    auto ev = [](void *e) { return static_cast<cudaEvent_t>(e); };
    // the inputs are ready when the caller's stream gets here
    rt_check(cudaEventRecord(ev(entry_ev_), main_s), "cudaEventRecord");
    rt_check(cudaStreamWaitEvent(pack_s, ev(entry_ev_), 0), "cudaStreamWaitEvent");
    bool used[2] = {false, false};
    for (AllReduceCall &c : calls) {
        c.off = world_->next_staging_slot();
        const int slot = static_cast<int>((c.off - kDataOffset) / world_->staging_bytes()) & 1;
        // the slot is free once the chunk that used it before has been unpacked
        if (used[slot]) {
            rt_check(cudaStreamWaitEvent(pack_s, ev(unpacked_ev_[slot]), 0), "cudaStreamWaitEvent");
        }
        AllReduceCall pack = c;
        pack.phases = kPhasePack;
        launch_ar(pack, pack_s);
        rt_check(cudaEventRecord(ev(packed_ev_[slot]), pack_s), "cudaEventRecord");

        rt_check(cudaStreamWaitEvent(main_s, ev(packed_ev_[slot]), 0), "cudaStreamWaitEvent");
        AllReduceCall red = c;
        red.phases = kPhaseReduce;
        // leave SMs to the copy phases of the neighbouring chunks
        const size_t esz = kElemSize[c.dt];
        red.blocks = std::min(64, world_->pick_blocks((c.count * esz + 15) / 16, c.algo));
        launch_ar(red, main_s);
        rt_check(cudaEventRecord(ev(reduced_ev_[slot]), main_s), "cudaEventRecord");

        rt_check(cudaStreamWaitEvent(unpack_s, ev(reduced_ev_[slot]), 0), "cudaStreamWaitEvent");
        AllReduceCall unpack = c;
        unpack.phases = kPhaseUnpack;
        launch_ar(unpack, unpack_s);
        rt_check(cudaEventRecord(ev(unpacked_ev_[slot]), unpack_s), "cudaEventRecord");
        used[slot] = true;
    }
    for (int i = 0; i < 2; ++i) {
        if (used[i]) {
            rt_check(cudaStreamWaitEvent(main_s, ev(unpacked_ev_[i]), 0), "cudaStreamWaitEvent");
        }
    }
    // The unpack ran outside the kernels that carry the barriers, so "a peer has
    // passed the barrier of my next call" no longer implies "it is done with its
    // slots": line the ranks up once, after which the slots are free everywhere.
    launch_check(world_->barrier(stream), "barrier (end of pipeline)");
    ++launches_;
}

void DeviceSession::all_reduce(const void *const *in, void *const *out, size_t count, int dt,
                               int op, double scale, int algo, void *stream)
{
    std::lock_guard<std::recursive_mutex> lk(mu_);
    check();
    order_after_previous(stream);
    if (count == 0) { return; }
    const size_t es = elem_size(dt);
    const int vr = world_->vranks();
    AllReduceCall c;
    c.dt = dt;
    c.op = op;
    c.algo = algo;
    c.has_scale = scale != 1.0;
    c.scale = scale;

    // zero-copy: the buffer lives at the same arena offset on every rank
    size_t off = world_->offset_of(in[0], 0);
    bool symmetric = off != SIZE_MAX && off % 16 == 0;
    bool in_place = true;
    for (int v = 0; v < vr && symmetric; ++v) {
        symmetric = world_->offset_of(in[v], v) == off;
        in_place = in_place && (in[v] == out[v]);
    }
    if (symmetric && in_place) {
        c.off = off;
        c.count = count;
        if (c.algo == kAlgoOneShot || c.algo == kAlgoNvlsOneShot) {
            throw std::invalid_argument(
                "all_reduce: one-shot algorithms cannot run in place on a symmetric buffer");
        }
        if (c.algo < 0) { c.algo = world_->pick_algo(count * es, dt, op, true); }
        launch_ar(c, stream);
        return;
    }
    int zc_algo = algo < 0 ? world_->pick_algo(count * es, dt, op, false) : algo;
    if (symmetric && (zc_algo == kAlgoOneShot || zc_algo == kAlgoNvlsOneShot)) {
        // read the symmetric input in place, write the user's output; the end
        // barrier keeps the input stable until every peer has read it
        c.off = off;
        c.count = count;
        c.dst = out;
        c.end_barrier = true;
        c.algo = zc_algo;
        launch_ar(c, stream);
        return;
    }

    // registered: ordinary device buffers whose allocations every peer has mapped;
    // the owners pull the operands from the inputs and store the results into the
    // outputs, nothing is packed or unpacked
    if (!symmetric && registered_path(count * es, stream) && (algo < 0 || is_owner_algo(algo))) {
        const int world = world_->world();
        void *p_out[kMaxRanks], *p_in[kMaxRanks];
        const bool same = in[0] == out[0];
        bool ok = world_->resolve_peers(out, count * es, p_out) && all_aligned16(p_out, world);
        if (ok && !same) {
            ok = world_->resolve_peers(in, count * es, p_in) && all_aligned16(p_in, world);
        }
        if (ok) {
            c.peer_data = same ? p_out : p_in;
            c.peer_push = same ? nullptr : p_out;
            c.count = count;
            c.algo = algo >= 0 ? algo : world_->pick_algo(count * es, dt, op, true);
            if (c.algo == kAlgoNvls) {  // the multicast mapping covers the arena only
                c.algo = world_->pick_peer_algo(count * es);
            }
            launch_ar(c, stream);
            return;
        }
    }

    // staged: pack into a staging slot inside the launch, one slot per chunk
    const bool in_capture = capturing(stream);
    size_t slot_elems = world_->staging_bytes() / 16 * (16 / es);
    const size_t total_bytes = count * es;
    if (world_->world() > 1 && total_bytes >= pipeline_min_bytes_ && !in_capture &&
        (algo < 0 || is_owner_algo(algo))) {
        // large message: chunks of about 1/8 of it (8 MB at least, a slot at most)
        const size_t lanes = 16 / es;
        size_t chunk = std::max<size_t>(pipeline_chunk_bytes_ / es,
                                        (count / 8 + lanes - 1) / lanes * lanes);
        chunk = std::min(chunk, slot_elems);
        const int owner = algo >= 0 ? algo : world_->pick_algo(chunk * es, dt, op, true);
        std::vector<std::vector<const void *>> srcs;
        std::vector<std::vector<void *>> dsts;
        std::vector<AllReduceCall> calls;
        for (size_t done = 0; done < count; done += chunk) {
            srcs.emplace_back(vr);
            dsts.emplace_back(vr);
            for (int v = 0; v < vr; ++v) {
                srcs.back()[v] = static_cast<const char *>(in[v]) + done * es;
                dsts.back()[v] = static_cast<char *>(out[v]) + done * es;
            }
            AllReduceCall k = c;
            k.count = std::min(chunk, count - done);
            k.algo = owner;
            calls.push_back(k);
        }
        for (size_t i = 0; i < calls.size(); ++i) {
            calls[i].src = srcs[i].data();
            calls[i].dst = dsts[i].data();
        }
        run_pipelined(calls, stream);
        return;
    }
    std::vector<const void *> src(vr);
    std::vector<void *> dst(vr);
    for (size_t done = 0; done < count; done += slot_elems) {
        const size_t n = std::min(slot_elems, count - done);
        for (int v = 0; v < vr; ++v) {
            src[v] = static_cast<const char *>(in[v]) + done * es;
            dst[v] = static_cast<char *>(out[v]) + done * es;
        }
        AllReduceCall k = c;
        k.off = world_->next_staging_slot();
        k.src = src.data();
        k.dst = dst.data();
        k.count = n;
        k.end_barrier = in_capture;
        launch_ar(k, stream);
    }
}

void DeviceSession::reduce(const void *const *in, void *const *out, size_t count, int dt, int op,
                           int root, double scale, void *stream)
{
    std::lock_guard<std::recursive_mutex> lk(mu_);
    check();
    order_after_previous(stream);
    if (count == 0) { return; }
    if (root < 0 || root >= world_->world()) { throw std::invalid_argument("reduce: bad root"); }
    const size_t es = elem_size(dt);
    const int vr = world_->vranks();
    // zero-copy: the inputs live in the symmetric heap; root alone reads them (the
    // switch reduces on the way when it can, else root loads every peer), nothing
    // is packed.  Without the switch only small messages go this way: root's
    // links would carry n-1 copies.
    const size_t in_off = symmetric_offset(in);
    const bool by_switch = world_->has_nvls() && nvls_supported(dt, op) && world_->world() > 2;
    if (in_off != SIZE_MAX && world_->world() > 1 && (by_switch || count * es <= (1u << 20))) {
        std::vector<void *> dsts(vr);
        const size_t slot_elems = world_->staging_bytes() / 16 * (16 / es);
        const bool small = count * es <= (1u << 20);
        // several slots: root copies chunk k out of its slot on a second stream while
        // the owners already reduce chunk k + 1 into the other slot
        const bool overlap = !small && count > slot_elems && vr == 1 && !capturing(stream);
        const bool i_am_root = world_->rank() == root;
        cudaStream_t main_s = static_cast<cudaStream_t>(stream);
        cudaStream_t unpack_s = nullptr;
        auto ev = [](void *e) { return static_cast<cudaEvent_t>(e); };
        bool used[2] = {false, false};
        if (overlap) {
            ensure_pipeline();
            unpack_s = static_cast<cudaStream_t>(unpack_stream_);
        }
        for (size_t done = 0; done < count; done += small ? count : slot_elems) {
            const size_t n = small ? count : std::min(slot_elems, count - done);
            for (int v = 0; v < vr; ++v) {
                dsts[v] = (out != nullptr && out[v] != nullptr)
                              ? static_cast<char *>(out[v]) + done * es
                              : nullptr;
            }
            AllReduceCall k;
            k.dt = dt;
            k.op = op;
            k.root = root;
            k.has_scale = scale != 1.0;
            k.scale = scale;
            k.off = in_off + done * es;
            k.dst = dsts.data();
            k.count = n;
            if (small) {
                // root alone reads everything (through the switch when it can)
                k.end_barrier = true;  // the inputs stay untouched until root has read them
                k.algo = by_switch ? kAlgoNvlsOneShot : kAlgoOneShot;
                launch_ar(k, stream);
                continue;
            }
            // every rank has the switch reduce its shard and stores it into root's
            // staging slot, from where root copies it out: one GPU alone cannot
            // draw the switch's full rate, eight together can
            k.algo = kAlgoNvls;
            k.push_off = world_->next_staging_slot();
            if (!overlap) {
                launch_ar(k, stream);
                continue;
            }
            const int slot =
                static_cast<int>((k.push_off - kDataOffset) / world_->staging_bytes()) & 1;
            if (used[slot]) {
                rt_check(cudaStreamWaitEvent(main_s, ev(unpacked_ev_[slot]), 0), "cudaStreamWaitEvent");
            }
            void *root_dst = dsts[0];
            dsts[0] = nullptr;  // copied out below, beside the next chunk
            launch_ar(k, stream);
            rt_check(cudaEventRecord(ev(reduced_ev_[slot]), main_s), "cudaEventRecord");
            rt_check(cudaStreamWaitEvent(unpack_s, ev(reduced_ev_[slot]), 0), "cudaStreamWaitEvent");
            if (i_am_root && root_dst != nullptr) {
                launch_check(world_->unpack_blocks(world_->ptr(world_->rank(), k.push_off), root_dst,
                                                   n * es, 0, 0, 1, unpack_s),
                             "unpack (reduce chunk)");
                ++launches_;
            }
            rt_check(cudaEventRecord(ev(unpacked_ev_[slot]), unpack_s), "cudaEventRecord");
            used[slot] = true;
        }
        if (overlap) {
            for (int i = 0; i < 2; ++i) {
                if (used[i]) {
                    rt_check(cudaStreamWaitEvent(main_s, ev(unpacked_ev_[i]), 0), "cudaStreamWaitEvent");
                }
            }
            launch_check(world_->barrier(stream), "barrier (end of pipeline)");
            ++launches_;
        }
        return;
    }
    if (registered_path(count * es, stream)) {
        // owners pull their shard from every rank's input and store the result
        // into root's output: root's links carry one copy of the message
        const int world = world_->world();
        void *p_in[kMaxRanks], *p_out[kMaxRanks];
        const void *mine_out[1] = {(world_->rank() == root && out != nullptr) ? out[0] : nullptr};
        if (world_->rank() == root && mine_out[0] == nullptr) {
            throw std::invalid_argument("reduce: root needs an output buffer");
        }
        const bool ok = world_->resolve_peers(in, count * es, p_in) && all_aligned16(p_in, world) &&
                        world_->resolve_peers(mine_out, count * es, p_out) &&
                        p_out[root] != nullptr &&
                        reinterpret_cast<uintptr_t>(p_out[root]) % 16 == 0;
        if (ok) {
            for (int r = 0; r < world; ++r) {
                if (r != root) { p_out[r] = p_in[r]; }  // never written: only [root] is used
            }
            AllReduceCall k;
            k.dt = dt;
            k.op = op;
            k.root = root;
            k.has_scale = scale != 1.0;
            k.scale = scale;
            k.peer_data = p_in;
            k.peer_push = p_out;
            k.count = count;
            k.algo = world_->pick_peer_algo(count * es);
            launch_ar(k, stream);
            return;
        }
    }
    const size_t slot_elems = world_->staging_bytes() / 16 * (16 / es);
    const bool in_capture = capturing(stream);
    std::vector<std::vector<const void *>> srcs;
    std::vector<std::vector<void *>> dsts;
    std::vector<AllReduceCall> calls;
    for (size_t done = 0; done < count; done += slot_elems) {
        const size_t n = std::min(slot_elems, count - done);
        srcs.emplace_back(vr);
        dsts.emplace_back(vr);
        for (int v = 0; v < vr; ++v) {
            srcs.back()[v] = static_cast<const char *>(in[v]) + done * es;
            dsts.back()[v] = (out != nullptr && out[v] != nullptr)
                                 ? static_cast<char *>(out[v]) + done * es
                                 : nullptr;
        }
        AllReduceCall k;
        k.dt = dt;
        k.op = op;
        k.root = root;
        k.has_scale = scale != 1.0;
        k.scale = scale;
        k.count = n;
        k.end_barrier = in_capture;
        // small (or two ranks): root pulls everything; large: owners reduce their
        // shard (through the switch where it can) and store it to root only, which
        // spreads the reads over all links
        if (n * es <= (1u << 20) || world_->world() <= 2) {
            k.algo = kAlgoOneShot;
        } else if (world_->has_nvls() && nvls_supported(dt, op)) {
            // (measured: one GPU pulling everything through the switch stops near 370 GB/s)
            k.algo = kAlgoNvls;
        } else {
            k.algo = kAlgoTwoShot;
        }
        calls.push_back(k);
    }
    for (size_t i = 0; i < calls.size(); ++i) {
        calls[i].src = srcs[i].data();
        calls[i].dst = dsts[i].data();
    }
    if (calls.size() >= 2 && world_->world() > 2 && vr == 1 && !in_capture) {
        run_pipelined(calls, stream);  // pack / reduce / unpack of neighbouring chunks overlap
        return;
    }
    for (AllReduceCall &k : calls) {
        k.off = world_->next_staging_slot();
        launch_ar(k, stream);
    }
}

std::vector<std::vector<GroupPiece>> plan_group_pieces(size_t n, const size_t *counts,
                                                       size_t lanes, size_t cap)
{
    std::vector<std::vector<GroupPiece>> chunks(1);
    size_t fill = 0;
    for (size_t i = 0; i < n; ++i) {
        size_t done = 0;
        while (done < counts[i]) {
            if (fill == cap) {
                chunks.emplace_back();
                fill = 0;
            }
            const size_t room = (cap - fill) * lanes;
            const size_t take = std::min(room, counts[i] - done);
            chunks.back().push_back(GroupPiece{i, done, take, fill});
            fill += (take + lanes - 1) / lanes;
            done += take;
        }
    }
    return chunks;
}

const DeviceSession::GroupPlan &DeviceSession::plan_group(size_t n, const void *const *ins,
                                                          void *const *outs,
                                                          const size_t *counts, int dt,
                                                          int user_dt)
{
    const int vr = world_->vranks();
    std::string key;
    key.reserve((2 * vr * n + n + 2) * sizeof(void *));
    key.append(reinterpret_cast<const char *>(ins), sizeof(void *) * n * vr);
    key.append(reinterpret_cast<const char *>(outs), sizeof(void *) * n * vr);
    key.append(reinterpret_cast<const char *>(counts), sizeof(size_t) * n);
    key.append(reinterpret_cast<const char *>(&dt), sizeof(dt));
    key.append(reinterpret_cast<const char *>(&user_dt), sizeof(user_dt));
    auto it = plans_.find(key);
    if (it != plans_.end()) { return it->second; }
    if (plans_.size() >= 64) {  // bounded cache; cudaFree waits for work in flight
        for (void *p : table_mem_) { (void)cudaFree(p); }
        table_mem_.clear();
        plans_.clear();
    }

    const size_t es = elem_size(dt);                          // wire element
    const size_t ues = user_dt >= 0 ? elem_size(user_dt) : es;  // user element
    const size_t lanes = 16 / es;
    // One chunk per staging slot.  (Cutting a pipelined set finer, 1/8 of it per
    // chunk, was measured slower at 8 GPUs: 605 against 671 GB/s on 438 MB.)
    const size_t cap = world_->staging_bytes() / 16;  // vectors per slot

    using Piece = GroupPiece;
    const std::vector<std::vector<Piece>> chunks = plan_group_pieces(n, counts, lanes, cap);

    GroupPlan plan;
    for (const auto &pieces : chunks) {
        if (pieces.empty()) { continue; }
        std::vector<Table> per_rank(vr);
        size_t nvec = 0;
        for (const auto &p : pieces) { nvec = std::max(nvec, p.voff + (p.count + lanes - 1) / lanes); }
        for (int v = 0; v < vr; ++v) {
            std::vector<GroupEntry> host(pieces.size());
            for (size_t j = 0; j < pieces.size(); ++j) {
                const Piece &p = pieces[j];
                const char *s = static_cast<const char *>(ins[v * n + p.tensor]);
                char *d = static_cast<char *>(outs[v * n + p.tensor]);
                host[j].src = s + p.first_elem * ues;
                host[j].dst = d + p.first_elem * ues;
                host[j].voff = p.voff;
                host[j].count = p.count;
            }
            void *dev = nullptr;
            rt_check(cudaMalloc(&dev, host.size() * sizeof(GroupEntry)), "cudaMalloc(table)");
            table_mem_.push_back(dev);
            rt_check(cudaMemcpy(dev, host.data(), host.size() * sizeof(GroupEntry),
                                cudaMemcpyHostToDevice),
                     "cudaMemcpy(table)");
            per_rank[v].dev = static_cast<GroupEntry *>(dev);
            per_rank[v].n = static_cast<int>(host.size());
            per_rank[v].nvec = nvec;
        }
        plan.chunks.push_back(std::move(per_rank));
    }
    return plans_.emplace(std::move(key), std::move(plan)).first->second;
}

bool DeviceSession::group_registered(size_t n, const void *const *ins, void *const *outs,
                                     const size_t *counts, int dt, int op, double scale,
                                     void *stream)
{
    const int world = world_->world();
    const int vr = world_->vranks();
    const size_t es = elem_size(dt);
    const size_t lanes = 16 / es;
    // the key: this rank's pointers and sizes, and the allocations behind them (an
    // allocation freed and made again at the same address has another id)
    std::string key;
    key.reserve((4 * vr * n + n + 1) * sizeof(void *));
    key.append(reinterpret_cast<const char *>(ins), sizeof(void *) * n * vr);
    key.append(reinterpret_cast<const char *>(outs), sizeof(void *) * n * vr);
    key.append(reinterpret_cast<const char *>(counts), sizeof(size_t) * n);
    key.append(reinterpret_cast<const char *>(&dt), sizeof(dt));
    for (size_t k = 0; register_verify_ && k < n * static_cast<size_t>(vr); ++k) {
        const unsigned long long a = world_->buffer_id(ins[k]);
        const unsigned long long b = outs[k] == ins[k] ? a : world_->buffer_id(outs[k]);
        key.append(reinterpret_cast<const char *>(&a), sizeof(a));
        key.append(reinterpret_cast<const char *>(&b), sizeof(b));
    }
    auto it = peer_plans_.find(key);
    const bool reuse = world_->all_same(it != peer_plans_.end() ? it->second.stamp : 0ull);
    if (!reuse) {
        // some rank has a new set (or a new allocation under an old one): all build
        if (it != peer_plans_.end()) {
            if (it->second.dev != nullptr) { (void)cudaFree(it->second.dev); }
            peer_plans_.erase(it);
        }
        if (peer_plans_.size() >= 64) { forget_peer_plans(); }  // bounded; cudaFree waits for work in flight
        PeerPlan plan;
        plan.stamp = ++peer_plan_builds_;
        std::vector<size_t> bytes(n);
        for (size_t i = 0; i < n; ++i) { bytes[i] = counts[i] * es; }
        std::vector<void *> p_in(n * world), p_out(n * world);
        bool same = true;
        for (size_t k = 0; k < n * static_cast<size_t>(vr) && same; ++k) { same = ins[k] == outs[k]; }
        // (a rank whose outputs are its inputs still joins both exchanges when another
        // rank's are not: the number of exchanges must not depend on local facts)
        same = world_->all_same(same ? 1ull : 2ull) && same;
        bool ok = world_->resolve_many(n, ins, bytes.data(), p_in.data()) &&
                  all_aligned16(p_in.data(), static_cast<int>(n) * world);
        if (ok && !same) {
            ok = world_->resolve_many(n, reinterpret_cast<const void *const *>(outs), bytes.data(),
                                      p_out.data()) &&
                 all_aligned16(p_out.data(), static_cast<int>(n) * world);
        }
        ok = world_->all_same(ok ? 1ull : 2ull) && ok;
        if (ok) {
            std::vector<PeerEntry> host(n);
            size_t voff = 0;
            for (size_t i = 0; i < n; ++i) {
                std::memset(&host[i], 0, sizeof(PeerEntry));
                for (int r = 0; r < world; ++r) {
                    host[i].in[r] = static_cast<char *>(p_in[i * world + r]);
                    host[i].out[r] = static_cast<char *>(same ? p_in[i * world + r] : p_out[i * world + r]);
                }
                host[i].voff = voff;
                host[i].count = counts[i];
                voff += (counts[i] + lanes - 1) / lanes;
            }
            // empty tensors would break the search for an entry by its first vector
            host.erase(std::remove_if(host.begin(), host.end(),
                                      [](const PeerEntry &e) { return e.count == 0; }),
                       host.end());
            plan.nvec = voff;
            plan.n = static_cast<int>(host.size());
            if (!host.empty()) {
                void *dev = nullptr;
                rt_check(cudaMalloc(&dev, host.size() * sizeof(PeerEntry)), "cudaMalloc(table)");
                if (cudaMemcpy(dev, host.data(), host.size() * sizeof(PeerEntry),
                               cudaMemcpyHostToDevice) != cudaSuccess) {
                    (void)cudaFree(dev);
                    rt_check(cudaGetLastError(), "cudaMemcpy(table)");
                    throw std::runtime_error("group_all_reduce: cannot upload the table of peer pointers");
                }
                plan.dev = static_cast<PeerEntry *>(dev);
            } else {
                return true;  // nothing to reduce
            }
        }
        it = peer_plans_.emplace(std::move(key), plan).first;
    }
    const PeerPlan &plan = it->second;
    if (plan.dev == nullptr) { return false; }
    launch_check(world_->group_peer(plan.dev, plan.n, plan.nvec, dt, op, scale, stream),
                 "group_all_reduce(registered)");
    ++launches_;
    return true;
}

void DeviceSession::group_all_reduce(size_t n, const void *const *ins, void *const *outs,
                                     const size_t *counts, int dt, int op, int user_dt,
                                     double scale, int algo, void *stream)
{
    std::lock_guard<std::recursive_mutex> lk(mu_);
    check();
    order_after_previous(stream);
    if (n == 0) { return; }
    const size_t es = elem_size(dt);
    const int vr = world_->vranks();
    if (user_dt == dt) { user_dt = -1; }

    // zero-copy: tensors sit back to back (16-byte granules) at the same arena
    // offsets on every rank and are reduced in place -> one flat all_reduce
    bool flat = user_dt < 0;
    size_t first = SIZE_MAX, total = 0;
    for (int v = 0; v < vr && flat; ++v) {
        size_t expect = SIZE_MAX;
        for (size_t i = 0; i < n && flat; ++i) {
            const size_t off = world_->offset_of(ins[v * n + i], v);
            flat = off != SIZE_MAX && off % 16 == 0 && ins[v * n + i] == outs[v * n + i] &&
                   (expect == SIZE_MAX || off == expect);
            if (i == 0) {
                if (v == 0) { first = off; }
                flat = flat && off == first;
            }
            expect = off + (counts[i] * es + 15) / 16 * 16;
        }
        if (flat) { total = expect - first; }
    }
    if (flat && total > 0) {
        AllReduceCall c;
        c.dt = dt;
        c.op = op;
        c.off = first;
        c.count = total / es;
        c.has_scale = scale != 1.0;
        c.scale = scale;
        c.algo = algo;
        if (c.algo == kAlgoOneShot || c.algo == kAlgoNvlsOneShot) { c.algo = -1; }
        if (c.algo < 0) { c.algo = world_->pick_algo(total, dt, op, true); }
        launch_ar(c, stream);
        return;
    }

    if (user_dt < 0 && (algo < 0 || algo == kAlgoTwoShot)) {
        size_t bytes = 0;
        for (size_t i = 0; i < n; ++i) { bytes += counts[i] * es; }
        // (a loopback world runs it too: there every "peer" pointer is a local one)
        if (world_->world() > 1 && bytes >= register_min_bytes_ && !capturing(stream) &&
            group_registered(n, ins, outs, counts, dt, op, scale, stream)) {
            return;
        }
    }

    const GroupPlan &plan = plan_group(n, ins, outs, counts, dt, user_dt);
    size_t plan_bytes = 0;
    for (const auto &chunk : plan.chunks) { plan_bytes += chunk[0].nvec * 16; }
    if (world_->world() > 1 && plan.chunks.size() >= 2 && plan_bytes >= pipeline_min_bytes_ &&
        !capturing(stream) && (algo < 0 || is_owner_algo(algo))) {
        std::vector<std::vector<const GroupEntry *>> all_tabs;
        std::vector<AllReduceCall> calls;
        for (const auto &chunk : plan.chunks) {
            all_tabs.emplace_back(vr);
            for (int v = 0; v < vr; ++v) { all_tabs.back()[v] = chunk[v].dev; }
            AllReduceCall c;
            c.dt = dt;
            c.op = op;
            c.user_dtype = user_dt;
            c.ntable = chunk[0].n;
            c.count = chunk[0].nvec * (16 / es);
            c.has_scale = scale != 1.0;
            c.scale = scale;
            c.algo = algo >= 0 ? algo : world_->pick_algo(chunk[0].nvec * 16, dt, op, true);
            calls.push_back(c);
        }
        for (size_t i = 0; i < calls.size(); ++i) { calls[i].table = all_tabs[i].data(); }
        run_pipelined(calls, stream);
        return;
    }
    std::vector<const GroupEntry *> tabs(vr);
    for (const auto &chunk : plan.chunks) {
        for (int v = 0; v < vr; ++v) { tabs[v] = chunk[v].dev; }
        AllReduceCall c;
        c.dt = dt;
        c.op = op;
        c.user_dtype = user_dt;
        c.off = world_->next_staging_slot();
        c.table = tabs.data();
        c.ntable = chunk[0].n;
        c.count = chunk[0].nvec * (16 / es);
        c.has_scale = scale != 1.0;
        c.scale = scale;
        c.algo = algo;
        c.end_barrier = capturing(stream);
        launch_ar(c, stream);
    }
}

// Same arena offset on every virtual rank, 16-byte aligned: the buffer can be
// addressed on every peer without any copy.
size_t DeviceSession::symmetric_offset(const void *const *ptrs) const
{
    const int vr = world_->vranks();
    if (ptrs == nullptr || ptrs[0] == nullptr) { return SIZE_MAX; }
    const size_t off = world_->offset_of(ptrs[0], 0);
    if (off == SIZE_MAX || off % 16 != 0) { return SIZE_MAX; }
    for (int v = 1; v < vr; ++v) {
        if (ptrs[v] == nullptr || world_->offset_of(ptrs[v], v) != off) { return SIZE_MAX; }
    }
    return off;
}

// Runs the chunks of a staged all_gather / broadcast with their local unpack on
// a second stream: while chunk k is copied out of its slot, chunk k+1 is on the
// links.  A chunk's push may start only when every rank has unpacked the chunk
// that used the slot before, hence the start barrier from the third chunk on
// (each rank's launch already waits for its own unpack).
void DeviceSession::run_gather_chunks(std::vector<GatherCall> &calls,
                                      const std::vector<std::vector<void *>> &dsts,
                                      int blocks_n, size_t stride, void *stream)
{
    ensure_pipeline();
    cudaStream_t main_s = static_cast<cudaStream_t>(stream);
    cudaStream_t unpack_s = static_cast<cudaStream_t>(unpack_stream_);
    auto ev = [](void *e) { return static_cast<cudaEvent_t>(e); };
    const int rank = world_->rank();
    bool used[2] = {false, false};
    for (size_t k = 0; k < calls.size(); ++k) {
        GatherCall &g = calls[k];
        g.off = world_->next_staging_slot();
        const int slot = static_cast<int>((g.off - kDataOffset) / world_->staging_bytes()) & 1;
        if (used[slot]) {
            rt_check(cudaStreamWaitEvent(main_s, ev(unpacked_ev_[slot]), 0), "cudaStreamWaitEvent");
            g.start_barrier = true;
        }
        g.dst = nullptr;  // unpacked by the copy kernel below
        // posted stores fill the links from few SMs; the rest belong to the unpack
        // of the previous chunk, which runs at the same time
        if (g.blocks <= 0) { g.blocks = chunk_push_blocks_; }
        launch_check(world_->gather(g, stream), "gather (chunk)");
        ++launches_;
        rt_check(cudaEventRecord(ev(reduced_ev_[slot]), main_s), "cudaEventRecord");
        rt_check(cudaStreamWaitEvent(unpack_s, ev(reduced_ev_[slot]), 0), "cudaStreamWaitEvent");
        launch_check(world_->unpack_blocks(world_->ptr(rank, g.off), dsts[k][0], g.bytes,
                                           g.sym_stride, stride, blocks_n, unpack_s,
                                           chunk_unpack_blocks_),
                     "unpack (chunk)");
        ++launches_;
        rt_check(cudaEventRecord(ev(unpacked_ev_[slot]), unpack_s), "cudaEventRecord");
        used[slot] = true;
    }
    for (int i = 0; i < 2; ++i) {
        if (used[i]) {
            rt_check(cudaStreamWaitEvent(main_s, ev(unpacked_ev_[i]), 0), "cudaStreamWaitEvent");
        }
    }
    // as at the end of run_pipelined: no rank may push into a slot that its owner
    // is still unpacking
    launch_check(world_->barrier(stream), "barrier (end of pipeline)");
    ++launches_;
}

void DeviceSession::all_gather(const void *const *in, void *const *out, size_t count, int dt,
                               void *stream)
{
    std::lock_guard<std::recursive_mutex> lk(mu_);
    check();
    order_after_previous(stream);
    const size_t bytes = count * elem_size(dt);
    if (bytes == 0) { return; }
    const int vr = world_->vranks();
    const int world = world_->world();

    // zero-copy: the output lives in the symmetric heap and blocks start on
    // 16-byte boundaries; every rank stores its block straight into every output
    const size_t out_off = symmetric_offset(out);
    if (out_off != SIZE_MAX && bytes % 16 == 0 && world > 1) {
        std::vector<const void *> src(vr);
        for (int v = 0; v < vr; ++v) {
            const char *own = static_cast<const char *>(out[v]) +
                              static_cast<size_t>(world_->rank() + v) * bytes;
            src[v] = (in[v] == own) ? nullptr : in[v];  // already in place
        }
        GatherCall g;
        g.off = out_off;
        g.src = src.data();
        g.bytes = bytes;
        g.sym_stride = bytes;
        g.start_barrier = true;  // peers write into memory this rank may still be reading
        g.algo = kGatherPush;
        launch_check(world_->gather(g, stream), "all_gather");
        ++launches_;
        return;
    }

    if (bytes % 16 == 0 && registered_path(bytes * static_cast<size_t>(world), stream)) {
        void *p_out[kMaxRanks];
        if (world_->resolve_peers(out, bytes * static_cast<size_t>(world), p_out) &&
            all_aligned16(p_out, world)) {
            const char *own = static_cast<const char *>(out[0]) +
                              static_cast<size_t>(world_->rank()) * bytes;
            const void *src[1] = {in[0] == own ? nullptr : in[0]};
            GatherCall g;
            g.peer_data = p_out;
            g.src = src;
            g.bytes = bytes;
            g.sym_stride = bytes;
            g.start_barrier = true;
            g.algo = kGatherPush;
            launch_check(world_->gather(g, stream), "all_gather");
            ++launches_;
            return;
        }
    }

    // staged: a slot holds one block of every rank
    const bool in_capture = capturing(stream);
    const size_t slot = world_->staging_bytes();
    const size_t chunk = std::max<size_t>(16, slot / static_cast<size_t>(world) / 16 * 16);
    std::vector<GatherCall> calls;
    std::vector<std::vector<const void *>> srcs;
    std::vector<std::vector<void *>> dsts;
    for (size_t done = 0; done < bytes; done += chunk) {
        srcs.emplace_back(vr);
        dsts.emplace_back(vr);
        for (int v = 0; v < vr; ++v) {
            srcs.back()[v] = static_cast<const char *>(in[v]) + done;
            dsts.back()[v] = static_cast<char *>(out[v]) + done;
        }
        GatherCall g;
        g.bytes = std::min(chunk, bytes - done);
        g.sym_stride = (g.bytes + 15) / 16 * 16;
        g.stride = bytes;
        g.end_barrier = in_capture;
        calls.push_back(g);
    }
    for (size_t k = 0; k < calls.size(); ++k) {
        calls[k].src = srcs[k].data();
        calls[k].dst = dsts[k].data();
    }
    if (calls.size() >= 2 && vr == 1 && world > 1 && !in_capture) {
        run_gather_chunks(calls, dsts, world, bytes, stream);
        return;
    }
    for (GatherCall &g : calls) {
        g.off = world_->next_staging_slot();
        launch_check(world_->gather(g, stream), "all_gather");
        ++launches_;
    }
}

void DeviceSession::broadcast(const void *const *in, void *const *out, size_t count, int dt,
                              int root, void *stream)
{
    std::lock_guard<std::recursive_mutex> lk(mu_);
    check();
    order_after_previous(stream);
    if (root < 0 || root >= world_->world()) { throw std::invalid_argument("broadcast: bad root"); }
    const size_t bytes = count * elem_size(dt);
    if (bytes == 0) { return; }
    const int vr = world_->vranks();
    const int world = world_->world();

    // zero-copy: the destination lives in the symmetric heap; root stores into it
    // on every rank (one multimem.st pass with NVLS)
    const size_t out_off = symmetric_offset(out);
    if (out_off != SIZE_MAX && world > 1) {
        std::vector<const void *> src(vr);
        for (int v = 0; v < vr; ++v) {
            const bool has_in = in != nullptr && in[v] != nullptr;
            src[v] = (!has_in || in[v] == out[v]) ? nullptr : in[v];
        }
        GatherCall g;
        g.off = out_off;
        g.src = src.data();
        g.bytes = bytes;
        g.root = root;
        g.start_barrier = true;
        if (bytes < (256u << 10)) { g.algo = kGatherPush; }  // small: root stores to every peer
        launch_check(world_->gather(g, stream), "broadcast");
        ++launches_;
        return;
    }

    if (registered_path(bytes, stream)) {
        void *p_out[kMaxRanks];
        if (world_->resolve_peers(out, bytes, p_out) && all_aligned16(p_out, world)) {
            const bool has_in = in != nullptr && in[0] != nullptr;
            const void *src[1] = {(!has_in || in[0] == out[0]) ? nullptr : in[0]};
            GatherCall g;
            g.peer_data = p_out;
            g.src = src;
            g.bytes = bytes;
            g.root = root;
            g.start_barrier = true;
            launch_check(world_->gather(g, stream), "broadcast");
            ++launches_;
            return;
        }
    }

    const bool in_capture = capturing(stream);
    const size_t slot = world_->staging_bytes();
    std::vector<GatherCall> calls;
    std::vector<std::vector<const void *>> srcs;
    std::vector<std::vector<void *>> dsts;
    for (size_t done = 0; done < bytes; done += slot) {
        srcs.emplace_back(vr);
        dsts.emplace_back(vr);
        for (int v = 0; v < vr; ++v) {
            srcs.back()[v] = (in != nullptr && in[v] != nullptr)
                                 ? static_cast<const char *>(in[v]) + done
                                 : nullptr;
            dsts.back()[v] = static_cast<char *>(out[v]) + done;
        }
        GatherCall g;
        g.bytes = std::min(slot, bytes - done);
        g.root = root;
        g.end_barrier = in_capture;
        calls.push_back(g);
    }
    for (size_t k = 0; k < calls.size(); ++k) {
        calls[k].src = srcs[k].data();
        calls[k].dst = dsts[k].data();
    }
    if (calls.size() >= 2 && vr == 1 && world > 1 && !in_capture) {
        run_gather_chunks(calls, dsts, 1, 0, stream);
        return;
    }
    for (GatherCall &g : calls) {
        g.off = world_->next_staging_slot();
        launch_check(world_->gather(g, stream), "broadcast");
        ++launches_;
    }
}

void DeviceSession::barrier(void *stream)
{
    std::lock_guard<std::recursive_mutex> lk(mu_);
    check();
    order_after_previous(stream);
    launch_check(world_->barrier(stream), "barrier");
    ++launches_;
}
}  // namespace stdml::collective::cuda
