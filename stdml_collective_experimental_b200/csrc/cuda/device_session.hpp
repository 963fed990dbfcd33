// DeviceSession: the collective front-end for CUDA buffers.  It decides, per
// call, between zero-copy (buffers that live in the symmetric heap) and staged
// execution (arbitrary device pointers packed into one of two staging slots
// inside the same kernel launch), splits messages larger than a slot, builds
// and caches the descriptor tables of fused groups, and turns a device-side
// timeout into an exception.
//
// It plays the role of the reference's session for device memory
// (include/stdml/bits/collective/session.hpp:25-178): all_reduce,
// group_all_reduce, all_gather, broadcast (any root; the reference fixes
// root 0), plus reduce, which the reference only declares
// (include/stdml/bits/collective/algorithm.hpp:16-18).
//
// Pointer arguments are arrays with one entry per virtual rank (`vranks()`):
// one entry for a real multi-GPU world, `world` entries for a loopback world.
#pragma once
#include <cstddef>
#include <map>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "device_world.hpp"

namespace stdml::collective::cuda
{
struct DeviceTimeout : std::runtime_error {
    DeviceStatus status;
    DeviceTimeout(const std::string &what, const DeviceStatus &s)
        : std::runtime_error(what), status(s)
    {
    }
};

// One tensor (or part of one) placed in a staging slot: elements
// [first_elem, first_elem + count) of tensor `tensor` at vector offset `voff`.
struct GroupPiece {
    size_t tensor, first_elem, count, voff;
};

// Cuts a sequence of tensors (element counts) into chunks of at most `cap`
// 16-byte vectors; a tensor that does not fit is split at a vector boundary.
// Every element appears in exactly one piece; pieces of one chunk are in tensor
// order and start on vector boundaries.  Pure function (tested on the CPU).
std::vector<std::vector<GroupPiece>> plan_group_pieces(size_t n, const size_t *counts,
                                                       size_t lanes, size_t cap);

class DeviceSession
{
  public:
    explicit DeviceSession(std::unique_ptr<DeviceWorld> world);
    ~DeviceSession();

    DeviceWorld &world() { return *world_; }
    int rank() const { return world_->rank(); }
    int size() const { return world_->world(); }
    int vranks() const { return world_->vranks(); }

    // out[i] = scale * (in_0[i] op in_1[i] op ... ), scale == 1 means none.
    // algo < 0 picks by size.  In-place (in == out) is allowed.
    void all_reduce(const void *const *in, void *const *out, size_t count, int dt, int op,
                    double scale, int algo, void *stream);
    // Only `root` receives the result; `out` of other ranks may be null.
    void reduce(const void *const *in, void *const *out, size_t count, int dt, int op, int root,
                double scale, void *stream);
    // n tensors, ins/outs laid out [vrank][tensor].  user_dt < 0: tensors have
    // the wire type `dt`; otherwise tensors are f32 and travel as bf16/f16.
    void group_all_reduce(size_t n, const void *const *ins, void *const *outs,
                          const size_t *counts, int dt, int op, int user_dt, double scale,
                          int algo, void *stream);
    void all_gather(const void *const *in, void *const *out, size_t count, int dt, void *stream);
    void broadcast(const void *const *in, void *const *out, size_t count, int dt, int root,
                   void *stream);
    void barrier(void *stream);

    // Knobs of the session (register_min_bytes) and of its world (see
    // DeviceWorld::set_knob).  register_min_bytes: collectives on ordinary device
    // buffers of at least this many bytes have the buffers' allocations mapped
    // on every peer (DeviceWorld::resolve_peers) and run zero-copy on them
    // instead of staging through the arena; negative: never (the default, also
    // STDML_COLLECTIVE_REGISTER_MIN_BYTES).  Such buffers must stay allocated
    // until drop_registrations() or the end of the session, and every rank must
    // make the same choice between in-place and out-of-place for a call.
    void set_knob(const std::string &name, long long value);
    // Collective: unmap every registered peer buffer (before memory that was
    // used in registered calls is freed).
    void drop_registrations();

    // Throws DeviceTimeout if a kernel reported a wait that ran out.
    void check();
    // Kernel launches issued so far (all kinds).
    unsigned long long launches() const { return launches_; }

  private:
    struct Table {
        GroupEntry *dev = nullptr;
        int n = 0;
        size_t nvec = 0;
    };
    struct GroupPlan {
        std::vector<std::vector<Table>> chunks;  // [chunk][vrank]
    };

    void launch_ar(AllReduceCall &c, void *stream);
    // Runs staged calls (one per staging slot) with their pack, reduce and
    // unpack phases on three streams, so that the HBM copies of one chunk
    // overlap the NVLink phase of its neighbours.
    void run_pipelined(std::vector<AllReduceCall> &calls, void *stream);
    void ensure_pipeline();
    size_t symmetric_offset(const void *const *ptrs) const;
    void run_gather_chunks(std::vector<GatherCall> &calls,
                           const std::vector<std::vector<void *>> &dsts, int blocks_n,
                           size_t stride, void *stream);
    const GroupPlan &plan_group(size_t n, const void *const *ins, void *const *outs,
                                const size_t *counts, int dt, int user_dt);

    // Every public call holds this from its first look at the session's state
    // to its last launch: calls from several threads of one rank are serialised
    // (the order in which they reach the stream must still be the same on every
    // rank: that is the callers' business).
    std::recursive_mutex mu_;
    std::unique_ptr<DeviceWorld> world_;
    std::map<std::string, GroupPlan> plans_;
    // Fused groups on registered tensors: the table of every rank's mappings,
    // kept per set of local pointers (and the allocations behind them).  `stamp`
    // counts the collective builds and is the same on every rank, which is how
    // the ranks confirm, with 8 bytes, that all of them still hold the same plan.
    struct PeerPlan {
        PeerEntry *dev = nullptr;  // null: this set cannot go the registered way
        int n = 0;
        size_t nvec = 0;
        unsigned long long stamp = 0;
    };
    std::map<std::string, PeerPlan> peer_plans_;
    unsigned long long peer_plan_builds_ = 0;
    // Look up the allocation id behind every tensor on every call (one driver query
    // per tensor), so that a tensor freed and allocated again at the same address
    // is noticed.  Knob register_verify = 0 trusts the addresses instead (for sets of
    // thousands of tensors in allocations that are never freed).
    bool register_verify_ = true;
    void forget_peer_plans();
    // Returns false when the set has to be staged (decided alike on every rank).
    bool group_registered(size_t n, const void *const *ins, void *const *outs,
                          const size_t *counts, int dt, int op, double scale, void *stream);
    std::vector<void *> table_mem_;
    unsigned long long launches_ = 0;
    // One signal pad serves the whole session, so its collectives must run on
    // the GPU one after the other, in the order issued.  On one stream that is
    // stream order; when a call comes in on another stream than the previous
    // one, it is made to wait for everything the previous stream holds.
    void order_after_previous(void *stream);
    void *last_stream_ = nullptr;
    bool have_last_stream_ = false;
    void *order_ev_ = nullptr;
    size_t register_min_bytes_ = SIZE_MAX;     // STDML_COLLECTIVE_REGISTER_MIN_BYTES
    int chunk_push_blocks_ = 128;   // grid of a chunk's push while the previous chunk is unpacked (knob;
                                    // 8 GPUs, 64 MB per rank: 128 / 96 gave 850 us where 64 / 0 gave 956)
    int chunk_unpack_blocks_ = 96;   // grid of that unpack (0: as many as the copy wants) (knob)
    bool registered_path(size_t bytes, void *stream) const;
    size_t pipeline_min_bytes_ = 256u << 20;   // STDML_COLLECTIVE_PIPELINE_MIN_BYTES
    size_t pipeline_chunk_bytes_ = 32u << 20;  // STDML_COLLECTIVE_PIPELINE_CHUNK_BYTES (smallest chunk)
    // pipeline resources (created on first use)
    void *pack_stream_ = nullptr;
    void *unpack_stream_ = nullptr;
    void *entry_ev_ = nullptr;
    void *packed_ev_[2] = {nullptr, nullptr};
    void *reduced_ev_[2] = {nullptr, nullptr};
    void *unpacked_ev_[2] = {nullptr, nullptr};
};
}  // namespace stdml::collective::cuda
