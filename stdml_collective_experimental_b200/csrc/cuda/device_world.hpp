// DeviceWorld: the symmetric-memory manager and kernel launcher of the NVLink
// data plane.  One per (process, GPU).  It owns
//   * this rank's arena (signal pad + two staging slots + a symmetric heap),
//     allocated with the CUDA VMM API and exported as a POSIX file descriptor
//     (or, as a fallback, cudaMalloc + CUDA IPC handles),
//   * the mappings of every peer's arena into this process,
//   * the NVLS multicast object bound over all arenas (when the box has it),
//   * a host-mapped status block that kernels write when a bounded wait runs out.
// A "loopback" world hosts all ranks on one GPU in one process; its kernels run
// as one cooperative launch with one grid row per virtual rank.  This is how
// the kernels are tested on a single GPU.
//
// The reference keeps the equivalent state (mailbox, slotbox, client pool) in
// `peer` (include/stdml/bits/collective/peer.hpp:26-32); it has no device
// memory of any kind.
#pragma once
#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "comm.cuh"

namespace stdml::collective::cuda
{
struct DeviceWorldOptions {
    int rank = 0;
    int world = 1;
    int device = 0;
    bool loopback = false;            // all ranks virtual, on `device`
    size_t heap_bytes = 1ull << 30;   // symmetric heap for user buffers
    size_t staging_bytes = 64ull << 20;  // each of the two staging slots
    std::string key = "default";      // rendezvous key (same on all ranks)
    std::string backend = "auto";     // auto | vmm | ipc
    bool enable_nvls = true;
    int setup_timeout_ms = 120000;
    unsigned long long wait_timeout_ms = 20000;  // device-side bounded waits
};

struct DeviceStatus {
    int code = 0;
    int rank = 0, block = 0, peer = 0, phase = 0;
    unsigned int want = 0, have = 0;
};

// What to run.  Pointers are per virtual rank: arrays of `vranks()` entries
// (1 for a real world, `world` for a loopback world).
struct AllReduceCall {
    size_t off = 0;  // arena byte offset of the symmetric buffer
    // Owner algorithms: store the results at this arena offset instead of over the
    // operands (0: in place).  Lets a reduce-to-root read symmetric inputs where
    // they are and deliver into root's staging slot.
    size_t push_off = 0;
    // Instead of `off`: the buffer of every rank of the world (world() entries) as
    // mapped in this process: a user buffer registered with register_buffer().
    // No NVLS then (the multicast mapping covers the arena only).
    void *const *peer_data = nullptr;
    // With peer_data: where the owner algorithms store results instead (world()
    // entries; reduce-to-root needs [root] only).  Null: into peer_data itself.
    void *const *peer_push = nullptr;
    const void *const *src = nullptr;
    void *const *dst = nullptr;
    const GroupEntry *const *table = nullptr;  // device pointers, one per vrank
    int ntable = 0;
    size_t count = 0;  // elements; for a group: flat length in wire elements
    int dt = 0;
    int op = 0;
    int user_dtype = -1;  // -1: same as dt
    int algo = -1;        // -1: pick by size
    int blocks = 0;       // 0: pick by size
    int root = -1;
    bool end_barrier = false;
    bool has_scale = false;
    double scale = 1.0;  // f64 buffers use all of it; other float types its f32 value
    int phases = 7;  // kPhasePack | kPhaseReduce | kPhaseUnpack
};

struct GatherCall {
    size_t off = 0;  // arena offset of the symmetric region (a staging slot or a heap buffer)
    // Instead of `off`: every rank's region as mapped here (registered user buffers).
    void *const *peer_data = nullptr;
    const void *const *src = nullptr;  // per vrank; null entry: block already in place
    void *const *dst = nullptr;        // per vrank; null entry: result stays in the region
    size_t bytes = 0;       // per rank block
    size_t sym_stride = 0;  // all_gather: distance between rank blocks in the region
    size_t stride = 0;      // all_gather: distance between rank blocks in dst (0: bytes)
    int root = -1;
    int blocks = 0;
    int algo = -1;       // -1 pick, else kBcast* / kGatherPush
    int use_mc = -1;     // -1 pick; push through the switch (needs NVLS and an arena region)
    bool start_barrier = false;  // the region is live memory of its owner (zero-copy)
    bool end_barrier = false;
};

class DeviceWorld
{
  public:
    static std::unique_ptr<DeviceWorld> create(const DeviceWorldOptions &opt);
    virtual ~DeviceWorld() = default;

    virtual int rank() const = 0;
    virtual int world() const = 0;
    virtual int vranks() const = 0;
    virtual int device() const = 0;
    virtual bool has_nvls() const = 0;
    virtual const char *backend() const = 0;
    virtual size_t arena_bytes() const = 0;
    // Where the set-up time of this world went, in milliseconds: [0] the local
    // rendezvous (UNIX-socket mesh among the ranks), [1] allocating and mapping
    // this rank's arena, [2] exchanging handles and mapping the peers' arenas,
    // [3] creating and binding the NVLS multicast object.
    virtual void setup_ms(double out[4]) const = 0;
    virtual size_t staging_bytes() const = 0;

    // Address of arena offset `off` of rank `r` as mapped here / of the
    // multicast mapping (nullptr without NVLS).
    virtual void *ptr(int r, size_t off) const = 0;
    virtual void *mc_ptr(size_t off) const = 0;
    // Offset of `p` inside the arena of virtual rank `vr`, or SIZE_MAX.
    virtual size_t offset_of(const void *p, int vr = 0) const = 0;

    // Registration of ordinary device memory (collective; every rank passes its
    // own buffer, or null for "none from me").  `ptrs` has vranks() entries,
    // `peer_ptrs` receives world() entries: rank r's buffer as mapped in this
    // process (own buffers as they are, null where a rank passed null).  The
    // base allocation of each buffer is exported once as a CUDA IPC handle over
    // the local rendezvous and stays mapped on the peers until
    // drop_registrations() or the end of the world: the owner must not free it
    // before.  Returns false, on every rank alike, when some rank cannot export
    // (memory that did not come from cudaMalloc) or import; callers then stage.
    virtual bool resolve_peers(const void *const *ptrs, size_t bytes, void **peer_ptrs) = 0;
    // The same for n buffers with ONE exchange: ptrs[v * n + i] is buffer i of
    // (virtual) rank v, peer_ptrs[i * world + r] buffer i of rank r as mapped here.
    virtual bool resolve_many(size_t n, const void *const *ptrs, const size_t *bytes,
                              void **peer_ptrs) = 0;
    // Collective: true when every rank passed the same non-zero token (8 bytes
    // over the local rendezvous; how cached plans are confirmed before reuse).
    virtual bool all_same(unsigned long long token) = 0;
    // A number that identifies the allocation behind `p` and is never used twice
    // in a process (0: not a device allocation the driver knows).
    virtual unsigned long long buffer_id(const void *p) const = 0;
    // Collective: unmaps every peer buffer imported so far.
    virtual void drop_registrations() = 0;
    virtual size_t registrations() const = 0;  // peer allocations mapped now

    // Symmetric heap: every rank must make the same calls in the same order.
    // Returns an arena offset (256-byte aligned).  Throws std::bad_alloc.
    virtual size_t alloc(size_t bytes) = 0;
    virtual void release(size_t off) = 0;
    // Staging slot for the next staged operation (alternates between two).
    virtual size_t next_staging_slot() = 0;

    virtual int pick_algo(size_t bytes, int dt, int op, bool need_owner) const = 0;
    // The owner algorithm for buffers outside the arena (no in-switch reduction there).
    virtual int pick_peer_algo(size_t bytes) const = 0;
    virtual int pick_blocks(size_t nvec, int algo) const = 0;

    // Launches.  Return 0 or a cudaError_t; throw std::invalid_argument on
    // arguments that the kernels could not run.
    virtual int all_reduce(const AllReduceCall &c, void *stream) = 0;
    virtual int gather(const GatherCall &c, void *stream) = 0;
    // Two-shot all-reduce over a table of registered tensors (see PeerEntry).
    virtual int group_peer(const PeerEntry *table, int ntable, size_t nvec, int dt, int op,
                           double scale, void *stream) = 0;
    // Local copy of `blocks_n` gathered blocks out of a region into user memory.
    virtual int unpack_blocks(const void *region, void *dst, size_t bytes, size_t sym_stride,
                              size_t stride, int blocks_n, void *stream, int grid = 0) = 0;
    virtual int barrier(void *stream) = 0;
    // Loopback worlds only: launch the barrier for the first `rows` virtual
    // ranks.  With rows < world the missing ranks never arrive, so the wait
    // runs out and the status block reports it; this is how the bounded wait
    // is exercised without any faulting code.
    virtual int barrier_rows(int rows, void *stream) = 0;

    // Bounded-wait status: poll_status() never blocks.
    virtual DeviceStatus poll_status() const = 0;
    // After a timeout: all ranks quiesce, clear their pads and meet again.
    virtual void recover() = 0;
    virtual void set_wait_timeout_ms(unsigned long long ms) = 0;
    virtual void set_tuning(int max_blocks, size_t oneshot_max_bytes,
                            size_t nvls_oneshot_max_bytes) = 0;
    // Named tuning knobs (each also has an environment variable, read at
    // creation): nvls_variant, nvls_blocks, tma_blocks, tma_tile_vec,
    // tma_min_bytes, tma_over_nvls_min_bytes (negative: never), debug_checks.
    // Every rank must set the same values.
    virtual void set_knob(const std::string &name, long long value) = 0;
};

// true when a usable CUDA device is present (never throws)
bool cuda_available();
int cuda_device_count();
// memory kind of a pointer: 0 host/unknown, 1 device
int pointer_kind(const void *p);
// Blocking copy between host and device memory in stream order: enqueues after
// what `stream` holds and returns when the copy is complete.
void copy_device_to_host(void *host, const void *device, size_t bytes, void *stream);
void copy_host_to_device(void *device, const void *host, size_t bytes, void *stream);
}  // namespace stdml::collective::cuda
