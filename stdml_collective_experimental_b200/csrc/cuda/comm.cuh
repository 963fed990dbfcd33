// Device-side contract of the NVLink data plane: the symmetric arena layout,
// the signal pad, the launch-time context, and the argument blocks of every
// collective kernel.  Shared by kernels_*.cu (device) and device_world.cpp
// (host launcher).
//
// The reference has no device code at all; these kernels replace its CPU hot
// loops: the elementwise reducer (src/stdml/collective/dtype.cpp:80-165), the
// star / ring graph executors
// (src/stdml/collective/run_graph_pair_list_multi_thread.cpp:58-97) and the
// full-mesh all_gather (src/stdml/collective/all_gather.cpp:16-56).
#pragma once
#include <cstddef>
#include <cstdint>

#if defined(__CUDACC__)
#define STDML_HD __host__ __device__
#else
#define STDML_HD
#endif

namespace stdml::collective::cuda
{
constexpr int kMaxRanks = 16;     // ranks addressable from one kernel
constexpr int kMaxBlocks = 1024;  // grid.x limit of every collective kernel
constexpr int kThreads = 512;     // block size of every collective kernel

// Every rank's arena starts with one SignalPad; the data region follows at
// kDataOffset.  flag[b][s] is written only by rank s (block b) with a value
// that grows by one per barrier; epoch[b] is private to the owning rank and
// remembers how many barriers block b has passed, so that launches need no
// host-side counter and all ranks agree as long as they launch the same
// sequence of grids.
//
// One pad per world means: the collectives of a world run on the GPU one at a
// time, in the same order on every rank.  Two kernels of one world running side
// by side (two streams, no dependency) would count each other's arrivals.  The
// session enforces the order (DeviceSession::order_after_previous: a call that
// arrives on another stream than the previous one first waits for that
// stream); code that launches through DeviceWorld directly must do the same.
struct SignalPad {
    uint32_t flag[kMaxBlocks][kMaxRanks];
    uint32_t epoch[kMaxBlocks];
};

constexpr size_t kDataOffset = 128u << 10;
static_assert(sizeof(SignalPad) <= kDataOffset, "signal pad must fit");

// Status codes written to the host-visible status block by a kernel that gave
// up.  A kernel never traps and never spins without a limit.
enum : int {
    kStatusOk = 0,
    kStatusTimeout = 1,    // a peer's flag did not arrive in time
    kStatusBadArgs = 2,    // launch arguments failed the kernel's own checks
};

struct StatusBlock {
    int code;      // first failure wins (atomicCAS from 0)
    int rank;      // rank that observed it
    int block;     // blockIdx.x
    int peer;      // peer whose flag was missing (timeout)
    unsigned int want;  // flag value waited for
    unsigned int have;  // flag value last seen
    int phase;     // barrier ordinal inside the kernel
    int pad;
};

struct CommCtx {
    char *base[kMaxRanks];  // arena base of rank r as mapped in this process
    char *mc_base;          // NVLS multicast mapping of the arena, or nullptr
    StatusBlock *status;    // host-mapped
    unsigned long long timeout_ns;
    unsigned int max_spins;  // hard iteration limit of one wait
    int world;
    int rank;  // rank served by blockIdx.y == 0 (virtual ranks: rank + blockIdx.y)
};

enum : int {
    kAlgoOneShot = 0,      // every rank reads all peers and reduces locally
    kAlgoTwoShot = 1,      // owner reduces its shard, stores it to all peers
    kAlgoNvls = 2,         // owner multimem.ld_reduce -> multimem.st
    kAlgoNvlsOneShot = 3,  // every rank multimem.ld_reduce of everything
    kAlgoTwoShotTma = 4,   // two-shot whose pulls are bulk async copies (TMA) of every
                           // rank's tile into a shared-memory ring; results leave as
                           // plain 16-byte stores
    kAlgoNvlsHybrid = 5,   // most of each shard through the switch (NVLS), the rest by
                           // peer loads and stores from other CTAs of the same launch:
                           // the two kinds of traffic load the links differently
    kAlgoCount = 6,
};

// Owner algorithms: rank r reduces shard r and writes the result into every
// rank's symmetric buffer, so they can run in place.
STDML_HD inline bool is_owner_algo(int algo)
{
    return algo == kAlgoTwoShot || algo == kAlgoNvls || algo == kAlgoTwoShotTma ||
           algo == kAlgoNvlsHybrid;
}

// Shared-memory ring of the bulk-copy two-shot kernel: `stages` slots, each
// holding one tile of `tile_vec` 16-byte vectors from every rank.
constexpr int kTmaMaxStages = 16;
constexpr unsigned int kTmaSmemBudget = 192u << 10;  // bytes of the 227 KB an SM offers

// Ring geometry for a world: the wanted tile (default: 1024 vectors, 16 KB per
// rank and copy; measured at 2 GPUs: 1024 > 512 > 256), halved until two slots
// fit the budget, then as many slots as fit.
inline void tma_geometry(int world, unsigned int want_tile_vec, int *stages,
                         unsigned int *tile_vec, unsigned int *smem_bytes)
{
    unsigned int tv = want_tile_vec > 0 ? want_tile_vec : 1024u;
    tv = (tv + 31u) / 32u * 32u;
    while (tv > 32u && 2ull * world * tv * 16ull > kTmaSmemBudget) { tv /= 2; }
    unsigned int st = static_cast<unsigned int>(
        kTmaSmemBudget / (static_cast<unsigned long long>(world) * tv * 16ull));
    if (st > static_cast<unsigned int>(kTmaMaxStages)) { st = kTmaMaxStages; }
    if (st < 1u) { st = 1u; }
    *stages = static_cast<int>(st);
    *tile_vec = tv;
    *smem_bytes = st * static_cast<unsigned int>(world) * tv * 16u;
}

// One tensor of a fused group: `count` elements that live at vector offset
// `voff` (16-byte units) of the flat symmetric region.
struct GroupEntry {
    const void *src;  // user memory to pack from (nullptr: already in the arena)
    void *dst;        // user memory to unpack to (nullptr: leave in the arena)
    unsigned long long voff;
    unsigned long long count;
};

struct AllReduceArgs {
    // Per virtual rank (index blockIdx.y); real multi-GPU launches use [0].
    const void *src[kMaxRanks];  // nullptr: input already at arena offset `off`
    void *dst[kMaxRanks];        // nullptr: result stays in the arena (two-shot/nvls)
    const GroupEntry *table[kMaxRanks];  // non-null: fused group, src/dst unused
    // Rank r's buffer as mapped in this process: arena base + `off` for symmetric
    // and staged buffers, the peer mapping of a registered user buffer otherwise
    // (then `off` is 0 and the NVLS algorithms, which need the arena's multicast
    // mapping, are not available).
    char *data[kMaxRanks];
    // Where the owner algorithms store results: the same buffers, except for
    // registered out-of-place calls (operands pulled from the peers' inputs,
    // results stored into their outputs; reduce-to-root: only [root] is used).
    char *push[kMaxRanks];
    unsigned long long off;    // byte offset of the symmetric buffer in the arena
    unsigned long long count;  // elements (single buffer) or padded elements (group)
    unsigned long long nvec;   // 16-byte vectors of the symmetric buffer
    int ntable;                // entries of a group table
    int algo;
    int user_dtype;   // dtype of src/dst memory; differs from the wire type only
                      // for f32 <-> bf16/f16
    int end_barrier;  // one-shot: protect an arena-resident input from reuse
    int root;         // >= 0: reduce-to-root (only `root` computes and stores)
    int has_scale;
    double scale;     // applied as f64 to f64 buffers, as its f32 value otherwise
    int phases;       // bit 0 pack, bit 1 reduce (with its barriers), bit 2 unpack
    int nvls_variant; // inner loop of the NVLS reduce: see kNvls* below
    int tma_stages;   // kAlgoTwoShotTma: slots of the shared-memory ring
    unsigned int tma_tile_vec;  // kAlgoTwoShotTma: vectors per rank per tile
    int hybrid_nvls_blocks;  // kAlgoNvlsHybrid: CTAs [0, this) take the NVLS region
    unsigned long long hybrid_split_vec;  // kAlgoNvlsHybrid: vectors [0, this) are the NVLS region
    int debug_checks; // != 0: validate offsets / table / alignment in the kernel and
                      // report kStatusBadArgs instead of touching memory
};

// NVLS inner loops (all produce the same values; measured against each other).
enum : int {
    kNvlsPlain4 = 0,  // 4 loads, then 4 stores per thread and iteration
    kNvlsPipe4 = 1,   // the loads of iteration i+1 are issued before the stores of i
    kNvlsPipe8 = 2,   // same with 8 vectors per thread
    kNvlsPlain8 = 3,
    kNvlsVariants = 4,
};

// A fused group on REGISTERED tensors: every tensor of every rank is addressed
// through its own peer mapping, nothing is packed.  Entry i covers the vectors
// [voff, voff + ceil(count / lanes)) of the group's flat index space.
struct PeerEntry {
    char *in[kMaxRanks];   // tensor i of rank r as mapped here (operands)
    char *out[kMaxRanks];  // where rank r wants the result (often the same memory)
    unsigned long long voff;
    unsigned long long count;  // elements
};

struct GroupPeerArgs {
    const PeerEntry *table;  // device memory, sorted by voff, entry 0 at 0
    int ntable;
    unsigned long long nvec;  // vectors of the flat index space
    int has_scale;
    double scale;
    // bulk-copy variant (see tma_geometry): 0 stages = plain peer loads
    int tma_stages;
    unsigned int tma_tile_vec;
};

enum : int { kPhasePack = 1, kPhaseReduce = 2, kPhaseUnpack = 4, kPhaseAll = 7 };

struct GatherArgs {
    const void *src[kMaxRanks];  // per virtual rank; nullptr: the rank's block is already in
                                 // place in its own symmetric region
    void *dst[kMaxRanks];        // per virtual rank; nullptr: the result stays in the region
    // Rank r's symmetric region as mapped here (an arena slot, a symmetric-heap
    // tensor, or a registered user buffer).  all_gather: world blocks, block p at
    // p * sym_stride; broadcast: one block.
    char *data[kMaxRanks];
    unsigned long long off;         // arena offset of the region (multimem), 0 if not in the arena
    unsigned long long bytes;       // bytes per rank block
    unsigned long long sym_stride;  // all_gather: distance between blocks in the region
    unsigned long long stride;      // all_gather: distance between blocks in dst
    int root;                       // < 0: all_gather; >= 0: broadcast from `root`
    int start_barrier;  // the region is memory its owner may still be using (zero-copy)
    int end_barrier;    // the region is reused by the next call (captured staged calls)
    int algo;           // see kGather* / kBcast*
    int use_mc;         // push through the switch (multimem.st) instead of one store per peer
    int rounds;         // kBcastPipelined: pieces per block and slice
};

enum : int {
    kBcastPull = 0,     // root packs, everybody reads root's region (small messages);
                        // all_gather: everybody packs, then reads every peer's region
    kBcastNvls = 1,     // root multimem.st once, everybody copies its own region
    kBcastScatter = 2,  // root stores slice r to rank r, then every rank stores its slice
                        // to all others (root's links carry ~2 copies, not n-1)
    kGatherPush = 3,    // every rank stores its block into every rank's region; broadcast:
                        // root stores the block into every rank's region
    kBcastPipelined = 4,  // kBcastScatter in rounds: root signals each round, the holders
                          // forward their part of it while root sends the next one, so
                          // root's links and everybody else's are busy at the same time
};

// kernels_misc.cu
void launch_barrier(const CommCtx &ctx, int vranks, void *stream);
int launch_gather(const CommCtx &ctx, const GatherArgs &a, int blocks, int vranks,
                  void *stream);
int launch_unpack_blocks(const void *region, void *dst, unsigned long long bytes,
                         unsigned long long sym_stride, unsigned long long stride, int blocks_n,
                         int grid, void *stream);
// kernels_ar_*.cu: returns cudaError_t as int; -1 if (dtype, op, algo) is not built
int launch_all_reduce(const CommCtx &ctx, const AllReduceArgs &a, int dt, int op,
                      int blocks, int vranks, void *stream);
bool nvls_supported(int dt, int op);
// kernels_group_peer.cu: two-shot over a table of registered tensors
int launch_group_peer(const CommCtx &ctx, const GroupPeerArgs &a, int dt, int op, int blocks,
                      int vranks, void *stream);
// world of one GPU: dst = scale * src (integers: copy), no arena involved
int launch_local_scale(const void *src, void *dst, unsigned long long count, int dt, double scale,
                       int has_scale, int sms, void *stream);
}  // namespace stdml::collective::cuda
