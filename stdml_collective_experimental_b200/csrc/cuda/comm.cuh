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
};

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
    float scale;
    int phases;       // bit 0 pack, bit 1 reduce (with its barriers), bit 2 unpack
};

enum : int { kPhasePack = 1, kPhaseReduce = 2, kPhaseUnpack = 4, kPhaseAll = 7 };

struct GatherArgs {
    const void *src[kMaxRanks];  // nullptr: block already at arena offset `off`
    void *dst[kMaxRanks];
    unsigned long long off;     // arena slot (one block per rank)
    unsigned long long bytes;   // bytes per rank block
    unsigned long long stride;  // distance between rank blocks in dst (all_gather)
    int root;                   // < 0: all_gather; >= 0: broadcast from `root`
    int end_barrier;
    int algo;                   // broadcast only: see kBcast*
};

enum : int {
    kBcastPull = 0,     // everybody reads root's slot (small messages)
    kBcastNvls = 1,     // root multimem.st once, everybody copies its own slot
    kBcastScatter = 2,  // rank r pulls slice r from root, then all ranks exchange slices
};

// kernels_misc.cu
void launch_barrier(const CommCtx &ctx, int vranks, void *stream);
int launch_gather(const CommCtx &ctx, const GatherArgs &a, int blocks, int vranks,
                  void *stream);
// kernels_ar_*.cu: returns cudaError_t as int; -1 if (dtype, op, algo) is not built
int launch_all_reduce(const CommCtx &ctx, const AllReduceArgs &a, int dt, int op,
                      int blocks, int vranks, void *stream);
bool nvls_supported(int dt, int op);
// world of one GPU: dst = scale * src (integers: copy), no arena involved
int launch_local_scale(const void *src, void *dst, unsigned long long count, int dt, float scale,
                       int has_scale, int sms, void *stream);
}  // namespace stdml::collective::cuda
