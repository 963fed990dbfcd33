// Barrier, all_gather and broadcast kernels, and the (dtype, op) dispatcher of
// the all-reduce kernels.
//
// all_gather replaces the reference's full-mesh exchange
// (src/stdml/collective/all_gather.cpp:16-56); broadcast replaces the walk of
// the broadcast graph from rank 0 (src/stdml/collective/session.cpp:49-62);
// the barrier replaces all_reduce(uint32 1) (src/stdml/collective/session.cpp:130-134).
#include "ar_kernel.cuh"

namespace stdml::collective::cuda
{
int launch_all_reduce_f(const CommCtx &, const AllReduceArgs &, int, int, int, int, void *);
int launch_all_reduce_i(const CommCtx &, const AllReduceArgs &, int, int, int, int, void *);
int launch_all_reduce_u(const CommCtx &, const AllReduceArgs &, int, int, int, int, void *);

int launch_all_reduce(const CommCtx &ctx, const AllReduceArgs &a, int dt, int op, int blocks,
                      int vranks, void *stream)
{
    if (dt >= DT_BF16 && dt <= DT_F64) {
        return launch_all_reduce_f(ctx, a, dt, op, blocks, vranks, stream);
    }
    if (dt >= DT_I8 && dt <= DT_I64) {
        return launch_all_reduce_i(ctx, a, dt, op, blocks, vranks, stream);
    }
    if (dt >= DT_U8 && dt <= DT_U64) {
        return launch_all_reduce_u(ctx, a, dt, op, blocks, vranks, stream);
    }
    return -1;
}

// A world of one GPU: all_reduce degenerates to out = scale * in.  No peers, no
// barrier, no arena: a copy in which every block walks contiguous 32 KB tiles
// (8 vectors per thread in flight), so that DRAM pages and TLB entries are used
// up before the block moves on.
constexpr int kLocalThreads = 256;
constexpr int kLocalUnroll = 8;

template <int DT>
__global__ void __launch_bounds__(kLocalThreads)
    local_scale_kernel(const void *src, void *dst,
                       unsigned long long count, double scale, int has_scale)
{
    constexpr unsigned long long N = lanes_of<DT>();
    constexpr unsigned long long kTile = static_cast<unsigned long long>(kLocalThreads) * kLocalUnroll;
    const unsigned long long nvec = (count + N - 1) / N;
    const unsigned long long ntiles = (nvec + kTile - 1) / kTile;
    const bool al = ptr_aligned16(src) && ptr_aligned16(dst);
    for (unsigned long long t = blockIdx.x; t < ntiles; t += gridDim.x) {
        const unsigned long long v0 = t * kTile + threadIdx.x;
        uint4 x[kLocalUnroll];
#pragma unroll
        for (int u = 0; u < kLocalUnroll; ++u) {
            const unsigned long long v = v0 + static_cast<unsigned long long>(u) * kLocalThreads;
            if (v < nvec) { x[u] = load_user_vec<DT>(src, false, v, count, al); }
        }
#pragma unroll
        for (int u = 0; u < kLocalUnroll; ++u) {
            const unsigned long long v = v0 + static_cast<unsigned long long>(u) * kLocalThreads;
            if (v < nvec) {
                if constexpr (Tr<DT>::is_float) {
                    if (has_scale) { x[u] = scale_vec<DT>(x[u], scale); }
                }
                store_user_vec<DT>(dst, false, v, count, al, x[u]);
            }
        }
    }
}

template <int DT>
static int launch_local_dt(const void *src, void *dst, unsigned long long count, double scale,
                           int has_scale, int sms, cudaStream_t s)
{
    constexpr unsigned long long N = lanes_of<DT>();
    const unsigned long long nvec = (count + N - 1) / N;
    const unsigned long long tile = static_cast<unsigned long long>(kLocalThreads) * kLocalUnroll;
    unsigned long long blocks = (nvec + tile - 1) / tile;
    const unsigned long long cap = static_cast<unsigned long long>(sms) * 8;  // 8 resident CTAs per SM
    if (blocks > cap) { blocks = cap; }
    if (blocks < 1) { blocks = 1; }
    local_scale_kernel<DT><<<static_cast<unsigned int>(blocks), kLocalThreads, 0, s>>>(
        src, dst, count, scale, has_scale);
    return static_cast<int>(cudaGetLastError());
}

int launch_local_scale(const void *src, void *dst, unsigned long long count, int dt, double scale,
                       int has_scale, int sms, void *stream)
{
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dt) {
    case DT_I8:
    case DT_U8:
        return launch_local_dt<DT_U8>(src, dst, count, scale, 0, sms, s);
    case DT_I16:
    case DT_U16:
        return launch_local_dt<DT_U16>(src, dst, count, scale, 0, sms, s);
    case DT_I32:
    case DT_U32:
        return launch_local_dt<DT_U32>(src, dst, count, scale, 0, sms, s);
    case DT_I64:
    case DT_U64:
        return launch_local_dt<DT_U64>(src, dst, count, scale, 0, sms, s);
    case DT_BF16:
        return launch_local_dt<DT_BF16>(src, dst, count, scale, has_scale, sms, s);
    case DT_F16:
        return launch_local_dt<DT_F16>(src, dst, count, scale, has_scale, sms, s);
    case DT_F32:
        return launch_local_dt<DT_F32>(src, dst, count, scale, has_scale, sms, s);
    case DT_F64:
        return launch_local_dt<DT_F64>(src, dst, count, scale, has_scale, sms, s);
    }
    return -1;
}

bool nvls_supported(int dt, int op)
{
    if (dt == DT_F32) { return op == OP_SUM; }
    if (dt == DT_BF16 || dt == DT_F16) { return op == OP_SUM || op == OP_MIN || op == OP_MAX; }
    return false;
}

__global__ void __launch_bounds__(kThreads) barrier_kernel(const __grid_constant__ CommCtx ctx)
{
    __shared__ BlockSync sync;
    const int rank = ctx.rank + static_cast<int>(blockIdx.y);
    sync_begin(ctx, rank, &sync);
    if (!peer_barrier(ctx, rank, &sync)) { return; }
    sync_end(ctx, rank, &sync);
}

void launch_barrier(const CommCtx &ctx, int vranks, void *stream)
{
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (vranks > 1) {
        void *params[1] = {const_cast<CommCtx *>(&ctx)};
        cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(&barrier_kernel),
                                    dim3(1, vranks, 1), dim3(kThreads), params, 0, s);
        return;
    }
    barrier_kernel<<<1, kThreads, 0, s>>>(ctx);
}

// all_gather and broadcast.  Data moves between GPUs either by pull (16-byte
// peer loads: small messages, one barrier) or by push (posted 16-byte stores, or
// multimem.st through the switch, into every rank's symmetric region: large
// messages; stores are not bound by the round trip that loads pay).  With a
// destination outside the region the kernel ends with a local unpack.
__device__ __forceinline__ void copy_span_to_user(char *out, unsigned long long bytes,
                                                  const char *from, const Span &sp)
{
    const bool al = ptr_aligned16(out);
    unsigned long long v = sp.lo + threadIdx.x;
    for (; v + 3ull * kThreads < sp.hi; v += 4ull * kThreads) {
        uint4 x[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) { x[u] = ld_arena_v4(from + (v + u * kThreads) * 16ull); }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            store_user_vec<DT_U8>(out, false, v + u * kThreads, bytes, al, x[u]);
        }
    }
    for (; v < sp.hi; v += kThreads) {
        store_user_vec<DT_U8>(out, false, v, bytes, al, ld_arena_v4(from + v * 16ull));
    }
}

// Vectors [sp.lo, sp.hi) of one block: read them from `src` (user memory, any
// alignment, `bytes` long) or from `sym` (16-byte vectors) and hand each to
// put(v, x), four loads in flight per thread.
template <typename Put>
__device__ __forceinline__ void for_each_block_vec(const void *src, const char *sym,
                                                   unsigned long long bytes, const Span &sp,
                                                   Put put)
{
    const bool al = src != nullptr && ptr_aligned16(src);
    unsigned long long v = sp.lo + threadIdx.x;
    for (; v + 3ull * kThreads < sp.hi; v += 4ull * kThreads) {
        uint4 x[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const unsigned long long vu = v + u * kThreads;
            x[u] = src != nullptr ? load_user_vec<DT_U8>(src, false, vu, bytes, al)
                                  : ld_arena_v4(sym + vu * 16ull);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) { put(v + u * kThreads, x[u]); }
    }
    for (; v < sp.hi; v += kThreads) {
        put(v, src != nullptr ? load_user_vec<DT_U8>(src, false, v, bytes, al)
                              : ld_arena_v4(sym + v * 16ull));
    }
}

__global__ void __launch_bounds__(kThreads)
    gather_kernel(const __grid_constant__ CommCtx ctx, const __grid_constant__ GatherArgs a)
{
    __shared__ BlockSync sync;
    const int vr = static_cast<int>(blockIdx.y);
    const int rank = ctx.rank + vr;
    const int world = ctx.world;
    const int nb = static_cast<int>(gridDim.x);
    const int b = static_cast<int>(blockIdx.x);
    sync_begin(ctx, rank, &sync);

    const unsigned long long nvec = (a.bytes + 15ull) / 16ull;
    const Span whole = span_of(nvec, 1, 0, nb, b);
    char *mine = a.data[rank];
    const void *src = a.src[vr];
    char *dst = static_cast<char *>(a.dst[vr]);
    const bool bcast = a.root >= 0;
    const bool is_root = a.root == rank;

    if (a.start_barrier) {
        if (!peer_barrier(ctx, rank, &sync)) { return; }
    }

    if (a.algo == kGatherPush && !bcast) {
        // ---- all_gather, push: my block goes into block `rank` of every region
        const unsigned long long at = static_cast<unsigned long long>(rank) * a.sym_stride;
        for_each_block_vec(src, mine + at, a.bytes, whole,
                           [&](unsigned long long v, const uint4 &x) {
                               if (a.use_mc) {
                                   mm_st_v4(ctx.mc_base + a.off + at + v * 16ull, x);
                                   return;
                               }
                               for (int i = 0; i < world; ++i) {
                                   const int r = (rank + 1 + i) % world;  // own region last
                                   if (r == rank && src == nullptr) { continue; }  // in place
                                   st_arena_v4(a.data[r] + at + v * 16ull, x);
                               }
                           });
        if (!peer_barrier(ctx, rank, &sync)) { return; }
        if (dst != nullptr) {
            for (int i = 0; i < world; ++i) {
                const int p = (rank + i) % world;
                copy_span_to_user(dst + static_cast<unsigned long long>(p) * a.stride, a.bytes,
                                  mine + static_cast<unsigned long long>(p) * a.sym_stride, whole);
            }
        }
    } else if (bcast && (a.algo == kBcastNvls || a.algo == kGatherPush)) {
        // ---- broadcast, push: root stores every vector into every region, through
        // the switch (one store, replicated) or peer by peer
        if (is_root) {
            const bool mc = a.use_mc || a.algo == kBcastNvls;
            for_each_block_vec(src, mine, a.bytes, whole,
                               [&](unsigned long long v, const uint4 &x) {
                                   if (mc) {
                                       mm_st_v4(ctx.mc_base + a.off + v * 16ull, x);
                                       return;
                                   }
                                   for (int i = 0; i < world; ++i) {
                                       const int r = (rank + 1 + i) % world;
                                       if (r == rank && src == nullptr) { continue; }
                                       st_arena_v4(a.data[r] + v * 16ull, x);
                                   }
                               });
        }
        if (!peer_barrier(ctx, rank, &sync)) { return; }
        if (dst != nullptr) { copy_span_to_user(dst, a.bytes, mine, whole); }
    } else if (bcast && a.algo == kBcastScatter) {
        // ---- broadcast without the switch: root stores slice r into rank r's
        // region (its own slice into its own), then every rank stores the slice it
        // holds into all the other regions
        if (is_root) {
            for (int i = 0; i < world; ++i) {
                const int s = (rank + 1 + i) % world;
                if (s == rank && src == nullptr) { continue; }
                const Span sp = span_of(nvec, world, s, nb, b);
                // from user memory root also fills its own region completely (nobody
                // sends root anything), so that its unpack below finds the whole block
                const bool also_mine = src != nullptr && s != rank;
                for_each_block_vec(src, mine, a.bytes, sp,
                                   [&](unsigned long long v, const uint4 &x) {
                                       st_arena_v4(a.data[s] + v * 16ull, x);
                                       if (also_mine) { st_arena_v4(mine + v * 16ull, x); }
                                   });
            }
        }
        if (!peer_barrier(ctx, rank, &sync)) { return; }
        {
            const Span sp = span_of(nvec, world, rank, nb, b);
            for_each_block_vec(nullptr, mine, a.bytes, sp,
                               [&](unsigned long long v, const uint4 &x) {
                                   for (int i = 1; i < world; ++i) {
                                       const int r = (rank + i) % world;
                                       if (r == a.root) { continue; }  // root has it all
                                       st_arena_v4(a.data[r] + v * 16ull, x);
                                   }
                               });
        }
        if (!peer_barrier(ctx, rank, &sync)) { return; }
        if (dst != nullptr) {
            // slice by slice, with the partition the writers used: the barriers only
            // vouch for what blocks of this index wrote
            for (int i = 0; i < world; ++i) {
                const int s = (rank + i) % world;
                copy_span_to_user(dst, a.bytes, mine, span_of(nvec, world, s, nb, b));
            }
        }
    } else if (bcast && a.algo == kBcastPipelined) {
        // ---- the same in rounds, with the block cut into world - 1 slices, one per
        // non-root rank (root holds everything already and forwards nothing, so
        // its links carry the message exactly once).  Block b's part of a slice is
        // cut into `rounds` pieces.  Root sends piece k of every slice to its
        // holder and signals; a holder waits for signal k and forwards its piece k
        // to the other non-root ranks while root is already sending piece k + 1.
        const int rounds = a.rounds > 0 ? a.rounds : 1;
        const int ns = world - 1;
        auto piece = [&](int j, int k) {
            const Span sp = span_of(nvec, ns, j, nb, b);
            const unsigned long long groups = (sp.hi - sp.lo + kSpanGranule - 1) / kSpanGranule;
            Span r;
            r.lo = sp.lo + groups * static_cast<unsigned long long>(k) / rounds * kSpanGranule;
            r.hi = sp.lo + groups * static_cast<unsigned long long>(k + 1) / rounds * kSpanGranule;
            r.lo = r.lo < sp.hi ? r.lo : sp.hi;
            r.hi = r.hi < sp.hi ? r.hi : sp.hi;
            return r;
        };
        const int my_slice = (rank - a.root - 1 + world) % world;  // non-root ranks
        for (int k = 0; k < rounds; ++k) {
            if (is_root) {
                for (int j = 0; j < ns; ++j) {
                    const int holder = (rank + 1 + j) % world;
                    for_each_block_vec(src, mine, a.bytes, piece(j, k),
                                       [&](unsigned long long v, const uint4 &x) {
                                           st_arena_v4(a.data[holder] + v * 16ull, x);
                                           // from user memory root fills its own region too,
                                           // for its unpack below
                                           if (src != nullptr) { st_arena_v4(mine + v * 16ull, x); }
                                       });
                }
                signal_from(ctx, rank, &sync, k);
            } else {
                if (!wait_for(ctx, rank, a.root, &sync, k)) { return; }
                for_each_block_vec(nullptr, mine, a.bytes, piece(my_slice, k),
                                   [&](unsigned long long v, const uint4 &x) {
                                       for (int i = 1; i < world; ++i) {
                                           const int r = (rank + i) % world;
                                           if (r == a.root) { continue; }
                                           st_arena_v4(a.data[r] + v * 16ull, x);
                                       }
                                   });
            }
        }
        rounds_done(&sync, rounds);
        if (!peer_barrier(ctx, rank, &sync)) { return; }
        if (dst != nullptr) {
            for (int j = 0; j < ns; ++j) {
                copy_span_to_user(dst, a.bytes, mine, span_of(nvec, ns, (my_slice + j) % ns, nb, b));
            }
        }
    } else {
        // ---- pull (small messages): pack, one barrier, read the peers' regions
        if (src != nullptr && (!bcast || is_root)) {
            const unsigned long long at =
                bcast ? 0ull : static_cast<unsigned long long>(rank) * a.sym_stride;
            for_each_block_vec(src, mine, a.bytes, whole,
                               [&](unsigned long long v, const uint4 &x) {
                                   st_arena_v4(mine + at + v * 16ull, x);
                               });
        }
        if (!peer_barrier(ctx, rank, &sync)) { return; }
        // without a user destination the region itself is the destination (zero-copy
        // on registered or symmetric memory): what is already in place is skipped
        if (dst != nullptr || !bcast || !is_root) {
            const int count = bcast ? 1 : world;
            for (int i = 0; i < count; ++i) {
                // start with the next rank so that peers do not all read the same GPU first
                const int p = bcast ? a.root : (rank + 1 + i) % world;
                if (dst == nullptr && p == rank) { continue; }
                const unsigned long long at =
                    bcast ? 0ull : static_cast<unsigned long long>(p) * a.sym_stride;
                char *out = dst != nullptr
                                ? (bcast ? dst : dst + static_cast<unsigned long long>(p) * a.stride)
                                : mine + at;
                copy_span_to_user(out, a.bytes, a.data[p] + at, whole);
            }
        }
    }

    if (a.end_barrier) {
        if (!peer_barrier(ctx, rank, &sync)) { return; }
    }
    sync_end(ctx, rank, &sync);
}

// Local copy of gathered blocks out of a region into user memory: the unpack
// of a chunk, run on its own stream while the next chunk is on the links.
__global__ void __launch_bounds__(kThreads)
    unpack_blocks_kernel(const char *region, char *dst, unsigned long long bytes,
                         unsigned long long sym_stride, unsigned long long stride, int blocks_n)
{
    const unsigned long long nvec = (bytes + 15ull) / 16ull;
    const Span whole = span_of(nvec, 1, 0, static_cast<int>(gridDim.x), static_cast<int>(blockIdx.x));
    for (int p = 0; p < blocks_n; ++p) {
        copy_span_to_user(dst + static_cast<unsigned long long>(p) * stride, bytes,
                          region + static_cast<unsigned long long>(p) * sym_stride, whole);
    }
}

int launch_unpack_blocks(const void *region, void *dst, unsigned long long bytes,
                         unsigned long long sym_stride, unsigned long long stride, int blocks_n,
                         int grid, void *stream)
{
    unpack_blocks_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const char *>(region), static_cast<char *>(dst), bytes, sym_stride, stride,
        blocks_n);
    return static_cast<int>(cudaGetLastError());
}

int launch_gather(const CommCtx &ctx, const GatherArgs &a, int blocks, int vranks, void *stream)
{
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    dim3 grid(blocks, vranks, 1);
    if (vranks > 1) {
        void *params[2] = {const_cast<CommCtx *>(&ctx), const_cast<GatherArgs *>(&a)};
        return static_cast<int>(cudaLaunchCooperativeKernel(
            reinterpret_cast<const void *>(&gather_kernel), grid, dim3(kThreads), params, 0, s));
    }
    gather_kernel<<<grid, kThreads, 0, s>>>(ctx, a);
    return static_cast<int>(cudaGetLastError());
}
}  // namespace stdml::collective::cuda
