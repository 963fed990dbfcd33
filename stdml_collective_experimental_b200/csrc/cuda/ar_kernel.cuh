// The fused all-reduce kernel: pack (optional) -> cross-rank barrier ->
// reduce over peer memory (one-shot, two-shot or NVLS) with the gradient scale
// and the dtype cast applied in registers -> barrier -> unpack (optional), in
// ONE launch.  A single buffer is a group of one tensor, so all_reduce,
// group_all_reduce and reduce-to-root share this code.
//
// Replaces the reference's per-chunk graph walk
// (src/stdml/collective/run_graph_pair_list_multi_thread.cpp:58-97), its
// 76-thread group_all_reduce (src/stdml/collective/session.cpp:83-97) and the
// reducer loop (src/stdml/collective/dtype.cpp:124-165).
//
// Reduction order is rank-ascending for the peer-load algorithms (bit-identical
// on every rank and equal to reduce_many() on the host); the NVLS algorithms
// reduce inside the switch, whose order is not specified.
#pragma once
#include "prims.cuh"

namespace stdml::collective::cuda
{
constexpr int kUnroll = 4;  // vectors per thread per iteration

struct Span {
    unsigned long long lo, hi;
};

// Sub-range `b` of `nb` of shard `s` of `shards` of [0, nvec).
__host__ __device__ __forceinline__ Span span_of(unsigned long long nvec, int shards, int s, int nb,
                                        int b)
{
    const unsigned long long s_lo = nvec * static_cast<unsigned long long>(s) / shards;
    const unsigned long long s_hi = nvec * static_cast<unsigned long long>(s + 1) / shards;
    const unsigned long long len = s_hi - s_lo;
    Span r;
    r.lo = s_lo + len * static_cast<unsigned long long>(b) / nb;
    r.hi = s_lo + len * static_cast<unsigned long long>(b + 1) / nb;
    return r;
}

template <int DT>
__host__ __device__ __forceinline__ unsigned long long entry_nvec(unsigned long long count)
{
    constexpr unsigned long long N = lanes_of<DT>();
    return (count + N - 1) / N;
}

// Vector `lv` (local index inside one tensor) of user memory -> wire vector.
// Lanes past `count` read as zero.  user_f32: the user tensor is f32 while the
// wire type is a 16-bit float (cast on the way in).
template <int DT>
__device__ __forceinline__ uint4 load_user_vec(const void *src, bool user_f32,
                                               unsigned long long lv,
                                               unsigned long long count, bool aligned)
{
    using S = typename Tr<DT>::storage;
    constexpr int N = lanes_of<DT>();
    const unsigned long long e0 = lv * N;
    VecU<DT> u;
    if constexpr (Tr<DT>::is_half) {
        if (user_f32) {
            const float *f = static_cast<const float *>(src) + e0;
            if (aligned && e0 + N <= count) {
                const float4 a = *reinterpret_cast<const float4 *>(f);
                const float4 b = *reinterpret_cast<const float4 *>(f + 4);
                u.e[0] = Tr<DT>::narrow(a.x);
                u.e[1] = Tr<DT>::narrow(a.y);
                u.e[2] = Tr<DT>::narrow(a.z);
                u.e[3] = Tr<DT>::narrow(a.w);
                u.e[4] = Tr<DT>::narrow(b.x);
                u.e[5] = Tr<DT>::narrow(b.y);
                u.e[6] = Tr<DT>::narrow(b.z);
                u.e[7] = Tr<DT>::narrow(b.w);
            } else {
#pragma unroll
                for (int i = 0; i < N; ++i) {
                    u.e[i] = (e0 + i < count) ? Tr<DT>::narrow(f[i]) : S(0);
                }
            }
            return u.v;
        }
    }
    const S *p = static_cast<const S *>(src) + e0;
    if (aligned && e0 + N <= count) { return *reinterpret_cast<const uint4 *>(p); }
#pragma unroll
    for (int i = 0; i < N; ++i) { u.e[i] = (e0 + i < count) ? p[i] : S(0); }
    return u.v;
}

template <int DT>
__device__ __forceinline__ void store_user_vec(void *dst, bool user_f32,
                                               unsigned long long lv,
                                               unsigned long long count, bool aligned,
                                               const uint4 &x)
{
    using S = typename Tr<DT>::storage;
    constexpr int N = lanes_of<DT>();
    const unsigned long long e0 = lv * N;
    VecU<DT> u;
    u.v = x;
    if constexpr (Tr<DT>::is_half) {
        if (user_f32) {
            float *f = static_cast<float *>(dst) + e0;
            if (aligned && e0 + N <= count) {
                float4 a, b;
                a.x = Tr<DT>::widen(u.e[0]);
                a.y = Tr<DT>::widen(u.e[1]);
                a.z = Tr<DT>::widen(u.e[2]);
                a.w = Tr<DT>::widen(u.e[3]);
                b.x = Tr<DT>::widen(u.e[4]);
                b.y = Tr<DT>::widen(u.e[5]);
                b.z = Tr<DT>::widen(u.e[6]);
                b.w = Tr<DT>::widen(u.e[7]);
                *reinterpret_cast<float4 *>(f) = a;
                *reinterpret_cast<float4 *>(f + 4) = b;
            } else {
#pragma unroll
                for (int i = 0; i < N; ++i) {
                    if (e0 + i < count) { f[i] = Tr<DT>::widen(u.e[i]); }
                }
            }
            return;
        }
    }
    S *p = static_cast<S *>(dst) + e0;
    if (aligned && e0 + N <= count) {
        *reinterpret_cast<uint4 *>(p) = x;
        return;
    }
#pragma unroll
    for (int i = 0; i < N; ++i) {
        if (e0 + i < count) { p[i] = u.e[i]; }
    }
}

__device__ __forceinline__ bool ptr_aligned16(const void *p)
{
    return (reinterpret_cast<unsigned long long>(p) & 15ull) == 0ull;
}

// Index of the last table entry whose first vector is <= v (entries are sorted
// by voff and entry 0 starts at 0).
__host__ __device__ __forceinline__ int find_entry(const GroupEntry *tab, int n, unsigned long long v)
{
    int lo = 0, hi = n - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (tab[mid].voff <= v) {
            lo = mid;
        } else {
            hi = mid - 1;
        }
    }
    return lo;
}

// Calls f(entry, lo, hi) for every tensor that intersects [v0, v1), with
// [lo, hi) the intersection in flat vector indices.
template <int DT, typename F>
__device__ __forceinline__ void for_each_entry(const GroupEntry *tab, int n,
                                               const GroupEntry &single,
                                               unsigned long long v0,
                                               unsigned long long v1, F f)
{
    if (v0 >= v1) { return; }
    if (tab == nullptr) {
        const unsigned long long end = entry_nvec<DT>(single.count);
        const unsigned long long hi = v1 < end ? v1 : end;
        if (v0 < hi) { f(single, v0, hi); }
        return;
    }
    for (int i = find_entry(tab, n, v0); i < n; ++i) {
        const GroupEntry e = tab[i];
        if (e.voff >= v1) { break; }
        const unsigned long long end = e.voff + entry_nvec<DT>(e.count);
        const unsigned long long lo = v0 > e.voff ? v0 : e.voff;
        const unsigned long long hi = v1 < end ? v1 : end;
        if (lo < hi) { f(e, lo, hi); }
    }
}

// Reduce vectors [lo, hi) of the symmetric buffer at arena offset `off` over
// all ranks with peer loads (rank-ascending) and hand each result to
// store(v, value).
template <int DT, int OP, typename Store>
__device__ __forceinline__ void reduce_span(const CommCtx &ctx, unsigned long long off,
                                            unsigned long long lo, unsigned long long hi,
                                            float scale, bool has_scale, Store store)
{
    const int world = ctx.world;
    for (unsigned long long v = lo + threadIdx.x; v < hi;
         v += static_cast<unsigned long long>(kThreads) * kUnroll) {
        Accum<DT> acc[kUnroll];
        for (int r0 = 0; r0 < world; r0 += 4) {
            uint4 x[kUnroll][4];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const unsigned long long vu = v + static_cast<unsigned long long>(u) * kThreads;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (r0 + j < world && vu < hi) {
                        x[u][j] = ld_arena_v4(ctx.base[r0 + j] + off + vu * 16ull);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const unsigned long long vu = v + static_cast<unsigned long long>(u) * kThreads;
                if (vu < hi) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (r0 + j < world) {
                            if (r0 + j == 0) {
                                acc[u].init(x[u][j]);
                            } else {
                                acc[u].template add<OP>(x[u][j]);
                            }
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const unsigned long long vu = v + static_cast<unsigned long long>(u) * kThreads;
            if (vu < hi) { store(vu, acc[u].finish(scale, has_scale)); }
        }
    }
}

// Same with the reduction done by the switch.
template <int DT, int OP, typename Store>
__device__ __forceinline__ void nvls_span(const CommCtx &ctx, unsigned long long off,
                                          unsigned long long lo, unsigned long long hi,
                                          float scale, bool has_scale, Store store)
{
    if constexpr (nvls_ok<DT, OP>()) {
        for (unsigned long long v = lo + threadIdx.x; v < hi;
             v += static_cast<unsigned long long>(kThreads) * kUnroll) {
            uint4 x[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const unsigned long long vu = v + static_cast<unsigned long long>(u) * kThreads;
                if (vu < hi) { x[u] = mm_ld_reduce<DT, OP>(ctx.mc_base + off + vu * 16ull); }
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const unsigned long long vu = v + static_cast<unsigned long long>(u) * kThreads;
                if (vu < hi) { store(vu, has_scale ? scale_vec<DT>(x[u], scale) : x[u]); }
            }
        }
    }
}

template <int DT, int OP>
__global__ void __launch_bounds__(kThreads)
    all_reduce_kernel(const __grid_constant__ CommCtx ctx, const __grid_constant__ AllReduceArgs a)
{
    __shared__ BlockSync sync;
    const int vr = static_cast<int>(blockIdx.y);
    const int rank = ctx.rank + vr;
    const int world = ctx.world;
    const int nb = static_cast<int>(gridDim.x);
    const int b = static_cast<int>(blockIdx.x);
    const int algo = a.algo;
    const bool owner_algo = (algo == kAlgoTwoShot || algo == kAlgoNvls);
    const bool nvls = (algo == kAlgoNvls || algo == kAlgoNvlsOneShot);
    const int shards = owner_algo ? world : 1;
    const bool user_f32 = Tr<DT>::is_half && a.user_dtype == DT_F32;
    const bool computes = (a.root < 0 || a.root == rank);

    // A launch may run only some phases: large staged messages are cut into
    // chunks whose pack / reduce / unpack run as separate launches on three
    // streams, so that the HBM copies of one chunk overlap the NVLink phase of
    // another.  Only the reduce phase synchronises with peers.
    const int phases = a.phases;
    const bool do_reduce = (phases & kPhaseReduce) != 0;
    if (do_reduce) { sync_begin(ctx, rank, &sync); }

    char *mine = ctx.base[rank] + a.off;
    const GroupEntry *tab = a.table[vr];
    GroupEntry single;
    single.src = a.src[vr];
    single.dst = a.dst[vr];
    single.voff = 0;
    single.count = a.count;

    // ---- pack: user memory -> own arena buffer (the parts peers' block b read)
    if ((phases & kPhasePack) != 0 && (tab != nullptr || single.src != nullptr)) {
        for (int s = 0; s < shards; ++s) {
            const Span sp = span_of(a.nvec, shards, s, nb, b);
            for_each_entry<DT>(tab, a.ntable, single, sp.lo, sp.hi,
                               [&](const GroupEntry &e, unsigned long long lo,
                                   unsigned long long hi) {
                                   if (e.src == nullptr) { return; }
                                   const bool al = ptr_aligned16(e.src);
                                   unsigned long long v = lo + threadIdx.x;
                                   for (; v + 3ull * kThreads < hi; v += 4ull * kThreads) {
                                       uint4 x[4];
#pragma unroll
                                       for (int u = 0; u < 4; ++u) {
                                           x[u] = load_user_vec<DT>(e.src, user_f32,
                                                                    v + u * kThreads - e.voff,
                                                                    e.count, al);
                                       }
#pragma unroll
                                       for (int u = 0; u < 4; ++u) {
                                           st_arena_v4(mine + (v + u * kThreads) * 16ull, x[u]);
                                       }
                                   }
                                   for (; v < hi; v += kThreads) {
                                       st_arena_v4(mine + v * 16ull,
                                                   load_user_vec<DT>(e.src, user_f32, v - e.voff,
                                                                     e.count, al));
                                   }
                               });
        }
    }

    if (do_reduce && !peer_barrier(ctx, rank, &sync)) { return; }

    // ---- reduce
    if (!do_reduce) {
        // pack-only or unpack-only launch
    } else if (owner_algo) {
        // the owner of shard `rank` reduces it and stores the result into every
        // rank's buffer (only into root's for reduce-to-root)
        const Span sp = span_of(a.nvec, shards, rank, nb, b);
        auto push = [&](unsigned long long v, const uint4 &x) {
            if (nvls && a.root < 0) {
                mm_st_v4(ctx.mc_base + a.off + v * 16ull, x);
            } else if (a.root >= 0) {
                st_arena_v4(ctx.base[a.root] + a.off + v * 16ull, x);
            } else {
                for (int r = 0; r < world; ++r) {
                    st_arena_v4(ctx.base[r] + a.off + v * 16ull, x);
                }
            }
        };
        if (nvls) {
            nvls_span<DT, OP>(ctx, a.off, sp.lo, sp.hi, a.scale, a.has_scale != 0, push);
        } else {
            reduce_span<DT, OP>(ctx, a.off, sp.lo, sp.hi, a.scale, a.has_scale != 0, push);
        }
    } else if (computes) {
        const Span sp = span_of(a.nvec, 1, 0, nb, b);
        for_each_entry<DT>(
            tab, a.ntable, single, sp.lo, sp.hi,
            [&](const GroupEntry &e, unsigned long long lo, unsigned long long hi) {
                if (e.dst == nullptr) { return; }
                const bool al = ptr_aligned16(e.dst);
                auto put = [&](unsigned long long v, const uint4 &x) {
                    store_user_vec<DT>(e.dst, user_f32, v - e.voff, e.count, al, x);
                };
                if (nvls) {
                    nvls_span<DT, OP>(ctx, a.off, lo, hi, a.scale, a.has_scale != 0, put);
                } else {
                    reduce_span<DT, OP>(ctx, a.off, lo, hi, a.scale, a.has_scale != 0, put);
                }
            });
    }

    if (do_reduce && (owner_algo || a.end_barrier)) {
        if (!peer_barrier(ctx, rank, &sync)) { return; }
    }

    // ---- unpack: own arena buffer -> user memory (two-shot / NVLS only)
    if ((phases & kPhaseUnpack) != 0 && owner_algo && computes &&
        (tab != nullptr || single.dst != nullptr)) {
        for (int s = 0; s < shards; ++s) {
            const Span sp = span_of(a.nvec, shards, s, nb, b);
            for_each_entry<DT>(tab, a.ntable, single, sp.lo, sp.hi,
                               [&](const GroupEntry &e, unsigned long long lo,
                                   unsigned long long hi) {
                                   if (e.dst == nullptr) { return; }
                                   const bool al = ptr_aligned16(e.dst);
                                   unsigned long long v = lo + threadIdx.x;
                                   for (; v + 3ull * kThreads < hi; v += 4ull * kThreads) {
                                       uint4 x[4];
#pragma unroll
                                       for (int u = 0; u < 4; ++u) {
                                           x[u] = ld_arena_v4(mine + (v + u * kThreads) * 16ull);
                                       }
#pragma unroll
                                       for (int u = 0; u < 4; ++u) {
                                           store_user_vec<DT>(e.dst, user_f32,
                                                              v + u * kThreads - e.voff, e.count,
                                                              al, x[u]);
                                       }
                                   }
                                   for (; v < hi; v += kThreads) {
                                       store_user_vec<DT>(e.dst, user_f32, v - e.voff, e.count,
                                                          al, ld_arena_v4(mine + v * 16ull));
                                   }
                               });
        }
    }

    if (do_reduce) { sync_end(ctx, rank, &sync); }
}

template <int DT, int OP>
int launch_one(const CommCtx &ctx, const AllReduceArgs &a, int blocks, int vranks,
               cudaStream_t stream)
{
    dim3 grid(blocks, vranks, 1);
    if (vranks > 1) {
        // Virtual ranks wait on one another inside one kernel: all blocks must
        // be resident at once, which only a cooperative launch guarantees.
        void *params[2] = {const_cast<CommCtx *>(&ctx), const_cast<AllReduceArgs *>(&a)};
        return static_cast<int>(cudaLaunchCooperativeKernel(
            reinterpret_cast<const void *>(&all_reduce_kernel<DT, OP>), grid, dim3(kThreads),
            params, 0, stream));
    }
    all_reduce_kernel<DT, OP><<<grid, kThreads, 0, stream>>>(ctx, a);
    return static_cast<int>(cudaGetLastError());
}

template <int DT>
int launch_ops(const CommCtx &ctx, const AllReduceArgs &a, int op, int blocks, int vranks,
               cudaStream_t stream)
{
    switch (op) {
    case OP_SUM:
        return launch_one<DT, OP_SUM>(ctx, a, blocks, vranks, stream);
    case OP_MIN:
        return launch_one<DT, OP_MIN>(ctx, a, blocks, vranks, stream);
    case OP_MAX:
        return launch_one<DT, OP_MAX>(ctx, a, blocks, vranks, stream);
    case OP_PROD:
        return launch_one<DT, OP_PROD>(ctx, a, blocks, vranks, stream);
    case OP_XOR:
        if constexpr (!Tr<DT>::is_float) {
            return launch_one<DT, OP_XOR>(ctx, a, blocks, vranks, stream);
        }
        return -1;
    }
    return -1;
}
}  // namespace stdml::collective::cuda
