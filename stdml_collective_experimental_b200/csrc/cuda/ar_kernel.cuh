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
//
// Two kernels share the pack / unpack code: all_reduce_kernel (register path:
// 16-byte peer loads or multimem) and all_reduce_tma_kernel, whose owner pulls
// every rank's tile into a shared-memory ring with bulk async copies (one
// elected thread issues them, an mbarrier per ring slot counts the bytes), so
// that far more remote bytes are in flight per SM than registers could hold.
// The bulk copies are plain (one destination CTA); they read peer memory over
// the same mappings as the vector loads.
#pragma once
#include "prims.cuh"

namespace stdml::collective::cuda
{
constexpr int kUnroll = 4;  // vectors per thread per iteration

struct Span {
    unsigned long long lo, hi;
};

// Spans start on multiples of this many vectors (512 bytes: what one warp moves
// with one 16-byte access per lane), so that no warp access of a span straddles
// a line it does not own; only the last span of a buffer may end elsewhere.
constexpr unsigned long long kSpanGranule = 32;

// Sub-range `b` of `nb` of shard `s` of `shards` of [0, nvec).
__host__ __device__ __forceinline__ Span span_of(unsigned long long nvec, int shards, int s, int nb,
                                        int b)
{
    const unsigned long long groups = (nvec + kSpanGranule - 1) / kSpanGranule;
    const unsigned long long s_lo = groups * static_cast<unsigned long long>(s) / shards;
    const unsigned long long s_hi = groups * static_cast<unsigned long long>(s + 1) / shards;
    const unsigned long long len = s_hi - s_lo;
    Span r;
    r.lo = (s_lo + len * static_cast<unsigned long long>(b) / nb) * kSpanGranule;
    r.hi = (s_lo + len * static_cast<unsigned long long>(b + 1) / nb) * kSpanGranule;
    r.lo = r.lo < nvec ? r.lo : nvec;
    r.hi = r.hi < nvec ? r.hi : nvec;
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

// Reduce vectors [lo, hi) of the buffers data[0..world) (rank r's buffer as
// mapped here) with peer loads (rank-ascending) and hand each result to
// store(v, value).
template <int DT, int OP, typename Store>
__device__ __forceinline__ void reduce_span(const CommCtx &ctx, char *const *data,
                                            unsigned long long lo, unsigned long long hi,
                                            double scale, bool has_scale, Store store)
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
                        x[u][j] = ld_arena_v4(data[r0 + j] + vu * 16ull);
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

// Same with the reduction done by the switch.  U vectors per thread and
// iteration; PIPE: the multimem.ld_reduce batch of the next iteration is issued
// before the multimem.st batch of the current one, so that a thread always has
// loads in flight while its stores drain.
template <int DT, int OP, int U, bool PIPE, typename Store>
__device__ __forceinline__ void nvls_loop(const CommCtx &ctx, unsigned long long off,
                                          unsigned long long lo, unsigned long long hi,
                                          double scale, bool has_scale, Store store)
{
    if constexpr (nvls_ok<DT, OP>()) {
        const unsigned long long step = static_cast<unsigned long long>(kThreads) * U;
        const char *mc = ctx.mc_base + off;
        unsigned long long v = lo + threadIdx.x;
        if constexpr (!PIPE) {
            for (; v < hi; v += step) {
                uint4 x[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const unsigned long long vu = v + static_cast<unsigned long long>(u) * kThreads;
                    if (vu < hi) { x[u] = mm_ld_reduce<DT, OP>(mc + vu * 16ull); }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const unsigned long long vu = v + static_cast<unsigned long long>(u) * kThreads;
                    if (vu < hi) { store(vu, has_scale ? scale_vec<DT>(x[u], scale) : x[u]); }
                }
            }
        } else {
            uint4 cur[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const unsigned long long vu = v + static_cast<unsigned long long>(u) * kThreads;
                if (vu < hi) { cur[u] = mm_ld_reduce<DT, OP>(mc + vu * 16ull); }
            }
            for (; v < hi; v += step) {
                uint4 nxt[U];
                const unsigned long long vn = v + step;
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const unsigned long long vu = vn + static_cast<unsigned long long>(u) * kThreads;
                    if (vu < hi) { nxt[u] = mm_ld_reduce<DT, OP>(mc + vu * 16ull); }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const unsigned long long vu = v + static_cast<unsigned long long>(u) * kThreads;
                    if (vu < hi) { store(vu, has_scale ? scale_vec<DT>(cur[u], scale) : cur[u]); }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) { cur[u] = nxt[u]; }
            }
        }
    }
}

// NV selects the loop at compile time: each variant is its own kernel
// instantiation, so the registers of the widest one are not charged to the rest.
template <int DT, int OP, int NV, typename Store>
__device__ __forceinline__ void nvls_span(const CommCtx &ctx, unsigned long long off,
                                          unsigned long long lo, unsigned long long hi,
                                          double scale, bool has_scale, Store store)
{
    if constexpr (NV == kNvlsPipe4) {
        nvls_loop<DT, OP, 4, true>(ctx, off, lo, hi, scale, has_scale, store);
    } else if constexpr (NV == kNvlsPipe8) {
        nvls_loop<DT, OP, 8, true>(ctx, off, lo, hi, scale, has_scale, store);
    } else if constexpr (NV == kNvlsPlain8) {
        nvls_loop<DT, OP, 8, false>(ctx, off, lo, hi, scale, has_scale, store);
    } else {
        nvls_loop<DT, OP, 4, false>(ctx, off, lo, hi, scale, has_scale, store);
    }
}

// ---- pack: user memory -> own arena buffer (the parts peers' block b read)
// span_at(s): the part of shard s that THIS block index serves.  The barriers
// pair blocks with the same index across ranks, so a block must pack exactly
// what the peers' block of the same index will read, and unpack exactly what
// they wrote.
template <int DT, typename SpanAt>
__device__ __forceinline__ void pack_phase(const AllReduceArgs &a, const GroupEntry *tab,
                                           const GroupEntry &single, char *mine, int shards,
                                           bool user_f32, SpanAt span_at)
{
    for (int s = 0; s < shards; ++s) {
        const Span sp = span_at(s);
        for_each_entry<DT>(
            tab, a.ntable, single, sp.lo, sp.hi,
            [&](const GroupEntry &e, unsigned long long lo, unsigned long long hi) {
                if (e.src == nullptr) { return; }
                const bool al = ptr_aligned16(e.src);
                unsigned long long v = lo + threadIdx.x;
                for (; v + 3ull * kThreads < hi; v += 4ull * kThreads) {
                    uint4 x[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        x[u] = load_user_vec<DT>(e.src, user_f32, v + u * kThreads - e.voff,
                                                 e.count, al);
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        st_arena_v4(mine + (v + u * kThreads) * 16ull, x[u]);
                    }
                }
                for (; v < hi; v += kThreads) {
                    st_arena_v4(mine + v * 16ull,
                                load_user_vec<DT>(e.src, user_f32, v - e.voff, e.count, al));
                }
            });
    }
}

// ---- unpack: own arena buffer -> user memory (owner algorithms only)
template <int DT, typename SpanAt>
__device__ __forceinline__ void unpack_phase(const AllReduceArgs &a, const GroupEntry *tab,
                                             const GroupEntry &single, const char *mine,
                                             int shards, bool user_f32, SpanAt span_at)
{
    for (int s = 0; s < shards; ++s) {
        const Span sp = span_at(s);
        for_each_entry<DT>(
            tab, a.ntable, single, sp.lo, sp.hi,
            [&](const GroupEntry &e, unsigned long long lo, unsigned long long hi) {
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
                        store_user_vec<DT>(e.dst, user_f32, v + u * kThreads - e.voff, e.count, al,
                                           x[u]);
                    }
                }
                for (; v < hi; v += kThreads) {
                    store_user_vec<DT>(e.dst, user_f32, v - e.voff, e.count, al,
                                       ld_arena_v4(mine + v * 16ull));
                }
            });
    }
}

// Debug builds of a call (AllReduceArgs::debug_checks): the kernel looks at its
// own arguments before it touches memory and reports kStatusBadArgs instead of
// running.  Checked: the symmetric buffer lies inside the data region and is
// 16-byte aligned, the table is sorted, starts at 0 and stays inside the
// buffer, the ring geometry fits the shared memory it was given.
// The range rules of the in-kernel checks, as plain functions (also run on the
// CPU by the tests): entry i of a table ends inside the buffer and before the
// next entry starts; a buffer offset is 16-byte aligned and past the signal pad
// (or 0 for registered buffers, which have no arena offset).
template <int DT>
__host__ __device__ __forceinline__ bool table_entry_in_range(const GroupEntry *tab, int i, int n,
                                                           unsigned long long nvec)
{
    const unsigned long long end = tab[i].voff + entry_nvec<DT>(tab[i].count);
    return end <= nvec && (i + 1 >= n || tab[i + 1].voff >= end);
}

__host__ __device__ __forceinline__ bool buffer_offset_ok(unsigned long long off)
{
    return off % 16ull == 0ull && (off >= kDataOffset || off == 0ull);
}

template <int DT>
__device__ __forceinline__ bool args_look_sane(const CommCtx &ctx, const AllReduceArgs &a,
                                               const GroupEntry *tab, unsigned int dyn_smem)
{
    bool ok = buffer_offset_ok(a.off) && ctx.world >= 1 && ctx.world <= kMaxRanks && a.algo >= 0 && a.algo < kAlgoCount &&
              a.root < ctx.world && a.nvec > 0;
    for (int r = 0; ok && r < ctx.world; ++r) {
        // every rank's buffer: mapped, 16-byte aligned, and (arena buffers) past the pad
        const unsigned long long p = reinterpret_cast<unsigned long long>(a.data[r]);
        const unsigned long long q = reinterpret_cast<unsigned long long>(a.push[r]);
        ok = p != 0ull && (p & 15ull) == 0ull && (q & 15ull) == 0ull &&
             (a.off == 0ull || a.data[r] == ctx.base[r] + a.off);
    }
    if (ok && tab != nullptr) {
        ok = a.ntable > 0 && tab[0].voff == 0;
        for (int i = threadIdx.x; ok && i < a.ntable; i += kThreads) {
            ok = table_entry_in_range<DT>(tab, i, a.ntable, a.nvec);
        }
    }
    if (ok && a.algo == kAlgoTwoShotTma) {
        ok = a.tma_stages >= 1 && a.tma_stages <= kTmaMaxStages && a.tma_tile_vec >= 1 &&
             static_cast<unsigned long long>(a.tma_stages) * ctx.world * a.tma_tile_vec * 16ull <=
                 dyn_smem;
    }
    return __syncthreads_and(ok ? 1 : 0) != 0;
}

static __device__ __noinline__ void report_bad_args(const CommCtx &ctx, int rank)
{
    StatusBlock *st = ctx.status;
    if (st == nullptr || threadIdx.x != 0) { return; }
    volatile StatusBlock *v = st;
    if (v->code == kStatusOk) {
        v->rank = rank;
        v->block = static_cast<int>(blockIdx.x);
        v->peer = -1;
        __threadfence_system();
        v->code = kStatusBadArgs;
        __threadfence_system();
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
    // the other owner algorithms (NVLS, bulk-copy two-shot) run in owner_kernel
    const bool owner_algo = (algo == kAlgoTwoShot);
    const bool nvls = (algo == kAlgoNvlsOneShot);
    const int shards = owner_algo ? world : 1;
    const bool user_f32 = Tr<DT>::is_half && a.user_dtype == DT_F32;
    const bool computes = (a.root < 0 || a.root == rank);
    const GroupEntry *tab = a.table[vr];

    if (a.debug_checks != 0 && !args_look_sane<DT>(ctx, a, tab, 0u)) {
        report_bad_args(ctx, rank);
        return;
    }

    // A launch may run only some phases: large staged messages are cut into
    // chunks whose pack / reduce / unpack run as separate launches on three
    // streams, so that the HBM copies of one chunk overlap the NVLink phase of
    // another.  Only the reduce phase synchronises with peers.
    const int phases = a.phases;
    const bool do_reduce = (phases & kPhaseReduce) != 0;
    if (do_reduce) { sync_begin(ctx, rank, &sync); }

    char *mine = a.data[rank];
    GroupEntry single;
    single.src = a.src[vr];
    single.dst = a.dst[vr];
    single.voff = 0;
    single.count = a.count;

    if ((phases & kPhasePack) != 0 && (tab != nullptr || single.src != nullptr)) {
        pack_phase<DT>(a, tab, single, mine, shards, user_f32,
                       [&](int s) { return span_of(a.nvec, shards, s, nb, b); });
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
            if (a.root >= 0) {
                st_arena_v4(a.push[a.root] + v * 16ull, x);
            } else {
                for (int r = 0; r < world; ++r) {
                    st_arena_v4(a.push[r] + v * 16ull, x);
                }
            }
        };
        reduce_span<DT, OP>(ctx, a.data, sp.lo, sp.hi, a.scale, a.has_scale != 0, push);
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
                    nvls_span<DT, OP, kNvlsPlain4>(ctx, a.off, lo, hi, a.scale, a.has_scale != 0,
                                                   put);
                } else {
                    reduce_span<DT, OP>(ctx, a.data, lo, hi, a.scale, a.has_scale != 0, put);
                }
            });
    }

    if (do_reduce && (owner_algo || a.end_barrier)) {
        if (!peer_barrier(ctx, rank, &sync)) { return; }
    }

    if ((phases & kPhaseUnpack) != 0 && owner_algo && computes &&
        (tab != nullptr || single.dst != nullptr)) {
        unpack_phase<DT>(a, tab, single, a.push[rank], shards, user_f32,
                         [&](int s) { return span_of(a.nvec, shards, s, nb, b); });
    }

    if (do_reduce) { sync_end(ctx, rank, &sync); }
}

// ------------------------------------------------------------------ bulk pulls
__device__ __forceinline__ uint32_t smem_addr(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

// One bulk asynchronous copy global -> shared memory of this CTA; completion
// is counted in bytes on `bar`.  Addresses and size are multiples of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void *src, uint32_t bytes,
                                          uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
            "r"(dst_smem),
        "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Bounded: false when the bytes did not arrive within the context's limits.
__device__ __forceinline__ bool mbar_wait(const CommCtx &ctx, uint32_t bar, uint32_t parity,
                                          unsigned long long limit_ns)
{
    unsigned int spins = 0;
    unsigned long long t0 = 0;
    while (!mbar_try_wait(bar, parity)) {
        ++spins;
        if ((spins & 63u) == 0u) {
            const unsigned long long now = global_ns();
            if (t0 == 0) { t0 = now; }
            if (now - t0 > limit_ns || spins >= ctx.max_spins) { return false; }
        }
    }
    return true;
}

// Orders this thread's earlier generic-proxy accesses (its acquire of the
// peers' flags, its own packed data) against the bulk copies it issues next.
__device__ __forceinline__ void fence_async_proxy()
{
    asm volatile("fence.proxy.async;" ::: "memory");
}

// The owner's reduce of span [lo, hi) with bulk pulls.  Ring slot s holds tile
// t (t % stages == s): `world` pieces of tile_vec vectors, rank-major.  Thread
// 0 issues the copies and every thread waits on the slot's mbarrier; one
// __syncthreads per tile both collects the outcome of that wait and frees the
// slot for its next tile.  Returns false after a wait that ran out.
template <int DT, int OP, typename Push>
__device__ __forceinline__ bool tma_reduce_span(const CommCtx &ctx, const AllReduceArgs &a,
                                                int rank, unsigned long long lo,
                                                unsigned long long hi, unsigned char *ring,
                                                unsigned long long *bars, BlockSync *sync,
                                                Push push)
{
    const int world = ctx.world;
    const int stages = a.tma_stages;
    const unsigned int tile_vec = a.tma_tile_vec;
    const unsigned int tile_bytes = tile_vec * 16u;
    const unsigned long long total = hi > lo ? hi - lo : 0ull;
    const unsigned long long ntiles = (total + tile_vec - 1) / tile_vec;
    const uint32_t ring_s = smem_addr(ring);
    const uint32_t bars_s = smem_addr(bars);

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) { mbar_init(bars_s + 8u * s, 1u); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_proxy();
    }
    __syncthreads();

    auto issue = [&](unsigned long long t) {
        const int s = static_cast<int>(t % static_cast<unsigned long long>(stages));
        const unsigned long long v0 = lo + t * tile_vec;
        const unsigned long long left = hi - v0;
        const uint32_t bytes = static_cast<uint32_t>(left < tile_vec ? left : tile_vec) * 16u;
        const uint32_t bar = bars_s + 8u * s;
        mbar_expect_tx(bar, bytes * static_cast<uint32_t>(world));
        for (int i = 0; i < world; ++i) {
            // start with the next rank, so that the owners do not all pull from
            // the same GPU at the same moment
            const int r = (rank + 1 + i) % world;
            bulk_load(ring_s + (static_cast<uint32_t>(s) * world + r) * tile_bytes,
                      a.data[r] + v0 * 16ull, bytes, bar);
        }
    };
    if (threadIdx.x == 0) {
        for (unsigned long long t = 0; t < ntiles && t < static_cast<unsigned long long>(stages);
             ++t) {
            issue(t);
        }
    }

    const double scale = a.scale;
    const bool has_scale = a.has_scale != 0;
    unsigned long long in_flight_from = 0;  // first tile whose copies may still be running
    bool ok = true;
    for (unsigned long long t = 0; t < ntiles; ++t) {
        const int s = static_cast<int>(t % static_cast<unsigned long long>(stages));
        const uint32_t parity = static_cast<uint32_t>((t / stages) & 1ull);
        const bool got = mbar_wait(ctx, bars_s + 8u * s, parity, ctx.timeout_ns);
        if (got) {
            const unsigned long long v0 = lo + t * tile_vec;
            const unsigned long long left = hi - v0;
            const unsigned int nv = static_cast<unsigned int>(left < tile_vec ? left : tile_vec);
            const uint4 *slot = reinterpret_cast<const uint4 *>(ring + static_cast<size_t>(s) *
                                                                           world * tile_bytes);
            for (unsigned int i = threadIdx.x; i < nv; i += kThreads) {
                Accum<DT> acc;
                for (int r0 = 0; r0 < world; r0 += 4) {
                    uint4 x[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (r0 + j < world) { x[j] = slot[static_cast<size_t>(r0 + j) * tile_vec + i]; }
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (r0 + j < world) {
                            if (r0 + j == 0) {
                                acc.init(x[j]);
                            } else {
                                acc.template add<OP>(x[j]);
                            }
                        }
                    }
                }
                push(v0 + i, acc.finish(scale, has_scale));
            }
        }
        // everybody has read slot s (or given up): it may be refilled
        if (__syncthreads_and(got ? 1 : 0) == 0) {
            ok = false;
            in_flight_from = t;
            break;
        }
        if (threadIdx.x == 0 && t + stages < ntiles) { issue(t + stages); }
    }
    if (!ok) {
        if (threadIdx.x == 0) {
            report_timeout(ctx, rank, -1, 0u, 0u, 64 + sync->phase);
            *reinterpret_cast<volatile int *>(&sync->failed) = 1;
            // copies already issued still write into this CTA's shared memory: give
            // them one more (bounded) chance to land before the CTA goes away
            for (unsigned long long t = in_flight_from;
                 t < ntiles && t < in_flight_from + static_cast<unsigned long long>(stages); ++t) {
                const int s = static_cast<int>(t % static_cast<unsigned long long>(stages));
                (void)mbar_wait(ctx, bars_s + 8u * s, static_cast<uint32_t>((t / stages) & 1ull),
                                ctx.timeout_ns / 4);
            }
        }
        __syncthreads();
    }
    return ok;
}

// The owner kernel: pack -> barrier -> rank r reduces shard r and writes the
// result into every rank's buffer -> barrier -> unpack.  MODE picks how the
// owner gets at the operands: kOwnerTma pulls tiles with bulk copies (any
// dtype and op, rank-ascending order); the other modes are the NVLS loops
// (kNvls*: the switch reduces, multimem.st spreads the result).
constexpr int kOwnerTma = 16;
constexpr int kOwnerHybrid = 17;  // NVLS (pipelined, 4 vectors) on one part, peer loads on the rest

template <int DT, int OP, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
    owner_kernel(const __grid_constant__ CommCtx ctx, const __grid_constant__ AllReduceArgs a,
                 unsigned int dyn_smem)
{
    extern __shared__ __align__(128) unsigned char ring[];
    __shared__ BlockSync sync;
    __shared__ __align__(8) unsigned long long bars[kTmaMaxStages];
    const int vr = static_cast<int>(blockIdx.y);
    const int rank = ctx.rank + vr;
    const int world = ctx.world;
    const int nb = static_cast<int>(gridDim.x);
    const int b = static_cast<int>(blockIdx.x);
    const bool user_f32 = Tr<DT>::is_half && a.user_dtype == DT_F32;
    const bool computes = (a.root < 0 || a.root == rank);
    const GroupEntry *tab = a.table[vr];

    if (a.debug_checks != 0 && !args_look_sane<DT>(ctx, a, tab, dyn_smem)) {
        report_bad_args(ctx, rank);
        return;
    }

    const int phases = a.phases;
    const bool do_reduce = (phases & kPhaseReduce) != 0;
    if (do_reduce) { sync_begin(ctx, rank, &sync); }

    char *mine = a.data[rank];
    GroupEntry single;
    single.src = a.src[vr];
    single.dst = a.dst[vr];
    single.voff = 0;
    single.count = a.count;

    // the part of shard s that blocks with this index serve (see pack_phase)
    auto span_at = [&](int s) {
        if constexpr (MODE == kOwnerHybrid) {
            const int nbn = a.hybrid_nvls_blocks;
            const unsigned long long n1 = a.hybrid_split_vec;
            if (b < nbn) { return span_of(n1, world, s, nbn, b); }
            Span t = span_of(a.nvec - n1, world, s, nb - nbn, b - nbn);
            t.lo += n1;
            t.hi += n1;
            return t;
        } else {
            return span_of(a.nvec, world, s, nb, b);
        }
    };

    if ((phases & kPhasePack) != 0 && (tab != nullptr || single.src != nullptr)) {
        pack_phase<DT>(a, tab, single, mine, world, user_f32, span_at);
        // the packed data is read by bulk copies (async proxy) of the peers
        if constexpr (MODE == kOwnerTma) { fence_async_proxy(); }
    }

    if (do_reduce) {
        if (!peer_barrier(ctx, rank, &sync)) { return; }
        const Span sp = span_of(a.nvec, world, rank, nb, b);
        if constexpr (MODE == kOwnerTma) {
            auto push = [&](unsigned long long v, const uint4 &x) {
                if (a.root >= 0) {
                    st_arena_v4(a.push[a.root] + v * 16ull, x);
                } else {
                    for (int i = 0; i < world; ++i) {
                        const int r = (rank + i) % world;
                        st_arena_v4(a.push[r] + v * 16ull, x);
                    }
                }
            };
            if (!tma_reduce_span<DT, OP>(ctx, a, rank, sp.lo, sp.hi, ring, bars, &sync, push)) {
                return;
            }
        } else if constexpr (MODE == kOwnerHybrid) {
            // vectors [0, n1): the switch reduces and replicates; [n1, nvec): this
            // rank loads its shard from every peer and stores the result to every
            // peer.  Different CTAs, one launch, one pair of barriers.
            const Span mine_sp = span_at(rank);
            if (b < a.hybrid_nvls_blocks) {
                auto push = [&](unsigned long long v, const uint4 &x) {
                    mm_st_v4(ctx.mc_base + a.off + v * 16ull, x);
                };
                nvls_span<DT, OP, kNvlsPipe4>(ctx, a.off, mine_sp.lo, mine_sp.hi, a.scale,
                                              a.has_scale != 0, push);
            } else {
                auto push = [&](unsigned long long v, const uint4 &x) {
                    for (int i = 0; i < world; ++i) {
                        const int r = (rank + i) % world;
                        st_arena_v4(a.push[r] + v * 16ull, x);
                    }
                };
                reduce_span<DT, OP>(ctx, a.data, mine_sp.lo, mine_sp.hi, a.scale,
                                    a.has_scale != 0, push);
            }
        } else {
            auto push = [&](unsigned long long v, const uint4 &x) {
                if (a.root >= 0) {
                    st_arena_v4(a.push[a.root] + v * 16ull, x);
                } else {
                    mm_st_v4(ctx.mc_base + a.off + v * 16ull, x);
                }
            };
            nvls_span<DT, OP, MODE>(ctx, a.off, sp.lo, sp.hi, a.scale, a.has_scale != 0, push);
        }
        if (!peer_barrier(ctx, rank, &sync)) { return; }
    }

    if ((phases & kPhaseUnpack) != 0 && computes && (tab != nullptr || single.dst != nullptr)) {
        unpack_phase<DT>(a, tab, single, a.push[rank], world, user_f32, span_at);
    }

    if (do_reduce) { sync_end(ctx, rank, &sync); }
}

template <int DT, int OP, int MODE>
int launch_owner(const CommCtx &ctx, const AllReduceArgs &a, dim3 grid, int vranks,
                 unsigned int smem, cudaStream_t stream)
{
    if (smem > (48u << 10)) {
        // the opt-in to more than 48 KB is per function and per device
        static bool opted_in[64] = {};
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { dev = 0; }
        if (!opted_in[dev]) {
            const cudaError_t e = cudaFuncSetAttribute(
                reinterpret_cast<const void *>(&owner_kernel<DT, OP, MODE>),
                cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kTmaSmemBudget));
            if (e != cudaSuccess) { return static_cast<int>(e); }
            opted_in[dev] = true;
        }
    }
    unsigned int dyn = smem;
    if (vranks > 1) {
        // Virtual ranks wait on one another inside one kernel: all blocks must
        // be resident at once, which only a cooperative launch guarantees.
        void *params[3] = {const_cast<CommCtx *>(&ctx), const_cast<AllReduceArgs *>(&a), &dyn};
        return static_cast<int>(cudaLaunchCooperativeKernel(
            reinterpret_cast<const void *>(&owner_kernel<DT, OP, MODE>), grid, dim3(kThreads),
            params, smem, stream));
    }
    owner_kernel<DT, OP, MODE><<<grid, kThreads, smem, stream>>>(ctx, a, dyn);
    return static_cast<int>(cudaGetLastError());
}

template <int DT, int OP>
int launch_one(const CommCtx &ctx, const AllReduceArgs &a, int blocks, int vranks,
               cudaStream_t stream)
{
    dim3 grid(blocks, vranks, 1);
    if (a.algo == kAlgoTwoShotTma) {
        const unsigned int smem = static_cast<unsigned int>(a.tma_stages) *
                                  static_cast<unsigned int>(ctx.world) * a.tma_tile_vec * 16u;
        return launch_owner<DT, OP, kOwnerTma>(ctx, a, grid, vranks, smem, stream);
    }
    if (a.algo == kAlgoNvlsHybrid) {
        if constexpr (nvls_ok<DT, OP>()) {
            return launch_owner<DT, OP, kOwnerHybrid>(ctx, a, grid, vranks, 0u, stream);
        }
        return -1;
    }
    if (a.algo == kAlgoNvls) {
        if constexpr (nvls_ok<DT, OP>()) {
            switch (a.nvls_variant) {
            case kNvlsPipe4:
                return launch_owner<DT, OP, kNvlsPipe4>(ctx, a, grid, vranks, 0u, stream);
            case kNvlsPipe8:
                return launch_owner<DT, OP, kNvlsPipe8>(ctx, a, grid, vranks, 0u, stream);
            case kNvlsPlain8:
                return launch_owner<DT, OP, kNvlsPlain8>(ctx, a, grid, vranks, 0u, stream);
            default:
                return launch_owner<DT, OP, kNvlsPlain4>(ctx, a, grid, vranks, 0u, stream);
            }
        }
        return -1;
    }
    if (vranks > 1) {
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
