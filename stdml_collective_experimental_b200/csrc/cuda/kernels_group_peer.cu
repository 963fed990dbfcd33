// Fused group all-reduce on registered tensors: the two-shot of ar_kernel.cuh
// walking a table of per-rank tensor pointers instead of one flat buffer.  The
// owner of a span loads every rank's piece of every tensor that intersects it
// (rank-ascending reduce in registers, scale fused) and stores the result into
// every rank's output tensor.  Nothing is packed or unpacked, so loose gradient
// tensors cost one launch and no extra HBM pass.  Two ways of loading: 16-byte
// peer loads (small sets), or bulk asynchronous copies into a shared-memory
// ring whose tiles run on across tensor boundaries, so that the copy pipeline
// never drains between tensors (BULK).
//
// The reference's counterpart is its per-tensor thread pool
// (src/stdml/collective/session.cpp:83-97 there).
#include "ar_kernel.cuh"
#include "group_walk.cuh"

namespace stdml::collective::cuda
{
namespace
{
// The owner's reduce of a span with bulk pulls.  Ring slot k % stages holds the
// k-th tile of the walk: `world` pieces of tile_vec vectors, rank-major.  Thread
// 0 issues the copies `stages` tiles ahead; every thread waits on the slot's
// mbarrier; one __syncthreads per tile collects the outcome of that wait and
// frees the slot.  Returns false after a wait that ran out.
template <int DT, int OP>
__device__ __forceinline__ bool bulk_walk(const CommCtx &ctx, const GroupPeerArgs &a, int rank,
                                          const Span &sp, unsigned char *ring,
                                          unsigned long long *bars, BlockSync *sync)
{
    constexpr unsigned long long N = lanes_of<DT>();
    const int world = ctx.world;
    const int stages = a.tma_stages;
    const unsigned int tile_vec = a.tma_tile_vec;
    const unsigned int tile_bytes = tile_vec * 16u;
    const uint32_t ring_s = smem_addr(ring);
    const uint32_t bars_s = smem_addr(bars);
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) { mbar_init(bars_s + 8u * s, 1u); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_proxy();
    }
    __syncthreads();

    TileCursor ahead, here;
    ahead.i = here.i = find_peer_entry(a.table, a.ntable, sp.lo);
    ahead.v = ahead.end = here.v = here.end = 0;
    if (!cursor_enter<N>(a, sp, &here)) { return true; }  // no whole vector in this span
    ahead = here;

    unsigned long long issued = 0;  // thread 0 only
    auto issue = [&]() {
        Tile t;
        if (!cursor_next<N>(a, sp, &ahead, tile_vec, &t)) { return; }
        const int s = static_cast<int>(issued % static_cast<unsigned long long>(stages));
        const uint32_t bytes = t.nv * 16u;
        const uint32_t bar = bars_s + 8u * s;
        mbar_expect_tx(bar, bytes * static_cast<uint32_t>(world));
        for (int i = 0; i < world; ++i) {
            // start with the next rank, so that the owners do not all pull from
            // the same GPU at the same moment
            const int r = (rank + 1 + i) % world;
            bulk_load(ring_s + (static_cast<uint32_t>(s) * world + r) * tile_bytes,
                      t.e->in[r] + t.v0 * 16ull, bytes, bar);
        }
        ++issued;
    };
    if (threadIdx.x == 0) {
        for (int k = 0; k < stages; ++k) { issue(); }
    }

    const bool has_scale = a.has_scale != 0;
    unsigned long long done = 0;
    bool ok = true;
    Tile t;
    while (cursor_next<N>(a, sp, &here, tile_vec, &t)) {
        const int s = static_cast<int>(done % static_cast<unsigned long long>(stages));
        const uint32_t parity = static_cast<uint32_t>((done / stages) & 1ull);
        const bool got = mbar_wait(ctx, bars_s + 8u * s, parity, ctx.timeout_ns);
        if (got) {
            const uint4 *slot =
                reinterpret_cast<const uint4 *>(ring + static_cast<size_t>(s) * world * tile_bytes);
            char *outs[kMaxRanks];
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r) {
                outs[r] = r < world ? t.e->out[r] + t.v0 * 16ull : nullptr;
            }
            for (unsigned int i = threadIdx.x; i < t.nv; i += kThreads) {
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
                const uint4 res = acc.finish(a.scale, has_scale);
#pragma unroll
                for (int r = 0; r < kMaxRanks; ++r) {
                    if (r < world) { st_arena_v4(outs[r] + i * 16ull, res); }
                }
            }
        }
        // everybody has read slot s (or given up): it may be refilled
        if (__syncthreads_and(got ? 1 : 0) == 0) {
            ok = false;
            break;
        }
        ++done;
        if (threadIdx.x == 0) { issue(); }
    }
    if (!ok) {
        if (threadIdx.x == 0) {
            report_timeout(ctx, rank, -1, 0u, 0u, 64 + sync->phase);
            *reinterpret_cast<volatile int *>(&sync->failed) = 1;
            // copies already issued still write into this CTA's shared memory: give
            // them one more (bounded) chance to land before the CTA goes away
            for (unsigned long long k = done; k < issued; ++k) {
                const int s = static_cast<int>(k % static_cast<unsigned long long>(stages));
                (void)mbar_wait(ctx, bars_s + 8u * s, static_cast<uint32_t>((k / stages) & 1ull),
                                ctx.timeout_ns / 4);
            }
        }
        __syncthreads();
    }
    return ok;
}

template <int DT, int OP, bool BULK>
__global__ void __launch_bounds__(kThreads)
    group_peer_kernel(const __grid_constant__ CommCtx ctx, const __grid_constant__ GroupPeerArgs a)
{
    using S = typename Tr<DT>::storage;
    constexpr unsigned long long N = lanes_of<DT>();
    extern __shared__ __align__(128) unsigned char ring[];
    __shared__ BlockSync sync;
    __shared__ __align__(8) unsigned long long bars[kTmaMaxStages];
    const int rank = ctx.rank + static_cast<int>(blockIdx.y);
    const int world = ctx.world;
    const int nb = static_cast<int>(gridDim.x);
    const int b = static_cast<int>(blockIdx.x);
    sync_begin(ctx, rank, &sync);
    // every rank is here: its inputs are final, its outputs may be written
    if (!peer_barrier(ctx, rank, &sync)) { return; }

    const Span sp = span_of(a.nvec, world, rank, nb, b);
    if constexpr (BULK) {
        if (sp.lo < sp.hi && !bulk_walk<DT, OP>(ctx, a, rank, sp, ring, bars, &sync)) { return; }
    }
    if (sp.lo < sp.hi) {
        for (int i = find_peer_entry(a.table, a.ntable, sp.lo); i < a.ntable; ++i) {
            const PeerEntry *e = &a.table[i];
            const unsigned long long voff = e->voff;
            if (voff >= sp.hi) { break; }
            const unsigned long long count = e->count;
            const unsigned long long full = count / N;            // whole vectors
            const unsigned long long nv = (count + N - 1) / N;    // with the ragged one
            const unsigned long long lo = (sp.lo > voff ? sp.lo : voff) - voff;
            unsigned long long hi = (sp.hi < voff + nv ? sp.hi : voff + nv);
            if (hi <= voff + lo) { continue; }
            hi -= voff;
            const unsigned long long hi_full = hi < full ? hi : full;
            if (!BULK && lo < hi_full) {
                reduce_span<DT, OP>(ctx, e->in, lo, hi_full, a.scale, a.has_scale != 0,
                                    [&](unsigned long long v, const uint4 &x) {
                                        for (int k = 0; k < world; ++k) {
                                            const int r = (rank + k) % world;
                                            st_arena_v4(e->out[r] + v * 16ull, x);
                                        }
                                    });
            }
            // the ragged last vector of a tensor: element by element, one thread
            if (full < nv && lo <= full && full < hi && threadIdx.x == 0) {
                const unsigned long long e0 = full * N;
                for (unsigned long long j = e0; j < count; ++j) {
                    typename Tr<DT>::acc acc = Tr<DT>::widen(
                        *reinterpret_cast<const volatile S *>(e->in[0] + j * sizeof(S)));
                    for (int r = 1; r < world; ++r) {
                        acc = combine<OP>(acc, Tr<DT>::widen(*reinterpret_cast<const volatile S *>(
                                                   e->in[r] + j * sizeof(S))));
                    }
                    if constexpr (Tr<DT>::is_float) {
                        if (a.has_scale != 0) { acc = acc * static_cast<typename Tr<DT>::acc>(a.scale); }
                    }
                    const S res = Tr<DT>::narrow(acc);
                    for (int r = 0; r < world; ++r) {
                        *reinterpret_cast<volatile S *>(e->out[r] + j * sizeof(S)) = res;
                    }
                }
            }
        }
    }
    if (!peer_barrier(ctx, rank, &sync)) { return; }
    sync_end(ctx, rank, &sync);
}

template <int DT, int OP, bool BULK>
int launch_gp_mode(const CommCtx &ctx, const GroupPeerArgs &a, dim3 grid, int vranks,
                   unsigned int smem, cudaStream_t s)
{
    if (smem > (48u << 10)) {
        // the opt-in to more than 48 KB is per function and per device
        static bool opted_in[64] = {};
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { dev = 0; }
        if (!opted_in[dev]) {
            const cudaError_t e = cudaFuncSetAttribute(
                reinterpret_cast<const void *>(&group_peer_kernel<DT, OP, BULK>),
                cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kTmaSmemBudget));
            if (e != cudaSuccess) { return static_cast<int>(e); }
            opted_in[dev] = true;
        }
    }
    if (vranks > 1) {
        void *params[2] = {const_cast<CommCtx *>(&ctx), const_cast<GroupPeerArgs *>(&a)};
        return static_cast<int>(cudaLaunchCooperativeKernel(
            reinterpret_cast<const void *>(&group_peer_kernel<DT, OP, BULK>), grid, dim3(kThreads),
            params, smem, s));
    }
    group_peer_kernel<DT, OP, BULK><<<grid, kThreads, smem, s>>>(ctx, a);
    return static_cast<int>(cudaGetLastError());
}

template <int DT, int OP>
int launch_gp(const CommCtx &ctx, const GroupPeerArgs &a, int blocks, int vranks, cudaStream_t s)
{
    dim3 grid(blocks, vranks, 1);
    if (a.tma_stages > 0) {
        const unsigned int smem = static_cast<unsigned int>(a.tma_stages) *
                                  static_cast<unsigned int>(ctx.world) * a.tma_tile_vec * 16u;
        return launch_gp_mode<DT, OP, true>(ctx, a, grid, vranks, smem, s);
    }
    return launch_gp_mode<DT, OP, false>(ctx, a, grid, vranks, 0u, s);
}

template <int DT>
int launch_gp_ops(const CommCtx &ctx, const GroupPeerArgs &a, int op, int blocks, int vranks,
                  cudaStream_t s)
{
    switch (op) {
    case OP_SUM:
        return launch_gp<DT, OP_SUM>(ctx, a, blocks, vranks, s);
    case OP_MIN:
        return launch_gp<DT, OP_MIN>(ctx, a, blocks, vranks, s);
    case OP_MAX:
        return launch_gp<DT, OP_MAX>(ctx, a, blocks, vranks, s);
    case OP_PROD:
        return launch_gp<DT, OP_PROD>(ctx, a, blocks, vranks, s);
    case OP_XOR:
        if constexpr (!Tr<DT>::is_float) { return launch_gp<DT, OP_XOR>(ctx, a, blocks, vranks, s); }
        return -1;
    }
    return -1;
}
}  // namespace

int launch_group_peer(const CommCtx &ctx, const GroupPeerArgs &a, int dt, int op, int blocks,
                      int vranks, void *stream)
{
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dt) {
    case DT_I8:
        return launch_gp_ops<DT_I8>(ctx, a, op, blocks, vranks, s);
    case DT_I16:
        return launch_gp_ops<DT_I16>(ctx, a, op, blocks, vranks, s);
    case DT_I32:
        return launch_gp_ops<DT_I32>(ctx, a, op, blocks, vranks, s);
    case DT_I64:
        return launch_gp_ops<DT_I64>(ctx, a, op, blocks, vranks, s);
    case DT_U8:
        return launch_gp_ops<DT_U8>(ctx, a, op, blocks, vranks, s);
    case DT_U16:
        return launch_gp_ops<DT_U16>(ctx, a, op, blocks, vranks, s);
    case DT_U32:
        return launch_gp_ops<DT_U32>(ctx, a, op, blocks, vranks, s);
    case DT_U64:
        return launch_gp_ops<DT_U64>(ctx, a, op, blocks, vranks, s);
    case DT_BF16:
        return launch_gp_ops<DT_BF16>(ctx, a, op, blocks, vranks, s);
    case DT_F16:
        return launch_gp_ops<DT_F16>(ctx, a, op, blocks, vranks, s);
    case DT_F32:
        return launch_gp_ops<DT_F32>(ctx, a, op, blocks, vranks, s);
    case DT_F64:
        return launch_gp_ops<DT_F64>(ctx, a, op, blocks, vranks, s);
    }
    return -1;
}
}  // namespace stdml::collective::cuda
