// Device primitives of the NVLink data plane: system-scope flag accesses,
// 16-byte peer loads/stores, NVLS multimem wrappers, the bounded cross-rank
// block barrier, and per-dtype vector arithmetic.
//
// Remote data is always fetched by the CTA itself with plain vector loads over
// the peer mapping or with multimem instructions through the switch; there is
// no bulk/TMA copy in this data plane.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <type_traits>

#include "comm.cuh"

namespace stdml::collective::cuda
{
// dtype / op enumerator values (must match stdml/bits/collective/dtype.hpp)
enum : int { DT_I8, DT_I16, DT_I32, DT_I64, DT_U8, DT_U16, DT_U32, DT_U64, DT_BF16, DT_F16, DT_F32, DT_F64 };
enum : int { OP_SUM, OP_MIN, OP_MAX, OP_PROD, OP_XOR };

// ---------------------------------------------------------------- memory ops
__device__ __forceinline__ void st_release_sys_u32(uint32_t *p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Coherent 16-byte load (bypasses L1): used for every read of arena memory,
// local or remote, because peers write it while the kernel runs.
__device__ __forceinline__ uint4 ld_arena_v4(const void *p)
{
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}

__device__ __forceinline__ void st_arena_v4(void *p, const uint4 &v)
{
    asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x),
                 "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

__device__ __forceinline__ unsigned long long global_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ------------------------------------------------------------ block barrier
struct BlockSync {
    uint32_t epoch;  // barriers this block index has passed (all launches)
    int failed;
    int phase;
};

__device__ __forceinline__ SignalPad *pad_of(const CommCtx &ctx, int r)
{
    return reinterpret_cast<SignalPad *>(ctx.base[r]);
}

__device__ __forceinline__ void sync_begin(const CommCtx &ctx, int rank, BlockSync *s)
{
    if (threadIdx.x == 0) {
        s->epoch = pad_of(ctx, rank)->epoch[blockIdx.x];
        s->failed = 0;
        s->phase = 0;
    }
    __syncthreads();
}

__device__ __forceinline__ void sync_end(const CommCtx &ctx, int rank, BlockSync *s)
{
    __syncthreads();
    if (threadIdx.x == 0 && !s->failed) { pad_of(ctx, rank)->epoch[blockIdx.x] = s->epoch; }
}

static __device__ __noinline__ void report_timeout(const CommCtx &ctx, int rank, int peer,
                                            uint32_t want, uint32_t have, int phase)
{
    StatusBlock *st = ctx.status;
    if (st == nullptr) { return; }
    volatile StatusBlock *v = st;
    if (v->code == kStatusOk) {
        v->rank = rank;
        v->block = static_cast<int>(blockIdx.x);
        v->peer = peer;
        v->want = want;
        v->have = have;
        v->phase = phase;
        __threadfence_system();
        v->code = kStatusTimeout;
        __threadfence_system();
    }
}

// Barrier between the blocks with the same blockIdx.x on every rank.  Thread p
// (p < world) publishes this block's arrival to rank p with a release store and
// waits, with a time and an iteration limit, for rank p's arrival with acquire
// loads.  Writes made by any thread of the block before the call are visible
// to the peers' threads after their call returns.  Returns false (for the whole
// block) when a wait ran out; the caller must then skip its remaining work.
__device__ __forceinline__ bool peer_barrier(const CommCtx &ctx, int rank, BlockSync *s)
{
    __syncthreads();
    const uint32_t target = s->epoch + 1u;
    const int p = static_cast<int>(threadIdx.x);
    if (p < ctx.world) {
        st_release_sys_u32(&pad_of(ctx, p)->flag[blockIdx.x][rank], target);
        const uint32_t *f = &pad_of(ctx, rank)->flag[blockIdx.x][p];
        unsigned int spins = 0;
        unsigned long long t0 = 0;
        for (;;) {
            const uint32_t seen = ld_acquire_sys_u32(f);
            if (static_cast<int32_t>(seen - target) >= 0) { break; }
            ++spins;
            if ((spins & 127u) == 0u) {
                const unsigned long long now = global_ns();
                if (t0 == 0) { t0 = now; }
                if (now - t0 > ctx.timeout_ns || spins >= ctx.max_spins) {
                    report_timeout(ctx, rank, p, target, seen, s->phase);
                    *reinterpret_cast<volatile int *>(&s->failed) = 1;
                    break;
                }
            }
        }
    }
    __syncthreads();
    const bool ok = (*reinterpret_cast<volatile int *>(&s->failed) == 0);
    __syncthreads();
    if (threadIdx.x == 0) {
        s->epoch = target;
        s->phase += 1;
    }
    return ok;
}

// One-way signals on the barrier's flags, for kernels in which one rank feeds
// the others in rounds.  signal_from(): this block of `rank` tells block
// blockIdx.x of every rank that everything its threads stored so far is in
// place (value = epoch + round + 1).  wait_for(): the others wait for it, with
// the barrier's limits.  After `rounds` rounds every rank calls rounds_done(),
// so that the next full barrier of all ranks starts from the same epoch.
__device__ __forceinline__ void signal_from(const CommCtx &ctx, int rank, BlockSync *s, int round)
{
    __syncthreads();
    const int p = static_cast<int>(threadIdx.x);
    if (p < ctx.world) {
        st_release_sys_u32(&pad_of(ctx, p)->flag[blockIdx.x][rank],
                           s->epoch + static_cast<uint32_t>(round) + 1u);
    }
}

__device__ __forceinline__ bool wait_for(const CommCtx &ctx, int rank, int src, BlockSync *s,
                                         int round)
{
    if (threadIdx.x == 0) {
        const uint32_t target = s->epoch + static_cast<uint32_t>(round) + 1u;
        const uint32_t *f = &pad_of(ctx, rank)->flag[blockIdx.x][src];
        unsigned int spins = 0;
        unsigned long long t0 = 0;
        for (;;) {
            const uint32_t seen = ld_acquire_sys_u32(f);
            if (static_cast<int32_t>(seen - target) >= 0) { break; }
            ++spins;
            if ((spins & 127u) == 0u) {
                const unsigned long long now = global_ns();
                if (t0 == 0) { t0 = now; }
                if (now - t0 > ctx.timeout_ns || spins >= ctx.max_spins) {
                    report_timeout(ctx, rank, src, target, seen, 32 + round);
                    *reinterpret_cast<volatile int *>(&s->failed) = 1;
                    break;
                }
            }
        }
    }
    __syncthreads();
    const bool ok = (*reinterpret_cast<volatile int *>(&s->failed) == 0);
    __syncthreads();
    return ok;
}

__device__ __forceinline__ void rounds_done(BlockSync *s, int rounds)
{
    __syncthreads();
    if (threadIdx.x == 0) { s->epoch += static_cast<uint32_t>(rounds); }
    __syncthreads();
}

// ------------------------------------------------------------- dtype traits
template <int DT>
struct Tr;

#define STDML_INT_TRAITS(E, S)                                                 \
    template <>                                                                \
    struct Tr<E> {                                                             \
        using storage = S;                                                     \
        using acc = S;                                                         \
        static constexpr bool is_float = false;                                \
        static constexpr bool is_half = false;                                 \
        static __device__ __forceinline__ acc widen(storage x) { return x; }   \
        static __device__ __forceinline__ storage narrow(acc x) { return x; }  \
    };
STDML_INT_TRAITS(DT_I8, int8_t)
STDML_INT_TRAITS(DT_I16, int16_t)
STDML_INT_TRAITS(DT_I32, int32_t)
STDML_INT_TRAITS(DT_I64, long long)
STDML_INT_TRAITS(DT_U8, uint8_t)
STDML_INT_TRAITS(DT_U16, uint16_t)
STDML_INT_TRAITS(DT_U32, uint32_t)
STDML_INT_TRAITS(DT_U64, unsigned long long)
#undef STDML_INT_TRAITS

template <>
struct Tr<DT_BF16> {
    using storage = uint16_t;
    using acc = float;
    static constexpr bool is_float = true;
    static constexpr bool is_half = true;
    static __device__ __forceinline__ acc widen(storage x)
    {
        return __uint_as_float(static_cast<uint32_t>(x) << 16);
    }
    static __device__ __forceinline__ storage narrow(acc x)
    {
        return __bfloat16_as_ushort(__float2bfloat16_rn(x));
    }
};

template <>
struct Tr<DT_F16> {
    using storage = uint16_t;
    using acc = float;
    static constexpr bool is_float = true;
    static constexpr bool is_half = true;
    static __device__ __forceinline__ acc widen(storage x)
    {
        return __half2float(__ushort_as_half(x));
    }
    static __device__ __forceinline__ storage narrow(acc x)
    {
        return __half_as_ushort(__float2half_rn(x));
    }
};

template <>
struct Tr<DT_F32> {
    using storage = float;
    using acc = float;
    static constexpr bool is_float = true;
    static constexpr bool is_half = false;
    static __device__ __forceinline__ acc widen(storage x) { return x; }
    static __device__ __forceinline__ storage narrow(acc x) { return x; }
};

template <>
struct Tr<DT_F64> {
    using storage = double;
    using acc = double;
    static constexpr bool is_float = true;
    static constexpr bool is_half = false;
    static __device__ __forceinline__ acc widen(storage x) { return x; }
    static __device__ __forceinline__ storage narrow(acc x) { return x; }
};

template <int DT>
__host__ __device__ constexpr int lanes_of()
{
    return 16 / static_cast<int>(sizeof(typename Tr<DT>::storage));
}

// Same expressions as the host reducers (src/dtype.cpp) so that results are
// bit-identical: wrap-around integer sum/prod, `b < a ? b : a` min/max (a NaN
// on the right-hand side is dropped, on the left-hand side kept).
template <int OP, typename A>
__device__ __forceinline__ A combine(A a, A b)
{
    if constexpr (std::is_integral_v<A>) {
        using U = std::make_unsigned_t<A>;
        if constexpr (OP == OP_SUM) {
            return static_cast<A>(static_cast<U>(a) + static_cast<U>(b));
        } else if constexpr (OP == OP_PROD) {
            return static_cast<A>(static_cast<U>(a) * static_cast<U>(b));
        } else if constexpr (OP == OP_MIN) {
            return b < a ? b : a;
        } else if constexpr (OP == OP_MAX) {
            return a < b ? b : a;
        } else {
            return static_cast<A>(a ^ b);
        }
    } else {
        if constexpr (OP == OP_SUM) {
            return a + b;
        } else if constexpr (OP == OP_PROD) {
            return a * b;
        } else if constexpr (OP == OP_MIN) {
            return b < a ? b : a;
        } else {
            return a < b ? b : a;
        }
    }
}

template <int DT>
union VecU {
    uint4 v;
    typename Tr<DT>::storage e[lanes_of<DT>()];
    __device__ VecU() {}
};

template <int DT>
struct Accum {
    static constexpr int N = lanes_of<DT>();
    typename Tr<DT>::acc a[N];

    __device__ __forceinline__ void init(const uint4 &x)
    {
        VecU<DT> u;
        u.v = x;
#pragma unroll
        for (int i = 0; i < N; ++i) { a[i] = Tr<DT>::widen(u.e[i]); }
    }

    template <int OP>
    __device__ __forceinline__ void add(const uint4 &x)
    {
        VecU<DT> u;
        u.v = x;
#pragma unroll
        for (int i = 0; i < N; ++i) { a[i] = combine<OP>(a[i], Tr<DT>::widen(u.e[i])); }
    }

    // `scale` is used in the accumulator's type: all 53 bits for f64, its f32
    // value for f32 and the 16-bit floats (as the host reducers do)
    __device__ __forceinline__ uint4 finish(double scale, bool has_scale) const
    {
        VecU<DT> u;
#pragma unroll
        for (int i = 0; i < N; ++i) {
            typename Tr<DT>::acc x = a[i];
            if constexpr (Tr<DT>::is_float) {
                if (has_scale) { x = x * static_cast<typename Tr<DT>::acc>(scale); }
            }
            u.e[i] = Tr<DT>::narrow(x);
        }
        return u.v;
    }
};

template <int DT>
__device__ __forceinline__ uint4 scale_vec(const uint4 &x, double scale)
{
    Accum<DT> a;
    a.init(x);
    return a.finish(scale, true);
}

// --------------------------------------------------------------- NVLS (multimem)
template <int DT, int OP>
constexpr bool nvls_ok()
{
    // f32/f16/bf16 add; f16/bf16 min and max.  Everything else (prod, f64,
    // float min/max in f32, integers) takes the peer-load kernels.
    if (DT == DT_F32) { return OP == OP_SUM; }
    if (DT == DT_BF16 || DT == DT_F16) { return OP == OP_SUM || OP == OP_MIN || OP == OP_MAX; }
    return false;
}

#define STDML_MM_LD(NAME, INSTR)                                               \
    __device__ __forceinline__ uint4 NAME(const void *mc)                      \
    {                                                                          \
        uint4 v;                                                               \
        asm volatile(INSTR " {%0,%1,%2,%3}, [%4];"                             \
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)              \
                     : "l"(mc)                                                 \
                     : "memory");                                              \
        return v;                                                              \
    }
STDML_MM_LD(mm_add_f32, "multimem.ld_reduce.relaxed.sys.global.add.v4.f32")
STDML_MM_LD(mm_add_bf16, "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2")
STDML_MM_LD(mm_min_bf16, "multimem.ld_reduce.relaxed.sys.global.min.v4.bf16x2")
STDML_MM_LD(mm_max_bf16, "multimem.ld_reduce.relaxed.sys.global.max.v4.bf16x2")
STDML_MM_LD(mm_add_f16, "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2")
STDML_MM_LD(mm_min_f16, "multimem.ld_reduce.relaxed.sys.global.min.v4.f16x2")
STDML_MM_LD(mm_max_f16, "multimem.ld_reduce.relaxed.sys.global.max.v4.f16x2")
#undef STDML_MM_LD

template <int DT, int OP>
__device__ __forceinline__ uint4 mm_ld_reduce(const void *mc)
{
    if constexpr (DT == DT_F32) {
        return mm_add_f32(mc);
    } else if constexpr (DT == DT_BF16) {
        if constexpr (OP == OP_SUM) {
            return mm_add_bf16(mc);
        } else if constexpr (OP == OP_MIN) {
            return mm_min_bf16(mc);
        } else {
            return mm_max_bf16(mc);
        }
    } else {
        if constexpr (OP == OP_SUM) {
            return mm_add_f16(mc);
        } else if constexpr (OP == OP_MIN) {
            return mm_min_f16(mc);
        } else {
            return mm_max_f16(mc);
        }
    }
}

// Untyped 16-byte store to every replica of the multicast address.
__device__ __forceinline__ void mm_st_v4(void *mc, const uint4 &v)
{
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc),
                 "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}
}  // namespace stdml::collective::cuda
