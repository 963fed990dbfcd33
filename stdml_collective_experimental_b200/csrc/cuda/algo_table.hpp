// Which algorithm and how many CTAs a collective gets: pure functions of the
// message and of the world, so that every rank reaches the same answer and the
// table can be checked without a GPU.  Thresholds come from device-timed sweeps
// on 2, 4 and 8 B200s (f32 sum, 4 KB ... 1 GiB, all four algorithms against each
// other and against NCCL).
#pragma once
#include <algorithm>
#include <cstddef>

#include "comm.cuh"

namespace stdml::collective::cuda
{
struct AlgoTuning {
    int world = 1;
    int vranks = 1;       // > 1: ranks emulated as grid rows of one launch
    int num_sms = 148;
    int max_blocks = 128;
    size_t oneshot_max = 0;       // 0: measured default
    size_t nvls_oneshot_max = 0;  // 0: measured default
    bool has_nvls = false;
    // two-shot calls of at least this many bytes pull with bulk async copies
    // (kAlgoTwoShotTma); SIZE_MAX: never
    size_t tma_min = 64u << 20;  // measured at 2 GPUs: ahead of the register path from 64 MB
    // NVLS worlds: owner calls of at least this many bytes prefer the bulk-copy
    // two-shot over the in-switch reduction (fewer bytes per link direction:
    // (n-1)/n x S instead of (n+1)/n x S); SIZE_MAX: never
    size_t tma_over_nvls_min = SIZE_MAX;
    int nvls_blocks = 0;  // > 0: grid of large NVLS calls
    int tma_blocks = 0;   // > 0: grid of bulk-copy two-shot calls
};

inline size_t oneshot_limit(const AlgoTuning &t)
{
    if (t.oneshot_max != 0) { return t.oneshot_max; }
    const size_t w = static_cast<size_t>(t.world);
    return w <= 2 ? (8u << 20) : (16u << 20) / (w * w);
}

inline size_t nvls_oneshot_limit(const AlgoTuning &t)
{
    if (t.nvls_oneshot_max != 0) { return t.nvls_oneshot_max; }
    // only staged / out-of-place calls can take it; it beats a staged owner
    // algorithm up to a few MB
    return 2u << 20;
}

// need_owner: the result must stay in the symmetric buffer (in place), which
// only the owner algorithms (two-shot, NVLS) can do.
inline int select_algo(const AlgoTuning &t, size_t bytes, bool nvls_defined_for_op,
                       bool need_owner)
{
    if (t.world == 1) { return need_owner ? kAlgoTwoShot : kAlgoOneShot; }
    // with two GPUs the switch has nothing to add: peer loads are faster
    const bool nvls = t.has_nvls && nvls_defined_for_op && t.world > 2;
    if (nvls) {
        if (!need_owner && bytes <= nvls_oneshot_limit(t)) { return kAlgoNvlsOneShot; }
        if (bytes >= t.tma_over_nvls_min) { return kAlgoTwoShotTma; }
        return kAlgoNvls;
    }
    if (!need_owner && bytes <= oneshot_limit(t)) { return kAlgoOneShot; }
    return bytes >= t.tma_min ? kAlgoTwoShotTma : kAlgoTwoShot;
}

inline int select_blocks(const AlgoTuning &t, size_t nvec, int algo)
{
    const bool owner = is_owner_algo(algo);
    const size_t work = owner ? (nvec + t.world - 1) / t.world : nvec;
    const size_t per_block = static_cast<size_t>(kThreads) * 4;
    size_t b = (work + per_block - 1) / per_block;
    size_t cap = static_cast<size_t>(t.max_blocks);
    if (algo == kAlgoNvls || algo == kAlgoNvlsOneShot) {
        // the switch saturates with few CTAs; more only add contention (measured at
        // 8 GPUs, 64 MB - 1 GiB: 16 and 24 CTAs lead, 32 within 1 %, 64 and up behind)
        cap = std::min<size_t>(cap, nvec * 16 >= (16u << 20) ? 24 : 64);
        if (t.nvls_blocks > 0 && nvec * 16 >= (16u << 20)) { cap = static_cast<size_t>(t.nvls_blocks); }
    }
    if (algo == kAlgoTwoShotTma) {
        // one CTA per SM at most (the ring takes the SM's shared memory)
        cap = static_cast<size_t>(t.tma_blocks > 0 ? t.tma_blocks : t.num_sms);
        cap = std::min<size_t>(cap, static_cast<size_t>(t.num_sms));
    }
    // alone on the GPU the kernel is an HBM copy: one resident CTA per SM
    if (t.world == 1) { cap = static_cast<size_t>(t.num_sms); }
    if (t.vranks > 1) { cap = std::min<size_t>(cap, std::max(1, t.num_sms / t.vranks)); }
    b = std::max<size_t>(1, std::min(b, std::min<size_t>(cap, kMaxBlocks)));
    return static_cast<int>(b);
}
}  // namespace stdml::collective::cuda
