// The walk over a table of registered tensors (PeerEntry): which tensor holds a
// vector of the group's flat index space, and the sequence of tiles that covers
// the whole vectors of a span, tensor after tensor.  Host and device code: the
// index arithmetic is exercised on the CPU (tests/test_partition_cuda.cpp).
#pragma once
#include "ar_kernel.cuh"

namespace stdml::collective::cuda
{
// Index of the last entry whose first vector is <= v.
__host__ __device__ __forceinline__ int find_peer_entry(const PeerEntry *tab, int n, unsigned long long v)
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

// Walks the whole vectors of a span tile by tile, tensor after tensor.
struct TileCursor {
    int i;                    // entry
    unsigned long long v;     // next vector, relative to the entry
    unsigned long long end;   // end of the entry's piece inside the span, relative
};

struct Tile {
    const PeerEntry *e;
    unsigned long long v0;  // first vector, relative to the entry
    unsigned int nv;
};

// The piece of entry i inside [lo, hi): whole vectors only.  False: past the span.
template <unsigned long long N>
__host__ __device__ __forceinline__ bool cursor_enter(const GroupPeerArgs &a, const Span &sp, TileCursor *c)
{
    for (; c->i < a.ntable; ++c->i) {
        const PeerEntry *e = &a.table[c->i];
        const unsigned long long voff = e->voff;
        if (voff >= sp.hi) { return false; }
        const unsigned long long full = e->count / N;
        const unsigned long long lo = (sp.lo > voff ? sp.lo : voff) - voff;
        const unsigned long long hi_abs = sp.hi < voff + full ? sp.hi : voff + full;
        if (hi_abs > voff + lo) {
            c->v = lo;
            c->end = hi_abs - voff;
            return true;
        }
    }
    return false;
}

template <unsigned long long N>
__host__ __device__ __forceinline__ bool cursor_next(const GroupPeerArgs &a, const Span &sp, TileCursor *c,
                                            unsigned int tile_vec, Tile *t)
{
    if (c->v >= c->end) {
        ++c->i;
        if (!cursor_enter<N>(a, sp, c)) {
            c->i = a.ntable;
            return false;
        }
    }
    const unsigned long long left = c->end - c->v;
    t->e = &a.table[c->i];
    t->v0 = c->v;
    t->nv = static_cast<unsigned int>(left < tile_vec ? left : tile_vec);
    c->v += t->nv;
    return true;
}
}  // namespace stdml::collective::cuda
