// Index arithmetic of the kernels, checked on the CPU (the functions are
// __host__ __device__): for many (vectors, shards, blocks) the block spans tile
// the buffer exactly once, and the descriptor-table search lands on the tensor
// that holds a vector.  compute-sanitizer is not available for the device
// code, so the arithmetic that decides every address is exercised here.
#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

#include "../cuda/ar_kernel.cuh"
#include "../cuda/group_walk.cuh"
#include "../cuda/device_session.hpp"
#include "../cuda/algo_table.hpp"
#include "../cuda/offset_heap.hpp"

using namespace stdml::collective::cuda;

static int failures = 0;
#define EXPECT(c)                                                              \
    do {                                                                       \
        if (!(c)) {                                                            \
            std::printf("%s:%d: %s\n", __FILE__, __LINE__, #c);                \
            ++failures;                                                        \
        }                                                                      \
    } while (0)

int main()
{
    std::mt19937_64 rng(7);
    // spans: contiguous, ordered, exact cover, every boundary but the buffer's end on a
    // 512-byte granule, balanced within one granule
    for (int trial = 0; trial < 20000; ++trial) {
        const unsigned long long nvec = rng() % (trial % 3 == 0 ? 50 : 5000000) ;
        const int shards = 1 + static_cast<int>(rng() % 16);
        const int nb = 1 + static_cast<int>(rng() % 200);
        unsigned long long expect = 0;
        for (int s = 0; s < shards; ++s) {
            unsigned long long lo_min = ~0ull, len_min = ~0ull, len_max = 0;
            for (int b = 0; b < nb; ++b) {
                const Span sp = span_of(nvec, shards, s, nb, b);
                EXPECT(sp.lo == expect && sp.hi >= sp.lo && sp.hi <= nvec);
                EXPECT(sp.lo % kSpanGranule == 0 || sp.lo == nvec);
                EXPECT(sp.hi % kSpanGranule == 0 || sp.hi == nvec);
                expect = sp.hi;
                lo_min = sp.lo < lo_min ? sp.lo : lo_min;
                const unsigned long long len = sp.hi - sp.lo;
                len_min = len < len_min ? len : len_min;
                len_max = len > len_max ? len : len_max;
            }
            EXPECT(len_max - len_min <= 2 * kSpanGranule);
        }
        EXPECT(expect == nvec);
    }
    // registered groups: over all ranks and blocks, the tiles of the walk cover every whole
    // vector of every tensor exactly once, in order, never across a tensor boundary and
    // never longer than a tile; the ragged last vectors are left to the element-wise tail
    for (int trial = 0; trial < 600; ++trial) {
        constexpr unsigned long long N = 4;  // f32 lanes
        const int n = 1 + static_cast<int>(rng() % 120);
        std::vector<PeerEntry> tab;
        unsigned long long voff = 0;
        for (int i = 0; i < n; ++i) {
            PeerEntry e;
            std::memset(&e, 0, sizeof(e));
            e.voff = voff;
            e.count = 1 + rng() % (i % 7 == 0 ? 300000 : 900);  // (empty tensors never enter a table)
            voff += (e.count + N - 1) / N;
            tab.push_back(e);
        }
        GroupPeerArgs a;
        std::memset(&a, 0, sizeof(a));
        a.table = tab.data();
        a.ntable = n;
        a.nvec = voff;
        const int world = 1 + static_cast<int>(rng() % 8);
        const int nb = 1 + static_cast<int>(rng() % 40);
        const unsigned int tile_vec = 32u << (rng() % 6);
        std::vector<unsigned long long> next(n, 0);  // first vector of each tensor not covered yet
        for (int r = 0; r < world; ++r) {
            for (int b = 0; b < nb; ++b) {
                const Span sp = span_of(a.nvec, world, r, nb, b);
                if (sp.lo >= sp.hi) { continue; }
                TileCursor c;
                c.i = find_peer_entry(a.table, a.ntable, sp.lo);
                c.v = c.end = 0;
                EXPECT(tab[c.i].voff <= sp.lo);
                if (!cursor_enter<N>(a, sp, &c)) { continue; }
                Tile t;
                while (cursor_next<N>(a, sp, &c, tile_vec, &t)) {
                    const int i = static_cast<int>(t.e - tab.data());
                    EXPECT(i >= 0 && i < n);
                    EXPECT(t.nv >= 1 && t.nv <= tile_vec);
                    EXPECT(t.v0 == next[i]);                         // in order, no gap, no overlap
                    EXPECT(t.v0 + t.nv <= tab[i].count / N);         // whole vectors of this tensor only
                    EXPECT(tab[i].voff + t.v0 >= sp.lo && tab[i].voff + t.v0 + t.nv <= sp.hi);
                    next[i] = t.v0 + t.nv;
                }
            }
        }
        for (int i = 0; i < n; ++i) { EXPECT(next[i] == tab[i].count / N); }
    }
    // descriptor tables: the entry found for v really contains v (or is the
    // last one starting at or before v when v falls into padding-free gaps)
    for (int trial = 0; trial < 2000; ++trial) {
        const int n = 1 + static_cast<int>(rng() % 300);
        std::vector<GroupEntry> tab(n);
        unsigned long long voff = 0;
        for (int i = 0; i < n; ++i) {
            tab[i].src = nullptr;
            tab[i].dst = nullptr;
            tab[i].voff = voff;
            tab[i].count = rng() % 5 == 0 ? 0 : 1 + rng() % 10000;  // some empty tensors
            voff += entry_nvec<DT_F32>(tab[i].count);
        }
        for (int q = 0; q < 50 && voff > 0; ++q) {
            const unsigned long long v = rng() % voff;
            const int i = find_entry(tab.data(), n, v);
            EXPECT(i >= 0 && i < n && tab[i].voff <= v);
            EXPECT(i == n - 1 || tab[i + 1].voff > v);
            // walking forward from i (as the kernel does) reaches the owner of v
            bool found = false;
            for (int j = i; j < n && tab[j].voff <= v; ++j) {
                found = found || v < tab[j].voff + entry_nvec<DT_F32>(tab[j].count);
            }
            EXPECT(found);
        }
    }
    // group planning: every element lands in exactly one piece, chunks respect
    // the slot size, pieces start on vector boundaries and keep tensor order
    for (int trial = 0; trial < 2000; ++trial) {
        const size_t n = 1 + rng() % 60;
        const size_t lanes = size_t(1) << (rng() % 5);  // 1, 2, 4, 8, 16 elements per vector
        const size_t cap = 1 + rng() % 3000;
        std::vector<size_t> counts(n);
        for (auto &c : counts) { c = rng() % 7 == 0 ? 0 : 1 + rng() % (cap * lanes * 3); }
        const auto chunks = plan_group_pieces(n, counts.data(), lanes, cap);
        std::vector<size_t> covered(n, 0);
        size_t last_tensor = 0;
        for (const auto &chunk : chunks) {
            size_t fill = 0;
            for (const auto &p : chunk) {
                EXPECT(p.tensor >= last_tensor && p.count > 0);
                last_tensor = p.tensor;
                EXPECT(p.voff == fill && p.first_elem == covered[p.tensor]);
                covered[p.tensor] += p.count;
                fill += (p.count + lanes - 1) / lanes;
                EXPECT(p.first_elem % lanes == 0);  // splits happen at vector boundaries
            }
            EXPECT(fill <= cap);
        }
        for (size_t i = 0; i < n; ++i) { EXPECT(covered[i] == counts[i]); }
    }
    // symmetric heap: deterministic first fit, 256-byte granules, coalescing
    {
        OffsetHeap h;
        h.reset(4096, 1 << 20);
        const size_t a = h.alloc(100), b = h.alloc(300), c = h.alloc(1);
        EXPECT(a == 4096 && b == 4096 + 256 && c == 4096 + 256 + 512);
        h.release(b);
        EXPECT(h.alloc(512) == b);   // exact hole reused
        h.release(a);
        h.release(b);
        EXPECT(h.alloc(700) == a);   // the two holes merged (256 + 512 >= 768)
        bool threw = false;
        try {
            h.alloc(2 << 20);
        } catch (const std::bad_alloc &) {
            threw = true;
        }
        EXPECT(threw);
        threw = false;
        try {
            h.release(12345);
        } catch (const std::invalid_argument &) {
            threw = true;
        }
        EXPECT(threw);
        // two heaps fed the same calls hand out the same offsets (ranks stay symmetric)
        OffsetHeap x, y;
        x.reset(0, 1 << 24);
        y.reset(0, 1 << 24);
        std::vector<size_t> live;
        for (int i = 0; i < 2000; ++i) {
            if (!live.empty() && rng() % 3 == 0) {
                const size_t k = rng() % live.size();
                x.release(live[k]);
                y.release(live[k]);
                live.erase(live.begin() + k);
            } else {
                const size_t bytes = 1 + rng() % 5000;
                const size_t ox = x.alloc(bytes), oy = y.alloc(bytes);
                EXPECT(ox == oy && ox % 256 == 0);
                live.push_back(ox);
            }
        }
    }
    // the measured algorithm table
    {
        AlgoTuning t8;
        t8.world = 8;
        t8.has_nvls = true;
        EXPECT(select_algo(t8, 64 << 10, true, false) == kAlgoNvlsOneShot);
        EXPECT(select_algo(t8, 2 << 20, true, false) == kAlgoNvlsOneShot);
        EXPECT(select_algo(t8, (2 << 20) + 16, true, false) == kAlgoNvls);
        EXPECT(select_algo(t8, 4096, true, true) == kAlgoNvls);            // in place
        EXPECT(select_algo(t8, 256 << 10, false, false) == kAlgoOneShot);  // e.g. prod: no NVLS
        EXPECT(select_algo(t8, (256 << 10) + 16, false, false) == kAlgoTwoShot);
        AlgoTuning t2 = t8;
        t2.world = 2;
        EXPECT(select_algo(t2, 8 << 20, true, false) == kAlgoOneShot);  // the switch adds nothing at 2
        EXPECT(select_algo(t2, 1 << 30, true, false) == kAlgoTwoShotTma);  // large: bulk-copy pulls
        EXPECT(select_algo(t2, 32 << 20, true, true) == kAlgoTwoShot);
        t2.tma_min = SIZE_MAX;
        EXPECT(select_algo(t2, 1 << 30, true, false) == kAlgoTwoShot);
        AlgoTuning t4 = t8;
        t4.world = 4;
        t4.has_nvls = false;
        EXPECT(select_algo(t4, 1 << 20, true, false) == kAlgoOneShot);
        EXPECT(select_algo(t4, (1 << 20) + 16, true, false) == kAlgoTwoShot);
        t4.tma_min = 1u << 20;
        EXPECT(select_algo(t4, (1 << 20) + 16, true, false) == kAlgoTwoShotTma);
        t4.tma_min = 64u << 20;
        EXPECT(select_algo(t4, 64u << 20, true, true) == kAlgoTwoShotTma);
        t8.tma_over_nvls_min = 32u << 20;  // NVLS worlds may prefer it from some size up
        EXPECT(select_algo(t8, 16u << 20, true, true) == kAlgoNvls);
        EXPECT(select_algo(t8, 32u << 20, true, true) == kAlgoTwoShotTma);
        t8.tma_over_nvls_min = SIZE_MAX;
        AlgoTuning t1;
        EXPECT(select_algo(t1, 1 << 20, true, false) == kAlgoOneShot);
        EXPECT(select_algo(t1, 1 << 20, true, true) == kAlgoTwoShot);
        t8.oneshot_max = 1024;  // overrides
        EXPECT(select_algo(t8, 2048, false, false) == kAlgoTwoShot);
        t8.oneshot_max = 0;
        // grids: one vector ... 1 GiB
        EXPECT(select_blocks(t8, 1, kAlgoNvls) == 1);
        EXPECT(select_blocks(t8, (1ull << 30) / 16, kAlgoNvls) == 24);
        EXPECT(select_blocks(t8, (8ull << 20) / 16, kAlgoNvls) == 32);  // 1 MB per rank / 32 KB per CTA
        EXPECT(select_blocks(t8, (1ull << 30) / 16, kAlgoTwoShot) == 128);
        EXPECT(select_blocks(t8, (1ull << 30) / 16, kAlgoOneShot) == 128);
        EXPECT(select_blocks(t1, (1ull << 30) / 16, kAlgoTwoShot) == 148);
        EXPECT(select_blocks(t8, (1ull << 30) / 16, kAlgoTwoShotTma) == 148);  // one CTA per SM
        t8.tma_blocks = 64;
        EXPECT(select_blocks(t8, (1ull << 30) / 16, kAlgoTwoShotTma) == 64);
        t8.tma_blocks = 0;
        {   // ring geometry: at least two slots, inside the budget, whole granules
            for (int w = 1; w <= kMaxRanks; ++w) {
                for (unsigned int want : {0u, 64u, 256u, 512u, 1000u, 4096u}) {
                    int st = 0;
                    unsigned int tv = 0, bytes = 0;
                    tma_geometry(w, want, &st, &tv, &bytes);
                    EXPECT(st >= 2 && st <= kTmaMaxStages && tv >= 32 && tv % 32 == 0);
                    EXPECT(bytes == st * w * tv * 16u && bytes <= kTmaSmemBudget);
                    EXPECT(w * tv * 16u < (1u << 20));  // one slot's bytes fit an mbarrier's count
                }
            }
        }
        AlgoTuning loop = t8;
        loop.vranks = 8;
        loop.has_nvls = false;
        EXPECT(select_blocks(loop, (1ull << 30) / 16, kAlgoTwoShot) == 18);  // 148 SMs / 8 rows
        for (int w = 1; w <= 16; ++w) {  // never zero, never above the pad size
            AlgoTuning t;
            t.world = w;
            for (unsigned long long nv : {1ull, 7ull, 4096ull, 1ull << 26}) {
                for (int algo = 0; algo < kAlgoCount; ++algo) {
                    const int b = select_blocks(t, nv, algo);
                    EXPECT(b >= 1 && b <= kMaxBlocks);
                }
            }
        }
    }
    {   // the rules of the in-kernel argument checks
        EXPECT(buffer_offset_ok(kDataOffset) && buffer_offset_ok(kDataOffset + 4096) && buffer_offset_ok(0));
        EXPECT(!buffer_offset_ok(kDataOffset + 8) && !buffer_offset_ok(64) && !buffer_offset_ok(kDataOffset - 16));
        GroupEntry tab[3];
        for (auto &e : tab) { e.src = nullptr; e.dst = nullptr; }
        tab[0].voff = 0;  tab[0].count = 10;   // 3 vectors of f32
        tab[1].voff = 3;  tab[1].count = 4;    // 1 vector
        tab[2].voff = 4;  tab[2].count = 1;
        for (int i = 0; i < 3; ++i) { EXPECT(table_entry_in_range<DT_F32>(tab, i, 3, 5)); }
        EXPECT(!table_entry_in_range<DT_F32>(tab, 2, 3, 4));   // runs past the buffer
        tab[1].voff = 2;                                       // overlaps its predecessor
        EXPECT(!table_entry_in_range<DT_F32>(tab, 0, 3, 5));
    }
    EXPECT(entry_nvec<DT_BF16>(9) == 2 && entry_nvec<DT_U8>(16) == 1 && entry_nvec<DT_F64>(3) == 2);
    std::printf("test-partition: %s\n", failures == 0 ? "OK" : "FAILED");
    return failures == 0 ? 0 : 1;
}
