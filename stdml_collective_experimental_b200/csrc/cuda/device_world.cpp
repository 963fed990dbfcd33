#include "device_world.hpp"

#include <algorithm>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <new>
#include <stdexcept>

#include <cuda.h>
#include <cuda_runtime.h>
#include <unistd.h>

#include "algo_table.hpp"
#include "local_rendezvous.hpp"
#include "offset_heap.hpp"

namespace stdml::collective::cuda
{
namespace
{
// ------------------------------------------------------------------ helpers
void rt_check(cudaError_t e, const char *what)
{
    if (e != cudaSuccess) {
        throw std::runtime_error(std::string("CUDA runtime: ") + what + ": " +
                                 cudaGetErrorString(e));
    }
}

size_t round_up(size_t x, size_t m) { return (x + m - 1) / m * m; }

// The driver API is reached through cudaGetDriverEntryPoint so that this
// library loads (and its host parts run) on machines without libcuda.
struct Driver {
    decltype(&cuGetErrorString) GetErrorString = nullptr;
    decltype(&cuDeviceGet) DeviceGet = nullptr;
    decltype(&cuDeviceGetAttribute) DeviceGetAttribute = nullptr;
    decltype(&cuMemGetAllocationGranularity) MemGetAllocationGranularity = nullptr;
    decltype(&cuMemCreate) MemCreate = nullptr;
    decltype(&cuMemRelease) MemRelease = nullptr;
    decltype(&cuMemAddressReserve) MemAddressReserve = nullptr;
    decltype(&cuMemAddressFree) MemAddressFree = nullptr;
    decltype(&cuMemMap) MemMap = nullptr;
    decltype(&cuMemUnmap) MemUnmap = nullptr;
    decltype(&cuMemSetAccess) MemSetAccess = nullptr;
    decltype(&cuMemExportToShareableHandle) MemExportToShareableHandle = nullptr;
    decltype(&cuMemImportFromShareableHandle) MemImportFromShareableHandle = nullptr;
    decltype(&cuMulticastCreate) MulticastCreate = nullptr;
    decltype(&cuMulticastAddDevice) MulticastAddDevice = nullptr;
    decltype(&cuMulticastBindMem) MulticastBindMem = nullptr;
    decltype(&cuMulticastUnbind) MulticastUnbind = nullptr;
    decltype(&cuMulticastGetGranularity) MulticastGetGranularity = nullptr;
    decltype(&cuMemGetAddressRange) MemGetAddressRange = nullptr;
    decltype(&cuPointerGetAttribute) PointerGetAttribute = nullptr;
    bool ok = false;
    bool multicast = false;

    template <typename F>
    bool load(const char *name, F &fn)
    {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess || p == nullptr) {
            (void)cudaGetLastError();
            return false;
        }
        fn = reinterpret_cast<F>(p);
        return true;
    }

    Driver()
    {
        ok = load("cuGetErrorString", GetErrorString) && load("cuDeviceGet", DeviceGet) &&
             load("cuDeviceGetAttribute", DeviceGetAttribute) &&
             load("cuMemGetAllocationGranularity", MemGetAllocationGranularity) &&
             load("cuMemCreate", MemCreate) && load("cuMemRelease", MemRelease) &&
             load("cuMemAddressReserve", MemAddressReserve) &&
             load("cuMemAddressFree", MemAddressFree) && load("cuMemMap", MemMap) &&
             load("cuMemUnmap", MemUnmap) && load("cuMemSetAccess", MemSetAccess) &&
             load("cuMemExportToShareableHandle", MemExportToShareableHandle) &&
             load("cuMemImportFromShareableHandle", MemImportFromShareableHandle);
        multicast = ok && load("cuMulticastCreate", MulticastCreate) &&
                    load("cuMulticastAddDevice", MulticastAddDevice) &&
                    load("cuMulticastBindMem", MulticastBindMem) &&
                    load("cuMulticastUnbind", MulticastUnbind) &&
                    load("cuMulticastGetGranularity", MulticastGetGranularity);
        (void)load("cuMemGetAddressRange", MemGetAddressRange);
        (void)load("cuPointerGetAttribute", PointerGetAttribute);
    }

    std::string err(CUresult r) const
    {
        const char *s = nullptr;
        if (GetErrorString != nullptr && GetErrorString(r, &s) == CUDA_SUCCESS && s != nullptr) {
            return s;
        }
        return "CUresult " + std::to_string(static_cast<int>(r));
    }
};

Driver &driver()
{
    static Driver d;
    return d;
}

struct DrvError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

void drv_check(CUresult r, const char *what)
{
    if (r != CUDA_SUCCESS) {
        throw DrvError(std::string("CUDA driver: ") + what + ": " + driver().err(r));
    }
}

struct Mapping {
    CUdeviceptr va = 0;
    CUmemGenericAllocationHandle handle = 0;
    bool mapped = false;
    bool have_handle = false;
};

class World final : public DeviceWorld
{
    DeviceWorldOptions opt_;
    int vranks_;
    size_t arena_bytes_ = 0;
    size_t staging_off_[2] = {0, 0};
    unsigned long long staged_ops_ = 0;
    OffsetHeap heap_;
    double setup_ms_[4] = {0, 0, 0, 0};
    std::map<size_t, size_t> guarded_;  // offset handed out -> bytes between its guard bands
    std::string backend_;

    std::vector<char *> base_;  // per rank
    char *mc_base_ = nullptr;

    // vmm state
    std::vector<Mapping> maps_;
    Mapping mc_map_;
    bool mc_bound_ = false;
    CUdevice cudev_ = 0;
    // ipc / loopback state
    std::vector<void *> owned_;   // cudaMalloc'd
    std::vector<void *> opened_;  // cudaIpcOpenMemHandle'd

    StatusBlock *status_host_ = nullptr;
    StatusBlock *status_dev_ = nullptr;

    // registered user memory: what this rank has exported (by base address) and
    // what it has imported from each peer (by that peer's base address)
    struct Exported {
        cudaIpcMemHandle_t handle;
        size_t size = 0;
        bool announced = false;  // the peers have seen this handle already
    };
    struct Imported {
        cudaIpcMemHandle_t handle;
        size_t size = 0;
        void *mapped = nullptr;
    };
    std::map<uintptr_t, Exported> exported_;
    std::vector<std::map<uintptr_t, Imported>> imported_;  // per peer

    std::unique_ptr<LocalRendezvous> rdv_;
    int num_sms_ = 148;
    int max_blocks_ = 128;
    size_t oneshot_max_ = 0;       // 0: measured default for this world size
    size_t nvls_oneshot_max_ = 0;  // 0: measured default for this world size
    size_t tma_min_ = 64u << 20;           // STDML_COLLECTIVE_TMA_MIN_BYTES (-1: never)
    size_t tma_over_nvls_min_ = SIZE_MAX;  // STDML_COLLECTIVE_TMA_OVER_NVLS_MIN_BYTES
    int nvls_blocks_ = 0;                  // STDML_COLLECTIVE_NVLS_BLOCKS
    int tma_blocks_ = 0;                   // STDML_COLLECTIVE_TMA_BLOCKS
    unsigned int tma_tile_vec_ = 0;        // STDML_COLLECTIVE_TMA_TILE_VEC (0: 1024, two vectors per thread)
    int nvls_variant_ = kNvlsPipe4;        // STDML_COLLECTIVE_NVLS_VARIANT
    bool debug_checks_ = false;            // STDML_COLLECTIVE_DEBUG
    size_t bcast_pipelined_min_ = 8u << 20;  // STDML_COLLECTIVE_BCAST_PIPELINED_MIN_BYTES
    size_t group_bulk_min_ = 4u << 20;       // registered groups: bulk copies from here (knob group_bulk_min_bytes)
    size_t bcast_piece_vec_ = 1024;          // vectors per round, block and slice (knob bcast_piece_vec)
    size_t gather_push_min_ = 64u << 10;  // STDML_COLLECTIVE_GATHER_PUSH_MIN_BYTES
    bool gather_mc_ = false;  // STDML_COLLECTIVE_GATHER_MC: all_gather through the switch (measured
                              // at 8 GPUs: plain stores 653-660 GB/s, multimem.st 614-625)
    int hybrid_permille_ = 150;        // share of a hybrid call that goes by peer loads (knob hybrid_permille)
    int hybrid_twoshot_blocks_ = 64;   // CTAs of that share (knob hybrid_twoshot_blocks)
    static constexpr unsigned long long kHybridGranule = 32;  // the spans' own granule
    int debug_inject_ = 0;  // tests: hand the next all_reduce kernel arguments that its
                            // own checks must refuse (1: misaligned offset, 2: offset
                            // inside the signal pad); implies debug_checks for that launch
    unsigned long long wait_timeout_ns_;

  public:
    explicit World(const DeviceWorldOptions &o)
        : opt_(o), vranks_(o.loopback ? o.world : 1),
          wait_timeout_ns_(o.wait_timeout_ms * 1000000ull)
    {
        if (o.world < 1 || o.world > kMaxRanks) {
            throw std::invalid_argument("device world: world size must be in [1, " +
                                        std::to_string(kMaxRanks) + "]");
        }
        if (!o.loopback && (o.rank < 0 || o.rank >= o.world)) {
            throw std::invalid_argument("device world: bad rank");
        }
        rt_check(cudaSetDevice(o.device), "cudaSetDevice");
        rt_check(cudaFree(nullptr), "context creation");
        cudaDeviceProp prop;
        rt_check(cudaGetDeviceProperties(&prop, o.device), "cudaGetDeviceProperties");
        num_sms_ = prop.multiProcessorCount;
        if (const char *e = std::getenv("STDML_COLLECTIVE_MAX_BLOCKS")) {
            max_blocks_ = std::max(1, std::min(kMaxBlocks, std::atoi(e)));
        }
        if (const char *e = std::getenv("STDML_COLLECTIVE_ONESHOT_MAX_BYTES")) {
            oneshot_max_ = static_cast<size_t>(std::atoll(e));
        }
        if (const char *e = std::getenv("STDML_COLLECTIVE_NVLS_ONESHOT_MAX_BYTES")) {
            nvls_oneshot_max_ = static_cast<size_t>(std::atoll(e));
        }
        auto env_bytes = [](const char *name, size_t &out) {
            if (const char *e = std::getenv(name)) {
                const long long v = std::atoll(e);
                out = v < 0 ? SIZE_MAX : static_cast<size_t>(v);
            }
        };
        env_bytes("STDML_COLLECTIVE_TMA_MIN_BYTES", tma_min_);
        env_bytes("STDML_COLLECTIVE_TMA_OVER_NVLS_MIN_BYTES", tma_over_nvls_min_);
        env_bytes("STDML_COLLECTIVE_GROUP_BULK_MIN_BYTES", group_bulk_min_);
        if (const char *e = std::getenv("STDML_COLLECTIVE_NVLS_BLOCKS")) { nvls_blocks_ = std::atoi(e); }
        if (const char *e = std::getenv("STDML_COLLECTIVE_TMA_BLOCKS")) { tma_blocks_ = std::atoi(e); }
        if (const char *e = std::getenv("STDML_COLLECTIVE_TMA_TILE_VEC")) {
            tma_tile_vec_ = static_cast<unsigned int>(std::max(0, std::atoi(e)));
        }
        if (const char *e = std::getenv("STDML_COLLECTIVE_NVLS_VARIANT")) {
            nvls_variant_ = std::max(0, std::min(kNvlsVariants - 1, std::atoi(e)));
        }
        env_bytes("STDML_COLLECTIVE_GATHER_PUSH_MIN_BYTES", gather_push_min_);
        env_bytes("STDML_COLLECTIVE_BCAST_PIPELINED_MIN_BYTES", bcast_pipelined_min_);
        if (const char *e = std::getenv("STDML_COLLECTIVE_GATHER_MC")) { gather_mc_ = std::atoi(e) != 0; }
        if (const char *e = std::getenv("STDML_COLLECTIVE_DEBUG")) {
            debug_checks_ = std::atoi(e) != 0;
        }

        const size_t staging = round_up(std::max<size_t>(o.staging_bytes, 4096), 4096);
        staging_off_[0] = kDataOffset;
        staging_off_[1] = kDataOffset + staging;
        const size_t heap_off = kDataOffset + 2 * staging;
        arena_bytes_ = heap_off + round_up(o.heap_bytes, 4096);
        opt_.staging_bytes = staging;

        rt_check(cudaHostAlloc(reinterpret_cast<void **>(&status_host_), sizeof(StatusBlock),
                               cudaHostAllocMapped),
                 "cudaHostAlloc(status)");
        std::memset(status_host_, 0, sizeof(StatusBlock));
        rt_check(cudaHostGetDevicePointer(reinterpret_cast<void **>(&status_dev_), status_host_, 0),
                 "cudaHostGetDevicePointer");

        base_.assign(o.world, nullptr);
        try {
            if (o.loopback) {
                setup_loopback();
            } else {
                if (o.world > 1) {
                    const auto t0 = std::chrono::steady_clock::now();
                    rdv_ = std::make_unique<LocalRendezvous>(o.key, o.rank, o.world,
                                                             o.setup_timeout_ms);
                    setup_ms_[0] = ms_since(t0);
                }
                setup_real();
            }
        } catch (...) {
            teardown();
            throw;
        }
        heap_.reset(heap_off, arena_bytes_ - heap_off);
    }

    ~World() override { teardown(); }

    // ------------------------------------------------------------ accessors
    int rank() const override { return opt_.loopback ? 0 : opt_.rank; }
    int world() const override { return opt_.world; }
    int vranks() const override { return vranks_; }
    int device() const override { return opt_.device; }
    bool has_nvls() const override { return mc_base_ != nullptr; }
    const char *backend() const override { return backend_.c_str(); }
    size_t arena_bytes() const override { return arena_bytes_; }
    void setup_ms(double out[4]) const override
    {
        for (int i = 0; i < 4; ++i) { out[i] = setup_ms_[i]; }
    }
    size_t staging_bytes() const override { return opt_.staging_bytes; }

    void *ptr(int r, size_t off) const override
    {
        if (r < 0 || r >= opt_.world || off > arena_bytes_) {
            throw std::out_of_range("device world: ptr()");
        }
        return base_[r] + off;
    }

    void *mc_ptr(size_t off) const override
    {
        return mc_base_ == nullptr ? nullptr : mc_base_ + off;
    }

    size_t offset_of(const void *p, int vr) const override
    {
        const int r = opt_.loopback ? vr : opt_.rank;
        const char *c = static_cast<const char *>(p);
        if (c >= base_[r] && c < base_[r] + arena_bytes_) {
            return static_cast<size_t>(c - base_[r]);
        }
        return SIZE_MAX;
    }

    // Every heap allocation sits between two guard bands filled with a known
    // word; release() reads them back and reports a band that changed (a kernel,
    // ours or the user's, that wrote outside its buffer).  Peers write into this
    // arena too, so the bands of every rank's copy tell on remote writers as well.
    static constexpr size_t kGuardBytes = 256;
    static constexpr unsigned char kGuardByte = 0xA5;

    size_t alloc(size_t bytes) override
    {
        const size_t body = round_up(std::max<size_t>(bytes, 16), 256);
        const size_t off = heap_.alloc(body + 2 * kGuardBytes);
        for (int r = 0; r < opt_.world; ++r) {
            if (!opt_.loopback && r != opt_.rank) { continue; }  // each rank paints its own
            rt_check(cudaMemset(base_[r] + off, kGuardByte, kGuardBytes), "cudaMemset(guard)");
            rt_check(cudaMemset(base_[r] + off + kGuardBytes + body, kGuardByte, kGuardBytes),
                     "cudaMemset(guard)");
        }
        rt_check(cudaStreamSynchronize(nullptr), "cudaStreamSynchronize");
        guarded_[off + kGuardBytes] = body;
        return off + kGuardBytes;
    }

    void release(size_t off) override
    {
        const auto it = guarded_.find(off);
        if (it == guarded_.end()) {
            throw std::invalid_argument("device world: release() of an offset that alloc() did "
                                        "not return");
        }
        const size_t body = it->second;
        guarded_.erase(it);
        std::string damage;
        unsigned char band[kGuardBytes];
        for (int r = 0; r < opt_.world; ++r) {
            if (!opt_.loopback && r != opt_.rank) { continue; }
            for (int side = 0; side < 2; ++side) {
                const char *at = base_[r] + (side == 0 ? off - kGuardBytes : off + body);
                if (cudaMemcpy(band, at, kGuardBytes, cudaMemcpyDeviceToHost) != cudaSuccess) {
                    (void)cudaGetLastError();
                    continue;
                }
                for (size_t i = 0; i < kGuardBytes; ++i) {
                    if (band[i] != kGuardByte) {
                        damage += " rank " + std::to_string(r) + (side == 0 ? " below" : " above") +
                                  " (first changed byte " + std::to_string(i) + ")";
                        break;
                    }
                }
            }
        }
        heap_.release(off - kGuardBytes);
        if (!damage.empty()) {
            throw std::runtime_error("device world: the guard bands of the symmetric buffer at "
                                     "offset " + std::to_string(off) + " were overwritten:" + damage);
        }
    }

    size_t next_staging_slot() override { return staging_off_[(staged_ops_++) & 1ull]; }

    void set_wait_timeout_ms(unsigned long long ms) override { wait_timeout_ns_ = ms * 1000000ull; }

    void set_tuning(int max_blocks, size_t oneshot_max_bytes,
                    size_t nvls_oneshot_max_bytes) override
    {
        if (max_blocks > 0) { max_blocks_ = std::min(max_blocks, kMaxBlocks); }
        if (oneshot_max_bytes != SIZE_MAX) { oneshot_max_ = oneshot_max_bytes; }
        if (nvls_oneshot_max_bytes != SIZE_MAX) { nvls_oneshot_max_ = nvls_oneshot_max_bytes; }
    }

    void set_knob(const std::string &name, long long value) override
    {
        if (name == "nvls_variant") {
            nvls_variant_ = static_cast<int>(std::max<long long>(0, std::min<long long>(kNvlsVariants - 1, value)));
        } else if (name == "nvls_blocks") {
            nvls_blocks_ = static_cast<int>(std::max<long long>(0, std::min<long long>(kMaxBlocks, value)));
        } else if (name == "tma_blocks") {
            tma_blocks_ = static_cast<int>(std::max<long long>(0, std::min<long long>(kMaxBlocks, value)));
        } else if (name == "tma_tile_vec") {
            tma_tile_vec_ = static_cast<unsigned int>(std::max<long long>(0, value));
        } else if (name == "tma_min_bytes") {
            tma_min_ = value < 0 ? SIZE_MAX : static_cast<size_t>(value);
        } else if (name == "tma_over_nvls_min_bytes") {
            tma_over_nvls_min_ = value < 0 ? SIZE_MAX : static_cast<size_t>(value);
        } else if (name == "group_bulk_min_bytes") {
            group_bulk_min_ = value < 0 ? SIZE_MAX : static_cast<size_t>(value);
        } else if (name == "bcast_piece_vec") {
            bcast_piece_vec_ = static_cast<size_t>(std::max<long long>(32, value));
        } else if (name == "bcast_pipelined_min_bytes") {
            bcast_pipelined_min_ = value < 0 ? SIZE_MAX : static_cast<size_t>(value);
        } else if (name == "gather_push_min_bytes") {
            gather_push_min_ = value < 0 ? SIZE_MAX : static_cast<size_t>(value);
        } else if (name == "gather_mc") {
            gather_mc_ = value != 0;
        } else if (name == "hybrid_permille") {
            hybrid_permille_ = static_cast<int>(std::max<long long>(0, std::min<long long>(1000, value)));
        } else if (name == "hybrid_twoshot_blocks") {
            hybrid_twoshot_blocks_ = static_cast<int>(std::max<long long>(1, std::min<long long>(512, value)));
        } else if (name == "debug_checks") {
            debug_checks_ = value != 0;
        } else if (name == "debug_inject") {
            debug_inject_ = static_cast<int>(value);
        } else {
            throw std::invalid_argument("device world: unknown knob '" + name + "'");
        }
    }

    // ------------------------------------------------------------ registration
    struct RegRecord {
        int ok;      // this rank's buffer can be exported (or it passed none)
        int fresh;   // the handle below has not been announced before
        unsigned long long base, size, offset;
        cudaIpcMemHandle_t handle;
    };

    // What this rank tells the others about one of its buffers.
    RegRecord make_record(void *mine, size_t bytes)
    {
        RegRecord rec;
        std::memset(&rec, 0, sizeof(rec));
        rec.ok = 1;
        if (mine == nullptr) { return rec; }
        rec.ok = 0;
        Driver &d = driver();
        CUdeviceptr base = 0;
        size_t size = 0;
        if (d.MemGetAddressRange != nullptr &&
            d.MemGetAddressRange(&base, &size, reinterpret_cast<CUdeviceptr>(mine)) ==
                CUDA_SUCCESS &&
            reinterpret_cast<uintptr_t>(mine) + bytes <= static_cast<uintptr_t>(base) + size) {
            // The handle is asked for on every call: an allocation that was freed and
            // made again at the same address and size has another handle, and only
            // a fresh look tells (the driver call costs microseconds).
            auto it = exported_.find(static_cast<uintptr_t>(base));
            cudaIpcMemHandle_t now;
            if (cudaIpcGetMemHandle(&now, reinterpret_cast<void *>(base)) == cudaSuccess) {
                if (it == exported_.end() || it->second.size != size ||
                    std::memcmp(&it->second.handle, &now, sizeof(now)) != 0) {
                    Exported e;
                    e.handle = now;
                    e.size = size;
                    exported_[static_cast<uintptr_t>(base)] = e;  // not announced yet
                    it = exported_.find(static_cast<uintptr_t>(base));
                }
            } else {
                (void)cudaGetLastError();  // e.g. memory from the VMM allocator
                if (it != exported_.end()) { exported_.erase(it); }
                it = exported_.end();
            }
            if (it != exported_.end()) {
                rec.ok = 1;
                rec.fresh = it->second.announced ? 0 : 1;
                rec.base = static_cast<unsigned long long>(base);
                rec.size = size;
                rec.offset = reinterpret_cast<uintptr_t>(mine) - static_cast<uintptr_t>(base);
                rec.handle = it->second.handle;
            }
        }
        return rec;
    }

    // Rank r's buffer as mapped here (null: that rank passed none, or the import failed,
    // which clears *imported_all).
    void *import_record(int r, const RegRecord &pr, bool *imported_all)
    {
        if (pr.base == 0) { return nullptr; }
        auto &table = imported_[r];
        auto it = table.find(static_cast<uintptr_t>(pr.base));
        if (it != table.end() &&
            (it->second.size != pr.size ||
             std::memcmp(&it->second.handle, &pr.handle, sizeof(pr.handle)) != 0)) {
            (void)cudaIpcCloseMemHandle(it->second.mapped);  // a new allocation at that address
            table.erase(it);
            it = table.end();
        }
        if (it == table.end()) {
            Imported im;
            im.handle = pr.handle;
            im.size = pr.size;
            if (cudaIpcOpenMemHandle(&im.mapped, pr.handle, cudaIpcMemLazyEnablePeerAccess) !=
                cudaSuccess) {
                (void)cudaGetLastError();
                *imported_all = false;
                return nullptr;
            }
            it = table.emplace(static_cast<uintptr_t>(pr.base), im).first;
        }
        return static_cast<char *>(it->second.mapped) + pr.offset;
    }

    bool resolve_peers(const void *const *ptrs, size_t bytes, void **peer_ptrs) override
    {
        return resolve_many(1, ptrs, &bytes, peer_ptrs);
    }

    bool resolve_many(size_t n, const void *const *ptrs, const size_t *bytes,
                      void **peer_ptrs) override
    {
        const int world = opt_.world;
        for (size_t k = 0; k < n * static_cast<size_t>(world); ++k) { peer_ptrs[k] = nullptr; }
        if (opt_.loopback) {
            for (size_t i = 0; i < n; ++i) {
                for (int v = 0; v < vranks_; ++v) {
                    peer_ptrs[i * world + v] = const_cast<void *>(ptrs[v * n + i]);
                }
            }
            return true;
        }
        if (world == 1) {
            for (size_t i = 0; i < n; ++i) { peer_ptrs[i] = const_cast<void *>(ptrs[i]); }
            return true;
        }
        std::vector<RegRecord> mine(n);
        for (size_t i = 0; i < n; ++i) { mine[i] = make_record(const_cast<void *>(ptrs[i]), bytes[i]); }
        std::vector<std::vector<char>> all;
        rdv_->all_gather(mine.data(), n * sizeof(RegRecord), all);
        bool everyone = true, any_fresh = false;
        for (int r = 0; r < world && everyone; ++r) {
            everyone = all[r].size() == n * sizeof(RegRecord);  // the same set on every rank
        }
        if (!everyone) { return false; }
        std::vector<RegRecord> recs(n * static_cast<size_t>(world));
        for (int r = 0; r < world; ++r) {
            for (size_t i = 0; i < n; ++i) {
                RegRecord &pr = recs[i * world + r];
                std::memcpy(&pr, all[r].data() + i * sizeof(RegRecord), sizeof(RegRecord));
                everyone = everyone && pr.ok != 0;
                any_fresh = any_fresh || pr.fresh != 0;
            }
        }
        if (!everyone) { return false; }
        for (size_t i = 0; i < n; ++i) {
            if (ptrs[i] != nullptr) { exported_[static_cast<uintptr_t>(mine[i].base)].announced = true; }
        }
        imported_.resize(world);
        bool imported_all = true;
        for (size_t i = 0; i < n; ++i) {
            for (int r = 0; r < world; ++r) {
                peer_ptrs[i * world + r] =
                    r == opt_.rank ? const_cast<void *>(ptrs[i])
                                   : import_record(r, recs[i * world + r], &imported_all);
            }
        }
        // every handle was seen before: every import above came from the tables
        if (any_fresh || !imported_all) { imported_all = rdv_->all_agree(imported_all); }
        return imported_all;
    }

    bool all_same(unsigned long long token) override
    {
        if (opt_.loopback || opt_.world == 1) { return token != 0; }
        std::vector<std::vector<char>> all;
        rdv_->all_gather(&token, sizeof(token), all);
        bool same = token != 0;
        for (const auto &x : all) {
            same = same && x.size() == sizeof(token) && std::memcmp(x.data(), &token, sizeof(token)) == 0;
        }
        return same;
    }

    unsigned long long buffer_id(const void *p) const override
    {
        Driver &d = driver();
        unsigned long long id = 0;
        if (p == nullptr || d.PointerGetAttribute == nullptr ||
            d.PointerGetAttribute(&id, CU_POINTER_ATTRIBUTE_BUFFER_ID,
                                  reinterpret_cast<CUdeviceptr>(p)) != CUDA_SUCCESS) {
            return 0;
        }
        return id;
    }

    void drop_registrations() override
    {
        if (opt_.loopback || opt_.world == 1) { return; }
        rt_check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
        rdv_->barrier();  // nobody has a kernel on these mappings any more
        close_imports();
        exported_.clear();
        rdv_->barrier();
    }

    size_t registrations() const override
    {
        size_t n = 0;
        for (const auto &t : imported_) { n += t.size(); }
        return n;
    }

    void close_imports()
    {
        for (auto &table : imported_) {
            for (auto &kv : table) { (void)cudaIpcCloseMemHandle(kv.second.mapped); }
            table.clear();
        }
        (void)cudaGetLastError();
    }

    // ------------------------------------------------------- algorithm table
    AlgoTuning tuning() const
    {
        AlgoTuning t;
        t.world = opt_.world;
        t.vranks = vranks_;
        t.num_sms = num_sms_;
        t.max_blocks = max_blocks_;
        t.oneshot_max = oneshot_max_;
        t.nvls_oneshot_max = nvls_oneshot_max_;
        t.has_nvls = has_nvls();
        t.tma_min = tma_min_;
        t.tma_over_nvls_min = tma_over_nvls_min_;
        t.nvls_blocks = nvls_blocks_;
        t.tma_blocks = tma_blocks_;
        return t;
    }

    int pick_algo(size_t bytes, int dt, int op, bool need_owner) const override
    {
        return select_algo(tuning(), bytes, nvls_supported(dt, op), need_owner);
    }

    int pick_peer_algo(size_t bytes) const override
    {
        return select_algo(tuning(), bytes, false, true);
    }

    int pick_blocks(size_t nvec, int algo) const override
    {
        return select_blocks(tuning(), nvec, algo);
    }

    // --------------------------------------------------------------- launches
    CommCtx make_ctx() const
    {
        CommCtx ctx;
        std::memset(&ctx, 0, sizeof(ctx));
        for (int r = 0; r < opt_.world; ++r) { ctx.base[r] = base_[r]; }
        ctx.mc_base = mc_base_;
        ctx.status = status_dev_;
        ctx.timeout_ns = wait_timeout_ns_;
        ctx.max_spins = 1u << 30;
        ctx.world = opt_.world;
        ctx.rank = opt_.loopback ? 0 : opt_.rank;
        return ctx;
    }

    int all_reduce(const AllReduceCall &c, void *stream) override
    {
        if (c.dt < 0 || c.dt > DT_F64_) { throw std::invalid_argument("all_reduce: bad dtype"); }
        if (c.op < 0 || c.op > 4) { throw std::invalid_argument("all_reduce: bad op"); }
        if (c.op == 4 && c.dt >= 8) {
            throw std::invalid_argument("all_reduce: bit_xor is not defined for floating point");
        }
        if (c.count == 0) { return 0; }
        static const size_t sizes[12] = {1, 2, 4, 8, 1, 2, 4, 8, 2, 2, 4, 8};
        const size_t esize = sizes[c.dt];
        const size_t bytes = c.count * esize;
        const size_t nvec = (bytes + 15) / 16;
        const bool registered = c.peer_data != nullptr;
        if (!registered &&
            (c.off % 16 != 0 || c.off < kDataOffset || c.off + nvec * 16 > arena_bytes_)) {
            throw std::invalid_argument("all_reduce: symmetric buffer outside the arena");
        }
        if (registered) {
            for (int r = 0; r < opt_.world; ++r) {
                if (c.peer_data[r] == nullptr ||
                    reinterpret_cast<uintptr_t>(c.peer_data[r]) % 16 != 0) {
                    throw std::invalid_argument("all_reduce: registered buffers must be mapped "
                                                "on every rank and 16-byte aligned");
                }
            }
        }
        const int user_dt = c.user_dtype < 0 ? c.dt : c.user_dtype;
        if (user_dt != c.dt && !((c.dt == 8 || c.dt == 9) && user_dt == 10)) {
            throw std::invalid_argument(
                "all_reduce: only f32 user tensors may differ from a bf16/f16 wire type");
        }
        bool any_dst_null = false;
        for (int v = 0; v < vranks_; ++v) {
            const bool has_dst = (c.table != nullptr && c.table[v] != nullptr) ||
                                 (c.dst != nullptr && c.dst[v] != nullptr);
            any_dst_null = any_dst_null || !has_dst;
        }
        if (opt_.world == 1 && vranks_ == 1 && c.table == nullptr && user_dt == c.dt &&
            c.phases == kPhaseAll) {
            // alone on the GPU: one scaled copy, straight from the source to the
            // destination (the arena buffer stands in for whichever is absent)
            char *sym = registered ? static_cast<char *>(c.peer_data[0]) : base_[0] + c.off;
            const void *from = (c.src != nullptr && c.src[0] != nullptr) ? c.src[0] : sym;
            void *to = (c.dst != nullptr && c.dst[0] != nullptr) ? c.dst[0] : sym;
            return launch_local_scale(from, to, c.count, c.dt, c.scale, c.has_scale ? 1 : 0,
                                      num_sms_, stream);
        }
        int algo = c.algo;
        if (algo < 0) { algo = pick_algo(bytes, c.dt, c.op, any_dst_null); }
        if (algo >= kAlgoCount) { throw std::invalid_argument("all_reduce: unknown algorithm"); }
        const bool owner = is_owner_algo(algo);
        const bool nvls =
            (algo == kAlgoNvls || algo == kAlgoNvlsOneShot || algo == kAlgoNvlsHybrid);
        if (algo == kAlgoNvlsHybrid && c.root >= 0) {
            throw std::invalid_argument("all_reduce: the hybrid algorithm has no reduce-to-root form");
        }
        if (!owner && any_dst_null && c.table == nullptr && c.root < 0) {
            throw std::invalid_argument("all_reduce: one-shot algorithms need a destination");
        }
        if (nvls && registered) {
            throw std::invalid_argument("all_reduce: NVLS needs a buffer in the symmetric arena");
        }
        if (nvls && (!has_nvls() || !nvls_supported(c.dt, c.op))) {
            throw std::invalid_argument("all_reduce: NVLS not available for this dtype/op/world");
        }
        bool staged = false;
        for (int v = 0; v < vranks_; ++v) {
            staged = staged || (c.table != nullptr && c.table[v] != nullptr) ||
                     (c.src != nullptr && c.src[v] != nullptr);
        }
        int blocks = c.blocks > 0 ? c.blocks : pick_blocks(nvec, algo);
        if (c.blocks <= 0 && nvls && (staged || c.root >= 0)) {
            // the pack / unpack phases are plain HBM copies and a root-only pull
            // has the switch to itself: both want the full grid, not the small
            // one that suits all ranks pulling through the switch together
            blocks = std::max(blocks, pick_blocks(nvec, algo == kAlgoNvls ? kAlgoTwoShot
                                                                          : kAlgoOneShot));
        }
        if (algo == kAlgoTwoShotTma) { blocks = std::min(blocks, num_sms_); }
        if (vranks_ > 1) { blocks = std::min(blocks, std::max(1, num_sms_ / vranks_)); }
        blocks = std::min(blocks, kMaxBlocks);

        AllReduceArgs a;
        std::memset(&a, 0, sizeof(a));
        for (int v = 0; v < vranks_; ++v) {
            a.src[v] = c.src != nullptr ? c.src[v] : nullptr;
            a.dst[v] = c.dst != nullptr ? c.dst[v] : nullptr;
            a.table[v] = c.table != nullptr ? c.table[v] : nullptr;
        }
        for (int r = 0; r < opt_.world; ++r) {
            a.data[r] = registered ? static_cast<char *>(c.peer_data[r]) : base_[r] + c.off;
            a.push[r] = (registered && c.peer_push != nullptr)
                            ? static_cast<char *>(c.peer_push[r])
                            : ((!registered && c.push_off != 0) ? base_[r] + c.push_off : a.data[r]);
        }
        if (!registered && c.push_off != 0 &&
            (c.push_off % 16 != 0 || c.push_off < kDataOffset ||
             c.push_off + nvec * 16 > arena_bytes_)) {
            throw std::invalid_argument("all_reduce: result region outside the arena");
        }
        if (registered && c.peer_push != nullptr) {
            for (int r = 0; r < opt_.world; ++r) {
                const bool needed = c.root < 0 || c.root == r;
                if ((needed && a.push[r] == nullptr) ||
                    reinterpret_cast<uintptr_t>(a.push[r]) % 16 != 0) {
                    throw std::invalid_argument("all_reduce: registered outputs must be mapped "
                                                "and 16-byte aligned");
                }
            }
        }
        a.off = registered ? 0 : c.off;
        a.count = c.count;
        a.nvec = nvec;
        a.ntable = c.ntable;
        a.algo = algo;
        a.user_dtype = user_dt;
        a.end_barrier = c.end_barrier ? 1 : 0;
        a.root = c.root;
        a.has_scale = c.has_scale ? 1 : 0;
        a.scale = c.scale;
        a.phases = c.phases;
        a.nvls_variant = nvls_variant_;
        a.debug_checks = debug_checks_ ? 1 : 0;
        if (debug_inject_ != 0) {
            // after the host-side validation, on purpose: this is what the kernel's
            // self-check exists to catch.  The kernel returns before any access.
            a.debug_checks = 1;
            if (debug_inject_ == 1) { a.off += 8; }
            if (debug_inject_ == 2) { a.off = 64; }
            debug_inject_ = 0;
        }
        if (algo == kAlgoTwoShotTma) {
            unsigned int smem = 0;
            tma_geometry(opt_.world, tma_tile_vec_, &a.tma_stages, &a.tma_tile_vec, &smem);
        }
        if (algo == kAlgoNvlsHybrid) {
            const int nbn = nvls_blocks_ > 0 ? nvls_blocks_ : 24;
            int nbt = hybrid_twoshot_blocks_;
            if (vranks_ > 1) { nbt = std::max(1, std::min(nbt, num_sms_ / vranks_ - nbn)); }
            if (c.blocks <= 0) { blocks = std::min(nbn + nbt, kMaxBlocks); }
            a.hybrid_nvls_blocks = std::max(1, std::min(nbn, blocks - 1));
            const unsigned long long keep =
                nvec * static_cast<unsigned long long>(1000 - hybrid_permille_) / 1000ull;
            a.hybrid_split_vec = std::min<unsigned long long>(keep / kHybridGranule * kHybridGranule, nvec);
        }
        if ((c.phases & kPhaseReduce) == 0) {
            // a local copy phase: no peer waits, any grid will do
            blocks = static_cast<int>(std::min<size_t>(
                std::max<size_t>(1, nvec / (static_cast<size_t>(kThreads) * 4)),
                static_cast<size_t>(2 * num_sms_)));
            if (vranks_ > 1) { blocks = std::min(blocks, std::max(1, num_sms_ / vranks_)); }
        }
        const CommCtx ctx = make_ctx();
        const int rc = launch_all_reduce(ctx, a, c.dt, c.op, blocks, vranks_, stream);
        if (rc < 0) { throw std::invalid_argument("all_reduce: (dtype, op) not built"); }
        return rc;
    }

    int gather(const GatherCall &c, void *stream) override
    {
        if (c.bytes == 0) { return 0; }
        const size_t nvec = (c.bytes + 15) / 16;
        const bool registered = c.peer_data != nullptr;
        const bool all_gather = c.root < 0;
        if (c.sym_stride % 16 != 0) {
            throw std::invalid_argument("gather: blocks of a region start on 16-byte boundaries");
        }
        const size_t span = all_gather
                                ? static_cast<size_t>(opt_.world - 1) * c.sym_stride + nvec * 16
                                : nvec * 16;
        if (!registered &&
            (c.off % 16 != 0 || c.off < kDataOffset || c.off + span > arena_bytes_)) {
            throw std::invalid_argument("gather: symmetric region outside the arena");
        }
        GatherArgs a;
        std::memset(&a, 0, sizeof(a));
        for (int v = 0; v < vranks_; ++v) {
            a.src[v] = c.src != nullptr ? c.src[v] : nullptr;
            a.dst[v] = c.dst != nullptr ? c.dst[v] : nullptr;
        }
        for (int r = 0; r < opt_.world; ++r) {
            a.data[r] = registered ? static_cast<char *>(c.peer_data[r]) : base_[r] + c.off;
            if (a.data[r] == nullptr || reinterpret_cast<uintptr_t>(a.data[r]) % 16 != 0) {
                throw std::invalid_argument("gather: regions must be mapped and 16-byte aligned");
            }
        }
        a.off = registered ? 0 : c.off;
        a.bytes = c.bytes;
        a.sym_stride = c.sym_stride;
        a.stride = c.stride != 0 ? c.stride : c.bytes;
        a.root = c.root;
        a.start_barrier = c.start_barrier ? 1 : 0;
        a.end_barrier = c.end_barrier ? 1 : 0;
        // with two GPUs the switch has nothing to add (measured: multimem.st 340 GB/s
        // against 640 GB/s for plain stores at 256 MB)
        const bool mc_possible = has_nvls() && !registered && opt_.world > 2;
        if (c.algo >= 0) {
            a.algo = c.algo;
        } else if (all_gather) {
            // measured: posted stores beat peer loads once the message is past the
            // latency-bound sizes
            a.algo = (opt_.world > 1 && c.bytes >= gather_push_min_) ? kGatherPush : kBcastPull;
        } else if (opt_.world > 2 && c.bytes >= bcast_pipelined_min_) {
            a.algo = kBcastPipelined;
        } else if (opt_.world > 1 && c.bytes >= (256u << 10)) {
            // pulling from root costs (n-1) copies on root's links
            a.algo = mc_possible ? kBcastNvls : (opt_.world > 2 ? kBcastScatter : kGatherPush);
        } else {
            a.algo = kBcastPull;
        }
        if (a.algo == kBcastNvls && !mc_possible) {
            throw std::invalid_argument("broadcast: NVLS needs the multicast mapping of the arena");
        }
        if (a.algo == kBcastPull && c.start_barrier) {
            // zero-copy pull: the peers read live memory of its owner, who may only go
            // on once they are done
            a.end_barrier = 1;
        }
        a.use_mc = c.use_mc >= 0 ? (c.use_mc != 0 && mc_possible) : (mc_possible && gather_mc_);
        if (all_gather && a.algo == kBcastPull && c.src != nullptr && c.sym_stride == 0) {
            // one block per region: block p is read at p * 0
        }
        int blocks = c.blocks > 0 ? c.blocks : pick_blocks(nvec, kAlgoOneShot);
        if (vranks_ > 1) { blocks = std::min(blocks, std::max(1, num_sms_ / vranks_)); }
        if (a.algo == kBcastPipelined) {
            // about 16 KB per piece: long enough to fill the links, short enough that
            // the holders start forwarding early; at most 9 rounds (8 GPUs, 256 MB:
            // 9 rounds 454 us, 18 rounds 501 us, 4 rounds 497 us)
            const size_t per_block_slice = nvec / static_cast<size_t>(opt_.world - 1) /
                                           static_cast<size_t>(std::max(1, blocks));
            a.rounds = static_cast<int>(std::max<size_t>(
                1, std::min<size_t>(9, per_block_slice / std::max<size_t>(32, bcast_piece_vec_))));
        }
        return launch_gather(make_ctx(), a, blocks, vranks_, stream);
    }

    int group_peer(const PeerEntry *table, int ntable, size_t nvec, int dt, int op, double scale,
                   void *stream) override
    {
        if (dt < 0 || dt > DT_F64_) { throw std::invalid_argument("group_peer: bad dtype"); }
        if (table == nullptr || ntable <= 0 || nvec == 0) { return 0; }
        GroupPeerArgs a;
        std::memset(&a, 0, sizeof(a));
        a.table = table;
        a.ntable = ntable;
        a.nvec = nvec;
        a.has_scale = scale != 1.0 ? 1 : 0;
        a.scale = scale;
        // bulk copies from 4 MB up (where the single-buffer sweep shows them ahead
        // of plain peer loads), unless the knob says otherwise
        const bool bulk = group_bulk_min_ != SIZE_MAX && nvec * 16 >= group_bulk_min_;
        int blocks = pick_blocks(nvec, bulk ? kAlgoTwoShotTma : kAlgoTwoShot);
        if (bulk) {
            unsigned int smem = 0;
            tma_geometry(opt_.world, tma_tile_vec_, &a.tma_stages, &a.tma_tile_vec, &smem);
            blocks = std::min(blocks, num_sms_);
        }
        if (vranks_ > 1) { blocks = std::min(blocks, std::max(1, num_sms_ / vranks_)); }
        blocks = std::min(blocks, kMaxBlocks);
        return launch_group_peer(make_ctx(), a, dt, op, blocks, vranks_, stream);
    }

    int unpack_blocks(const void *region, void *dst, size_t bytes, size_t sym_stride,
                      size_t stride, int blocks_n, void *stream, int want_grid) override
    {
        if (bytes == 0 || blocks_n <= 0) { return 0; }
        const size_t nvec = (bytes + 15) / 16;
        int grid = static_cast<int>(std::min<size_t>(
            std::max<size_t>(1, nvec / (static_cast<size_t>(kThreads) * 4)),
            static_cast<size_t>(2 * num_sms_)));
        if (want_grid > 0) { grid = std::min(grid, want_grid); }
        return launch_unpack_blocks(region, dst, bytes, sym_stride, stride, blocks_n, grid, stream);
    }

    int barrier(void *stream) override
    {
        launch_barrier(make_ctx(), vranks_, stream);
        return static_cast<int>(cudaGetLastError());
    }

    int barrier_rows(int rows, void *stream) override
    {
        if (!opt_.loopback || rows < 1 || rows > vranks_) {
            throw std::invalid_argument("barrier_rows: loopback world and 1 <= rows <= world");
        }
        launch_barrier(make_ctx(), rows, stream);
        return static_cast<int>(cudaGetLastError());
    }

    DeviceStatus poll_status() const override
    {
        DeviceStatus s;
        const volatile StatusBlock *v = status_host_;
        s.code = v->code;
        if (s.code != 0) {
            s.rank = v->rank;
            s.block = v->block;
            s.peer = v->peer;
            s.phase = v->phase;
            s.want = v->want;
            s.have = v->have;
        }
        return s;
    }

    void recover() override
    {
        rt_check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
        if (rdv_) { rdv_->barrier(); }
        if (opt_.loopback) {
            for (int r = 0; r < opt_.world; ++r) {
                rt_check(cudaMemset(base_[r], 0, kDataOffset), "cudaMemset(pad)");
            }
        } else {
            rt_check(cudaMemset(base_[opt_.rank], 0, kDataOffset), "cudaMemset(pad)");
        }
        rt_check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
        std::memset(status_host_, 0, sizeof(StatusBlock));
        staged_ops_ = 0;
        if (rdv_) { rdv_->barrier(); }
    }

  private:
    static constexpr int DT_F64_ = 11;

    void setup_loopback()
    {
        backend_ = "loopback";
        for (int r = 0; r < opt_.world; ++r) {
            void *p = nullptr;
            rt_check(cudaMalloc(&p, arena_bytes_), "cudaMalloc(arena)");
            owned_.push_back(p);
            rt_check(cudaMemset(p, 0, kDataOffset), "cudaMemset(pad)");
            base_[r] = static_cast<char *>(p);
        }
        rt_check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    }

    static double ms_since(std::chrono::steady_clock::time_point t0)
    {
        return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0)
            .count();
    }

    void setup_real()
    {
        const bool want_vmm = opt_.backend == "auto" || opt_.backend == "vmm";
        bool vmm_ok = false;
        std::string why;
        auto t0 = std::chrono::steady_clock::now();
        if (want_vmm) {
            try {
                vmm_ok = setup_vmm_local(why);
            } catch (const std::exception &e) {
                vmm_ok = false;
                why = e.what();
            }
        }
        setup_ms_[1] = ms_since(t0);
        // every rank must take the same path
        if (rdv_) { vmm_ok = rdv_->all_agree(vmm_ok); }
        if (vmm_ok) {
            backend_ = "vmm";
            t0 = std::chrono::steady_clock::now();
            exchange_vmm();
            setup_ms_[2] = ms_since(t0);
            t0 = std::chrono::steady_clock::now();
            if (opt_.enable_nvls && opt_.world > 1) { setup_multicast(); }
            setup_ms_[3] = ms_since(t0);
        } else {
            if (opt_.backend == "vmm") {
                throw std::runtime_error("device world: VMM backend unavailable: " + why);
            }
            release_vmm();
            backend_ = "ipc";
            setup_ipc();
        }
        if (rdv_) { rdv_->barrier(); }
    }

    // ------------------------------------------------------------------ VMM
    CUmemAllocationProp alloc_prop() const
    {
        CUmemAllocationProp prop;
        std::memset(&prop, 0, sizeof(prop));
        prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
        prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        prop.location.id = opt_.device;
        prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        return prop;
    }

    void map_rw(CUdeviceptr va, size_t size) const
    {
        CUmemAccessDesc acc;
        std::memset(&acc, 0, sizeof(acc));
        acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        acc.location.id = opt_.device;
        acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
        drv_check(driver().MemSetAccess(va, size, &acc, 1), "cuMemSetAccess");
    }

    bool multicast_capable() const
    {
        Driver &d = driver();
        if (!d.multicast) { return false; }
        int v = 0;
        if (d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cudev_) !=
            CUDA_SUCCESS) {
            return false;
        }
        return v != 0;
    }

    bool setup_vmm_local(std::string &why)
    {
        Driver &d = driver();
        if (!d.ok) {
            why = "driver entry points missing";
            return false;
        }
        drv_check(d.DeviceGet(&cudev_, opt_.device), "cuDeviceGet");
        int fd_ok = 0;
        drv_check(d.DeviceGetAttribute(
                      &fd_ok, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED,
                      cudev_),
                  "cuDeviceGetAttribute");
        if (!fd_ok) {
            why = "POSIX fd handles unsupported";
            return false;
        }
        const CUmemAllocationProp prop = alloc_prop();
        size_t gran = 0;
        drv_check(d.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED),
                  "cuMemGetAllocationGranularity");
        size_t size = round_up(arena_bytes_, gran);
        if (opt_.enable_nvls && opt_.world > 1 && multicast_capable()) {
            CUmulticastObjectProp mp;
            std::memset(&mp, 0, sizeof(mp));
            mp.numDevices = static_cast<unsigned int>(opt_.world);
            mp.size = size;
            mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
            size_t mg = 0;
            if (d.MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) ==
                    CUDA_SUCCESS &&
                mg > 0) {
                size = round_up(size, std::max(gran, mg));
            }
        }
        arena_bytes_ = size;  // the heap grows into the rounding slack
        maps_.assign(opt_.world, Mapping{});
        Mapping &me = maps_[opt_.rank];
        drv_check(d.MemCreate(&me.handle, size, &prop, 0), "cuMemCreate");
        me.have_handle = true;
        drv_check(d.MemAddressReserve(&me.va, size, gran, 0, 0), "cuMemAddressReserve");
        drv_check(d.MemMap(me.va, size, 0, me.handle, 0), "cuMemMap");
        me.mapped = true;
        map_rw(me.va, size);
        base_[opt_.rank] = reinterpret_cast<char *>(me.va);
        rt_check(cudaMemset(base_[opt_.rank], 0, kDataOffset), "cudaMemset(pad)");
        rt_check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
        return true;
    }

    void exchange_vmm()
    {
        if (opt_.world == 1) { return; }
        Driver &d = driver();
        // sizes can differ only if devices differ; insist on one size
        std::vector<std::vector<char>> sizes;
        const unsigned long long mine = arena_bytes_;
        rdv_->all_gather(&mine, sizeof(mine), sizes);
        for (const auto &s : sizes) {
            unsigned long long v;
            std::memcpy(&v, s.data(), sizeof(v));
            if (v != mine) { throw std::runtime_error("device world: arena sizes differ"); }
        }
        int my_fd = -1;
        drv_check(d.MemExportToShareableHandle(&my_fd, maps_[opt_.rank].handle,
                                               CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
                  "cuMemExportToShareableHandle");
        std::vector<int> fds = rdv_->all_gather_fd(my_fd);
        ::close(my_fd);
        const CUmemAllocationProp prop = alloc_prop();
        size_t gran = 0;
        drv_check(d.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED),
                  "cuMemGetAllocationGranularity");
        std::string first_error;
        for (int p = 0; p < opt_.world; ++p) {
            if (p == opt_.rank) { continue; }
            Mapping &m = maps_[p];
            try {
                drv_check(d.MemImportFromShareableHandle(
                              &m.handle, reinterpret_cast<void *>(static_cast<uintptr_t>(fds[p])),
                              CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
                          "cuMemImportFromShareableHandle");
                m.have_handle = true;
                drv_check(d.MemAddressReserve(&m.va, arena_bytes_, gran, 0, 0),
                          "cuMemAddressReserve(peer)");
                drv_check(d.MemMap(m.va, arena_bytes_, 0, m.handle, 0), "cuMemMap(peer)");
                m.mapped = true;
                map_rw(m.va, arena_bytes_);
                base_[p] = reinterpret_cast<char *>(m.va);
            } catch (const std::exception &e) {
                if (first_error.empty()) { first_error = e.what(); }
            }
            ::close(fds[p]);
        }
        if (!rdv_->all_agree(first_error.empty())) {
            throw std::runtime_error("device world: peer mapping failed: " +
                                     (first_error.empty() ? std::string("on another rank")
                                                          : first_error));
        }
    }

    // Builds the NVLS multicast mapping.  Any failure, on any rank, leaves all
    // ranks without it (peer loads still work); it never throws.
    void setup_multicast()
    {
        Driver &d = driver();
        bool ok = multicast_capable();
        if (!rdv_->all_agree(ok)) { return; }
        CUmulticastObjectProp mp;
        std::memset(&mp, 0, sizeof(mp));
        mp.numDevices = static_cast<unsigned int>(opt_.world);
        mp.size = arena_bytes_;
        mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        size_t mg = 0;
        ok = d.MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) ==
                 CUDA_SUCCESS &&
             mg > 0 && arena_bytes_ % mg == 0;

        // rank 0 creates and exports; everybody else imports
        int fd = -1;
        if (opt_.rank == 0) {
            if (ok) {
                ok = d.MulticastCreate(&mc_map_.handle, &mp) == CUDA_SUCCESS;
                mc_map_.have_handle = ok;
            }
            if (ok) {
                ok = d.MemExportToShareableHandle(&fd, mc_map_.handle,
                                                  CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR,
                                                  0) == CUDA_SUCCESS;
            }
            const char flag = ok ? 1 : 0;
            for (int p = 1; p < opt_.world; ++p) {
                rdv_->send_bytes(p, &flag, 1);
                if (ok) { rdv_->send_fd(p, fd); }
            }
            if (fd >= 0) { ::close(fd); }
        } else {
            char flag = 0;
            rdv_->recv_bytes(0, &flag, 1);
            if (flag) {
                fd = rdv_->recv_fd(0);
                if (ok) {
                    ok = d.MemImportFromShareableHandle(
                             &mc_map_.handle, reinterpret_cast<void *>(static_cast<uintptr_t>(fd)),
                             CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) == CUDA_SUCCESS;
                    mc_map_.have_handle = ok;
                }
                ::close(fd);
            } else {
                ok = false;
            }
        }
        if (ok) { ok = d.MulticastAddDevice(mc_map_.handle, cudev_) == CUDA_SUCCESS; }
        // every device must have been added before any memory is bound
        if (!rdv_->all_agree(ok)) {
            drop_multicast();
            return;
        }
        ok = d.MulticastBindMem(mc_map_.handle, 0, maps_[opt_.rank].handle, 0, arena_bytes_, 0) ==
             CUDA_SUCCESS;
        mc_bound_ = ok;
        if (ok) {
            ok = d.MemAddressReserve(&mc_map_.va, arena_bytes_, mg, 0, 0) == CUDA_SUCCESS;
        }
        if (ok) {
            ok = d.MemMap(mc_map_.va, arena_bytes_, 0, mc_map_.handle, 0) == CUDA_SUCCESS;
            mc_map_.mapped = ok;
        }
        if (ok) {
            try {
                map_rw(mc_map_.va, arena_bytes_);
            } catch (const std::exception &) {
                ok = false;
            }
        }
        if (!rdv_->all_agree(ok)) {
            drop_multicast();
            return;
        }
        mc_base_ = reinterpret_cast<char *>(mc_map_.va);
    }

    void drop_multicast()
    {
        Driver &d = driver();
        mc_base_ = nullptr;
        if (mc_map_.mapped) {
            d.MemUnmap(mc_map_.va, arena_bytes_);
            mc_map_.mapped = false;
        }
        if (mc_map_.va != 0) {
            d.MemAddressFree(mc_map_.va, arena_bytes_);
            mc_map_.va = 0;
        }
        if (mc_bound_) {
            d.MulticastUnbind(mc_map_.handle, cudev_, 0, arena_bytes_);
            mc_bound_ = false;
        }
        if (mc_map_.have_handle) {
            d.MemRelease(mc_map_.handle);
            mc_map_.have_handle = false;
        }
    }

    void release_vmm()
    {
        Driver &d = driver();
        if (!d.ok) { return; }
        drop_multicast();
        for (size_t p = 0; p < maps_.size(); ++p) {
            Mapping &m = maps_[p];
            if (m.mapped) { d.MemUnmap(m.va, arena_bytes_); }
            if (m.va != 0) { d.MemAddressFree(m.va, arena_bytes_); }
            if (m.have_handle) { d.MemRelease(m.handle); }
            m = Mapping{};
        }
        maps_.clear();
    }

    // ------------------------------------------------------------------ IPC
    void setup_ipc()
    {
        void *p = nullptr;
        rt_check(cudaMalloc(&p, arena_bytes_), "cudaMalloc(arena)");
        owned_.push_back(p);
        rt_check(cudaMemset(p, 0, kDataOffset), "cudaMemset(pad)");
        rt_check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
        base_[opt_.rank] = static_cast<char *>(p);
        if (opt_.world == 1) { return; }
        cudaIpcMemHandle_t h;
        rt_check(cudaIpcGetMemHandle(&h, p), "cudaIpcGetMemHandle");
        std::vector<std::vector<char>> all;
        rdv_->all_gather(&h, sizeof(h), all);
        std::string first_error;
        for (int r = 0; r < opt_.world; ++r) {
            if (r == opt_.rank) { continue; }
            cudaIpcMemHandle_t ph;
            std::memcpy(&ph, all[r].data(), sizeof(ph));
            void *q = nullptr;
            const cudaError_t e = cudaIpcOpenMemHandle(&q, ph, cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) {
                (void)cudaGetLastError();
                if (first_error.empty()) {
                    first_error = std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e);
                }
                continue;
            }
            opened_.push_back(q);
            base_[r] = static_cast<char *>(q);
        }
        if (!rdv_->all_agree(first_error.empty())) {
            throw std::runtime_error("device world: " + (first_error.empty()
                                                             ? std::string("IPC failed on a peer")
                                                             : first_error));
        }
    }

    void teardown()
    {
        // Nothing of ours may be in flight when mappings go away.
        (void)cudaSetDevice(opt_.device);
        (void)cudaDeviceSynchronize();
        if (rdv_) {
            try {
                rdv_->barrier();  // peers have stopped touching our memory
            } catch (const std::exception &) {
                // a peer is gone; carry on with local cleanup
            }
        }
        close_imports();
        release_vmm();
        for (void *q : opened_) { (void)cudaIpcCloseMemHandle(q); }
        opened_.clear();
        for (void *p : owned_) { (void)cudaFree(p); }
        owned_.clear();
        if (status_host_ != nullptr) {
            (void)cudaFreeHost(status_host_);
            status_host_ = nullptr;
        }
        (void)cudaGetLastError();
        rdv_.reset();
    }
};
}  // namespace

std::unique_ptr<DeviceWorld> DeviceWorld::create(const DeviceWorldOptions &opt)
{
    return std::make_unique<World>(opt);
}

int cuda_device_count()
{
    static const int count = [] {
        int n = 0;
        if (cudaGetDeviceCount(&n) != cudaSuccess) {
            (void)cudaGetLastError();
            return 0;
        }
        return n;
    }();
    return count;
}

bool cuda_available() { return cuda_device_count() > 0; }

void copy_device_to_host(void *host, const void *device, size_t bytes, void *stream)
{
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    rt_check(cudaMemcpyAsync(host, device, bytes, cudaMemcpyDeviceToHost, s), "cudaMemcpyAsync(D2H)");
    rt_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
}

void copy_host_to_device(void *device, const void *host, size_t bytes, void *stream)
{
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    rt_check(cudaMemcpyAsync(device, host, bytes, cudaMemcpyHostToDevice, s), "cudaMemcpyAsync(H2D)");
    rt_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
}

int pointer_kind(const void *p)
{
    if (p == nullptr || !cuda_available()) { return 0; }
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) ? 1 : 0;
}
}  // namespace stdml::collective::cuda
