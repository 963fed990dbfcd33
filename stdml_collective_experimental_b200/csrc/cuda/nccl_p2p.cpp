#include "nccl_p2p.hpp"

#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <vector>

#include <cuda_runtime.h>
#include <dlfcn.h>

namespace stdml::collective::cuda
{
namespace
{
// The part of NCCL's C interface that is used, declared here so that no NCCL
// header is needed to build.
struct UniqueId {
    char internal[128];
};
using comm_t = void *;
enum : int { kNcclInt8 = 0, kNcclUint8 = 1, kNcclInt32 = 2, kNcclUint32 = 3, kNcclInt64 = 4,
             kNcclUint64 = 5, kNcclHalf = 6, kNcclFloat = 7, kNcclDouble = 8, kNcclBfloat16 = 9 };

struct Api {
    void *lib = nullptr;
    int (*GetUniqueId)(UniqueId *) = nullptr;
    int (*CommInitRank)(comm_t *, int, UniqueId, int) = nullptr;
    int (*CommDestroy)(comm_t) = nullptr;
    int (*Send)(const void *, size_t, int, int, comm_t, cudaStream_t) = nullptr;
    int (*Recv)(void *, size_t, int, int, comm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
    std::string why;

    Api()
    {
        std::vector<std::string> names;
        if (const char *e = std::getenv("STDML_COLLECTIVE_NCCL_LIB")) { names.push_back(e); }
        names.push_back("libnccl.so.2");
        names.push_back("libnccl.so");
        // a process that already holds NCCL (PyTorch brings its own) keeps using that copy
        for (const auto &n : names) {
            lib = dlopen(n.c_str(), RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
            if (lib != nullptr) { break; }
        }
        for (size_t i = 0; lib == nullptr && i < names.size(); ++i) {
            lib = dlopen(names[i].c_str(), RTLD_NOW | RTLD_GLOBAL);
        }
        if (lib == nullptr) {
            why = "libnccl.so.2 not found (set STDML_COLLECTIVE_NCCL_LIB)";
            return;
        }
        auto sym = [&](const char *s) { return dlsym(lib, s); };
        GetUniqueId = reinterpret_cast<decltype(GetUniqueId)>(sym("ncclGetUniqueId"));
        CommInitRank = reinterpret_cast<decltype(CommInitRank)>(sym("ncclCommInitRank"));
        CommDestroy = reinterpret_cast<decltype(CommDestroy)>(sym("ncclCommDestroy"));
        Send = reinterpret_cast<decltype(Send)>(sym("ncclSend"));
        Recv = reinterpret_cast<decltype(Recv)>(sym("ncclRecv"));
        GetErrorString = reinterpret_cast<decltype(GetErrorString)>(sym("ncclGetErrorString"));
        if (!GetUniqueId || !CommInitRank || !CommDestroy || !Send || !Recv || !GetErrorString) {
            why = "libnccl lacks ncclSend / ncclRecv (NCCL 2.7 or newer is needed)";
            lib = nullptr;
        }
    }
};

Api &api()
{
    static Api a;
    return a;
}

void nccl_check(int rc, const char *what)
{
    if (rc != 0) {
        throw std::runtime_error(std::string("NCCL: ") + what + ": " + api().GetErrorString(rc));
    }
}

void cu_check(cudaError_t e, const char *what)
{
    if (e != cudaSuccess) {
        throw std::runtime_error(std::string("CUDA runtime: ") + what + ": " +
                                 cudaGetErrorString(e));
    }
}

// dtype codes of stdml/bits/collective/dtype.hpp -> NCCL's
int nccl_type(int dt)
{
    static const int map[12] = {kNcclInt8, -1, kNcclInt32, kNcclInt64, kNcclUint8, -1,
                                kNcclUint32, kNcclUint64, kNcclBfloat16, kNcclHalf, kNcclFloat,
                                kNcclDouble};
    return (dt >= 0 && dt < 12) ? map[dt] : -1;
}
}  // namespace

bool nccl_available(std::string *why)
{
    Api &a = api();
    if (a.lib == nullptr && why != nullptr) { *why = a.why; }
    return a.lib != nullptr;
}

NcclP2P::NcclP2P(int rank, int device, exchange_fn exchange)
    : rank_(rank), device_(device), exchange_(std::move(exchange))
{
    std::string why;
    if (!nccl_available(&why)) {
        throw std::runtime_error("send/recv of device buffers needs NCCL: " + why);
    }
    cu_check(cudaSetDevice(device_), "cudaSetDevice");
    cudaStream_t s;
    cu_check(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "cudaStreamCreate");
    stream_ = s;
}

NcclP2P::~NcclP2P()
{
    (void)cudaSetDevice(device_);
    if (stream_ != nullptr) { (void)cudaStreamSynchronize(static_cast<cudaStream_t>(stream_)); }
    for (auto &kv : comms_) { (void)api().CommDestroy(kv.second); }
    comms_.clear();
    if (stream_ != nullptr) { (void)cudaStreamDestroy(static_cast<cudaStream_t>(stream_)); }
    (void)cudaGetLastError();
}

// The lower rank of the pair makes the id and sends it over the host path;
// both then join a communicator of two (the lower rank is its rank 0).
void *NcclP2P::comm_for(int peer)
{
    const auto it = comms_.find(peer);
    if (it != comms_.end()) { return it->second; }
    if (peer == rank_) { throw std::invalid_argument("send/recv: a rank cannot be its own peer"); }
    UniqueId id;
    std::memset(&id, 0, sizeof(id));
    const bool lead = rank_ < peer;
    if (lead) { nccl_check(api().GetUniqueId(&id), "ncclGetUniqueId"); }
    exchange_(peer, lead, &id, sizeof(id));
    comm_t comm = nullptr;
    cu_check(cudaSetDevice(device_), "cudaSetDevice");
    nccl_check(api().CommInitRank(&comm, 2, id, lead ? 0 : 1), "ncclCommInitRank");
    comms_[peer] = comm;
    return comm;
}

void NcclP2P::transfer(bool is_send, void *ptr, size_t count, int dt, int peer,
                       void *after_stream, void **done)
{
    std::lock_guard<std::mutex> lk(mu_);
    int type = nccl_type(dt);
    size_t n = count;
    if (type < 0) {  // 16-bit integers: NCCL has no such type, bytes travel the same
        type = kNcclUint8;
        n = count * 2;
    }
    comm_t comm = comm_for(peer);
    cudaStream_t s = static_cast<cudaStream_t>(stream_);
    // the buffer is ready (send) or free (recv) when the caller's stream gets here
    cudaEvent_t ready;
    cu_check(cudaEventCreateWithFlags(&ready, cudaEventDisableTiming), "cudaEventCreate");
    cu_check(cudaEventRecord(ready, static_cast<cudaStream_t>(after_stream)), "cudaEventRecord");
    cu_check(cudaStreamWaitEvent(s, ready, 0), "cudaStreamWaitEvent");
    (void)cudaEventDestroy(ready);
    const int other = rank_ < peer ? 1 : 0;  // the peer's rank inside the pair
    if (is_send) {
        nccl_check(api().Send(ptr, n, type, other, comm, s), "ncclSend");
    } else {
        nccl_check(api().Recv(ptr, n, type, other, comm, s), "ncclRecv");
    }
    if (done != nullptr) {
        cudaEvent_t e;
        cu_check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate");
        cu_check(cudaEventRecord(e, s), "cudaEventRecord");
        *done = e;
    }
}

void NcclP2P::send(const void *ptr, size_t count, int dt, int peer, void *after_stream,
                   void **done)
{
    transfer(true, const_cast<void *>(ptr), count, dt, peer, after_stream, done);
}

void NcclP2P::recv(void *ptr, size_t count, int dt, int peer, void *after_stream, void **done)
{
    transfer(false, ptr, count, dt, peer, after_stream, done);
}

void NcclP2P::wait_all()
{
    cu_check(cudaStreamSynchronize(static_cast<cudaStream_t>(stream_)), "cudaStreamSynchronize");
}
}  // namespace stdml::collective::cuda
