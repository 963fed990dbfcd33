// Point-to-point transfers of device buffers: NCCL send / recv on a stream of
// their own, so that they overlap the collectives of the session (which run on
// this library's kernels).  libnccl is opened at run time (no link-time
// dependency: the host-only build and the CPU tests never need it); each pair
// of ranks that talks gets a two-rank communicator, created on first use by
// just those two ranks, so that send/recv stays a two-party operation.
//
// The reference's send/recv (src/stdml/collective/send_recv.cpp:6-21) is the
// rendezvous message of its TCP transport; device buffers have no path there.
#pragma once
#include <cstddef>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>

namespace stdml::collective::cuda
{
// true if a libnccl with the needed entry points can be opened
bool nccl_available(std::string *why = nullptr);

class NcclP2P
{
  public:
    // How the 128-byte communicator id travels between the two ranks of a pair
    // (the session's own host send / recv).
    using exchange_fn = std::function<void(int peer, bool i_send, void *id, size_t size)>;

    NcclP2P(int rank, int device, exchange_fn exchange);
    ~NcclP2P();

    // Enqueue on the transfer stream, after everything `after_stream` holds now.
    // `done` (optional) receives a cudaEvent_t recorded behind the transfer; the
    // caller owns it (cudaEventDestroy).
    void send(const void *ptr, size_t count, int dt, int peer, void *after_stream, void **done);
    void recv(void *ptr, size_t count, int dt, int peer, void *after_stream, void **done);
    // Blocks the host until everything enqueued so far has run.
    void wait_all();
    void *stream() const { return stream_; }

  private:
    void *comm_for(int peer);
    void transfer(bool is_send, void *ptr, size_t count, int dt, int peer, void *after_stream,
                  void **done);

    int rank_;
    int device_;
    exchange_fn exchange_;
    std::mutex mu_;
    std::map<int, void *> comms_;  // peer -> ncclComm_t
    void *stream_ = nullptr;
};
}  // namespace stdml::collective::cuda
