// Same-host rendezvous over abstract UNIX-domain sockets.  Used while a device
// world is being set up (and torn down, and re-built on an elastic resize) to
// pass file descriptors of CUDA VMM allocations between the ranks of one box
// (SCM_RIGHTS), small byte blobs (CUDA IPC handles), and host barriers.
//
// The reference has no counterpart: its ranks only share TCP connections
// (src/stdml/collective/net/old/rchan.cpp).  File descriptors cannot travel
// over TCP, hence this side channel.
#pragma once
#include <cstddef>
#include <string>
#include <vector>

namespace stdml::collective::cuda
{
class LocalRendezvous
{
  public:
    // Collective.  `key` must be the same on every rank of the job and unique
    // among the jobs of this host.  Throws std::runtime_error after
    // `timeout_ms` without a full mesh.
    LocalRendezvous(const std::string &key, int rank, int world, int timeout_ms = 120000);
    ~LocalRendezvous();

    LocalRendezvous(const LocalRendezvous &) = delete;
    LocalRendezvous &operator=(const LocalRendezvous &) = delete;

    int rank() const { return rank_; }
    int world() const { return world_; }

    void send_bytes(int peer, const void *data, size_t size);
    void recv_bytes(int peer, void *data, size_t size);
    void send_fd(int peer, int fd);
    int recv_fd(int peer);

    // Everyone contributes `size` bytes; out[r] receives rank r's bytes.
    void all_gather(const void *mine, size_t size, std::vector<std::vector<char>> &out);
    // Everyone contributes one descriptor; returns rank -> received fd
    // (own slot is -1).  Received descriptors belong to the caller.
    std::vector<int> all_gather_fd(int my_fd);
    // Logical AND over all ranks (also a barrier).
    bool all_agree(bool mine);
    void barrier() { (void)all_agree(true); }

  private:
    void connect_mesh(const std::string &key, int timeout_ms);
    void close_all();

    int rank_;
    int world_;
    int listen_fd_;
    std::vector<int> conn_;  // conn_[peer], -1 for self
};
}  // namespace stdml::collective::cuda
