#include "local_rendezvous.hpp"

#include <algorithm>

#include <cerrno>
#include <chrono>
#include <cstring>
#include <stdexcept>
#include <thread>

#include <sys/socket.h>
#include <sys/time.h>
#include <sys/un.h>
#include <unistd.h>

namespace stdml::collective::cuda
{
namespace
{
using clock_type = std::chrono::steady_clock;

[[noreturn]] void fail(const std::string &what)
{
    throw std::runtime_error("local rendezvous: " + what + ": " + std::strerror(errno));
}

socklen_t make_addr(const std::string &key, int rank, sockaddr_un &addr)
{
    std::memset(&addr, 0, sizeof(addr));
    addr.sun_family = AF_UNIX;
    // abstract namespace: leading NUL, no file to clean up
    const std::string name = "stdml-collective/" + key + "/" + std::to_string(rank);
    if (name.size() + 1 > sizeof(addr.sun_path)) {
        throw std::runtime_error("local rendezvous: key too long");
    }
    std::memcpy(addr.sun_path + 1, name.data(), name.size());
    return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + name.size());
}

void set_timeouts(int fd, int timeout_ms)
{
    timeval tv;
    tv.tv_sec = timeout_ms / 1000;
    tv.tv_usec = (timeout_ms % 1000) * 1000;
    setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
    setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
}

void write_all(int fd, const void *data, size_t size)
{
    const char *p = static_cast<const char *>(data);
    while (size > 0) {
        const ssize_t n = ::send(fd, p, size, MSG_NOSIGNAL);
        if (n < 0) {
            if (errno == EINTR) { continue; }
            fail("send");
        }
        p += n;
        size -= static_cast<size_t>(n);
    }
}

void read_all(int fd, void *data, size_t size)
{
    char *p = static_cast<char *>(data);
    while (size > 0) {
        const ssize_t n = ::recv(fd, p, size, 0);
        if (n < 0) {
            if (errno == EINTR) { continue; }
            fail("recv");
        }
        if (n == 0) { throw std::runtime_error("local rendezvous: peer closed"); }
        p += n;
        size -= static_cast<size_t>(n);
    }
}
}  // namespace

LocalRendezvous::LocalRendezvous(const std::string &key, int rank, int world, int timeout_ms)
    : rank_(rank), world_(world), listen_fd_(-1), conn_(world, -1)
{
    if (world <= 1) { return; }
    try {
        connect_mesh(key, timeout_ms);
    } catch (...) {
        close_all();  // no destructor runs for an object whose constructor threw
        throw;
    }
}

void LocalRendezvous::close_all()
{
    for (int &fd : conn_) {
        if (fd >= 0) { ::close(fd); }
        fd = -1;
    }
    if (listen_fd_ >= 0) { ::close(listen_fd_); }
    listen_fd_ = -1;
}

void LocalRendezvous::connect_mesh(const std::string &key, int timeout_ms)
{
    const int rank = rank_, world = world_;
    const auto deadline = clock_type::now() + std::chrono::milliseconds(timeout_ms);

    listen_fd_ = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (listen_fd_ < 0) { fail("socket"); }
    sockaddr_un addr;
    socklen_t len = make_addr(key, rank, addr);
    if (::bind(listen_fd_, reinterpret_cast<sockaddr *>(&addr), len) != 0) { fail("bind"); }
    if (::listen(listen_fd_, world) != 0) { fail("listen"); }
    set_timeouts(listen_fd_, timeout_ms);

    // lower ranks are dialled, higher ranks dial us
    for (int peer = 0; peer < rank; ++peer) {
        sockaddr_un pa;
        const socklen_t pl = make_addr(key, peer, pa);
        for (;;) {
            const int fd = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
            if (fd < 0) { fail("socket"); }
            if (::connect(fd, reinterpret_cast<sockaddr *>(&pa), pl) == 0) {
                set_timeouts(fd, timeout_ms);
                conn_[peer] = fd;  // owned from here on (closed by close_all on failure)
                const int32_t hello = rank;
                write_all(fd, &hello, sizeof(hello));
                break;
            }
            ::close(fd);
            if (clock_type::now() > deadline) {
                throw std::runtime_error("local rendezvous: rank " + std::to_string(peer) +
                                         " did not show up (key " + key + ")");
            }
            std::this_thread::sleep_for(std::chrono::milliseconds(5));
        }
    }
    for (int i = rank + 1; i < world; ++i) {
        const int fd = ::accept4(listen_fd_, nullptr, nullptr, SOCK_CLOEXEC);
        if (fd < 0) { fail("accept"); }
        set_timeouts(fd, timeout_ms);
        int32_t hello = -1;
        try {
            read_all(fd, &hello, sizeof(hello));
        } catch (...) {
            ::close(fd);
            throw;
        }
        if (hello <= rank || hello >= world || conn_[hello] != -1) {
            ::close(fd);
            throw std::runtime_error("local rendezvous: unexpected hello");
        }
        conn_[hello] = fd;
    }
}

LocalRendezvous::~LocalRendezvous() { close_all(); }

void LocalRendezvous::send_bytes(int peer, const void *data, size_t size)
{
    write_all(conn_.at(peer), data, size);
}

void LocalRendezvous::recv_bytes(int peer, void *data, size_t size)
{
    read_all(conn_.at(peer), data, size);
}

void LocalRendezvous::send_fd(int peer, int fd)
{
    char payload = 'F';
    iovec iov{&payload, 1};
    alignas(cmsghdr) char control[CMSG_SPACE(sizeof(int))];
    std::memset(control, 0, sizeof(control));
    msghdr msg{};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = control;
    msg.msg_controllen = sizeof(control);
    cmsghdr *cm = CMSG_FIRSTHDR(&msg);
    cm->cmsg_level = SOL_SOCKET;
    cm->cmsg_type = SCM_RIGHTS;
    cm->cmsg_len = CMSG_LEN(sizeof(int));
    std::memcpy(CMSG_DATA(cm), &fd, sizeof(int));
    for (;;) {
        const ssize_t n = ::sendmsg(conn_.at(peer), &msg, MSG_NOSIGNAL);
        if (n == 1) { return; }
        if (n < 0 && errno == EINTR) { continue; }
        fail("sendmsg(SCM_RIGHTS)");
    }
}

int LocalRendezvous::recv_fd(int peer)
{
    char payload = 0;
    iovec iov{&payload, 1};
    alignas(cmsghdr) char control[CMSG_SPACE(sizeof(int))];
    std::memset(control, 0, sizeof(control));
    msghdr msg{};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = control;
    msg.msg_controllen = sizeof(control);
    for (;;) {
        const ssize_t n = ::recvmsg(conn_.at(peer), &msg, MSG_CMSG_CLOEXEC);
        if (n == 1) { break; }
        if (n < 0 && errno == EINTR) { continue; }
        if (n == 0) { throw std::runtime_error("local rendezvous: peer closed"); }
        fail("recvmsg(SCM_RIGHTS)");
    }
    cmsghdr *cm = CMSG_FIRSTHDR(&msg);
    if (cm == nullptr || cm->cmsg_level != SOL_SOCKET || cm->cmsg_type != SCM_RIGHTS) {
        throw std::runtime_error("local rendezvous: no descriptor in message");
    }
    int fd = -1;
    std::memcpy(&fd, CMSG_DATA(cm), sizeof(int));
    return fd;
}

void LocalRendezvous::all_gather(const void *mine, size_t size,
                                 std::vector<std::vector<char>> &out)
{
    out.assign(world_, std::vector<char>(size));
    if (size > 0) { std::memcpy(out[rank_].data(), mine, size); }
    // Every rank sends before it receives, so what is in flight per socket must fit
    // the socket's buffer: large contributions (a table of a few thousand buffer
    // registrations) go in pieces, each exchanged completely before the next.
    constexpr size_t kPiece = 32u << 10;
    for (size_t at = 0; at < size; at += kPiece) {
        const size_t piece = std::min(kPiece, size - at);
        for (int p = 0; p < world_; ++p) {
            if (p != rank_) { send_bytes(p, static_cast<const char *>(mine) + at, piece); }
        }
        for (int p = 0; p < world_; ++p) {
            if (p != rank_) { recv_bytes(p, out[p].data() + at, piece); }
        }
    }
}

std::vector<int> LocalRendezvous::all_gather_fd(int my_fd)
{
    std::vector<int> fds(world_, -1);
    for (int p = 0; p < world_; ++p) {
        if (p != rank_) { send_fd(p, my_fd); }
    }
    for (int p = 0; p < world_; ++p) {
        if (p != rank_) { fds[p] = recv_fd(p); }
    }
    return fds;
}

bool LocalRendezvous::all_agree(bool mine)
{
    const char v = mine ? 1 : 0;
    std::vector<std::vector<char>> all;
    all_gather(&v, 1, all);
    bool ok = true;
    for (const auto &x : all) { ok = ok && x[0] != 0; }
    return ok;
}
}  // namespace stdml::collective::cuda
