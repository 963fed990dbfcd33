// POSIX-socket implementation of the rchan endpoints.  One listening socket
// per peer; one reader thread per inbound connection; one outgoing connection
// per (type, target), dialled on first use.  TCP_NODELAY is set on every
// socket: control messages are latency-bound (the reference leaves Nagle on,
// src/stdml/collective/platforms/linux/socket_opt.c:41-45).
#include <algorithm>
#include <atomic>
#include <cerrno>
#include <cstddef>
#include <chrono>
#include <cstring>
#include <list>
#include <stdexcept>
#include <thread>
#include <vector>

#include <arpa/inet.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/mman.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <sys/uio.h>
#include <sys/un.h>
#include <unistd.h>

#include <stdml/bits/collective/config.hpp>
#include <stdml/bits/collective/log.hpp>
#include <stdml/bits/collective/rchan.hpp>
#include <stdml/bits/collective/stat.hpp>

#include "shm_ring.hpp"

namespace stdml::collective::rchan
{
namespace
{
void tune_socket(int fd)
{
    int one = 1;
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    int buf = 4 << 20;
    setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &buf, sizeof(buf));
    setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &buf, sizeof(buf));
}

// An outgoing connection takes an ephemeral local port, which can be the very
// port a peer or runner of a later job wants to listen on; its TIME_WAIT entry
// blocks that bind for a minute unless BOTH sockets were marked reusable.
void mark_reusable(int fd)
{
    int one = 1;
    setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
}

sockaddr_in to_sockaddr(const peer_id &id)
{
    sockaddr_in a;
    std::memset(&a, 0, sizeof(a));
    a.sin_family = AF_INET;
    a.sin_port = htons(id.port);
    a.sin_addr.s_addr = htonl(id.ipv4);
    return a;
}

// Second back-end: ranks of one host may talk over abstract UNIX-domain stream
// sockets instead of TCP loopback.  The framing is identical; only dialling
// and listening differ.  Every server listens on both, so mixed settings still
// connect.  STDML_COLLECTIVE_TRANSPORT = tcp | unix | shm | auto; unset means
// auto: peers of this host are dialled over a UNIX socket with a shared-memory
// ring (without one where none can be made).  unix: no ring; shm: the ring is
// required.  In all three a peer whose UNIX socket does not answer (it listens
// on TCP only, or lives in another network namespace) is dialled over TCP.
enum class transport_mode { tcp, unix_socket, shm, automatic };

transport_mode transport()
{
    static const transport_mode m = [] {
        const std::string v = safe_getenv("STDML_COLLECTIVE_TRANSPORT");
        if (v == "tcp") { return transport_mode::tcp; }
        if (v == "unix") { return transport_mode::unix_socket; }
        if (v == "shm") { return transport_mode::shm; }
        return transport_mode::automatic;
    }();
    return m;
}

// (automatic mode) a ring could not be set up once: plain UNIX sockets from then on
std::atomic<bool> g_ring_unavailable{false};

bool prefer_shared_memory()
{
    const transport_mode m = transport();
    return m == transport_mode::shm ||
           (m == transport_mode::automatic && !g_ring_unavailable.load(std::memory_order_relaxed));
}

bool prefer_unix_sockets() { return transport() != transport_mode::tcp; }

// Third back-end (STDML_COLLECTIVE_TRANSPORT=shm): the dialler of a UNIX-domain
// connection announces a ring with this bit of conn_header::type, creates it
// and hands its descriptor over the socket; from then on the socket carries no
// payload and only signals that the other side has gone.
constexpr uint16_t conn_type_ring_bit = 0x8000;

struct ring_offer {
    uint64_t capacity;
};

bool send_fd(int sock, int fd, const ring_offer &offer)
{
    msghdr msg{};
    iovec iov{const_cast<ring_offer *>(&offer), sizeof(offer)};
    alignas(cmsghdr) char ctl[CMSG_SPACE(sizeof(int))] = {};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = ctl;
    msg.msg_controllen = sizeof(ctl);
    cmsghdr *c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int));
    std::memcpy(CMSG_DATA(c), &fd, sizeof(int));
    ssize_t n;
    do {
        n = ::sendmsg(sock, &msg, MSG_NOSIGNAL);
    } while (n < 0 && errno == EINTR);
    return n == static_cast<ssize_t>(sizeof(offer));
}

int recv_fd(int sock, ring_offer &offer)
{
    msghdr msg{};
    iovec iov{&offer, sizeof(offer)};
    alignas(cmsghdr) char ctl[CMSG_SPACE(sizeof(int))] = {};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = ctl;
    msg.msg_controllen = sizeof(ctl);
    ssize_t n;
    do {
        n = ::recvmsg(sock, &msg, MSG_CMSG_CLOEXEC | MSG_WAITALL);
    } while (n < 0 && errno == EINTR);
    if (n != static_cast<ssize_t>(sizeof(offer))) { return -1; }
    for (cmsghdr *c = CMSG_FIRSTHDR(&msg); c != nullptr; c = CMSG_NXTHDR(&msg, c)) {
        if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) {
            int fd;
            std::memcpy(&fd, CMSG_DATA(c), sizeof(int));
            return fd;
        }
    }
    return -1;
}

socklen_t to_unix_addr(const peer_id &id, sockaddr_un &a)
{
    std::memset(&a, 0, sizeof(a));
    a.sun_family = AF_UNIX;
    const std::string name = "stdml-rchan/" + id.str();  // abstract namespace: leading NUL
    std::memcpy(a.sun_path + 1, name.data(), name.size());
    return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + name.size());
}

bool read_exact(int fd, void *data, size_t size)
{
    char *p = static_cast<char *>(data);
    while (size > 0) {
        const ssize_t n = ::recv(fd, p, size, 0);
        if (n > 0) {
            p += n;
            size -= static_cast<size_t>(n);
        } else if (n == 0) {
            return false;
        } else if (errno != EINTR) {
            return false;
        }
    }
    return true;
}

bool write_iov(int fd, iovec *iov, int cnt)
{
    while (cnt > 0) {
        msghdr msg{};
        msg.msg_iov = iov;
        msg.msg_iovlen = static_cast<size_t>(cnt);
        ssize_t n = ::sendmsg(fd, &msg, MSG_NOSIGNAL);
        if (n < 0) {
            if (errno == EINTR) { continue; }
            return false;
        }
        while (cnt > 0 && n >= static_cast<ssize_t>(iov->iov_len)) {
            n -= static_cast<ssize_t>(iov->iov_len);
            ++iov;
            --cnt;
        }
        if (cnt > 0 && n > 0) {
            iov->iov_base = static_cast<char *>(iov->iov_base) + n;
            iov->iov_len -= static_cast<size_t>(n);
        }
    }
    return true;
}

// Per-connection receive buffer: small messages (header, name, short bodies)
// are served from one recv() of whatever the socket holds, large bodies are
// read straight into their destination once the buffered part is copied out.
struct recv_buffer {
    std::vector<char> data;
    size_t head = 0, tail = 0;
    shm_ring *ring = nullptr;  // set: the ring is the buffer, the socket carries nothing

    recv_buffer() : data(256 << 10) {}

    bool read(int fd, void *dst, size_t n)
    {
        if (ring != nullptr) { return ring->read(dst, n); }
        char *out = static_cast<char *>(dst);
        while (n > 0) {
            if (head < tail) {
                const size_t take = std::min(n, tail - head);
                std::memcpy(out, data.data() + head, take);
                head += take;
                out += take;
                n -= take;
                continue;
            }
            head = tail = 0;
            if (n >= data.size() / 2) { return read_exact(fd, out, n); }
            const ssize_t got = ::recv(fd, data.data(), data.size(), 0);
            if (got > 0) {
                tail = static_cast<size_t>(got);
            } else if (got == 0 || errno != EINTR) {
                return false;
            }
        }
        return true;
    }
};

class reader_impl final : public message_reader
{
    int fd_;
    recv_buffer *buf_;
    uint32_t len_ = 0;

  public:
    reader_impl(int fd, recv_buffer *buf) : fd_(fd), buf_(buf) {}

    std::optional<received_header> read_header() override
    {
        STDML_COLLECTIVE_PROFILE_RATE("read_header", 0);
        received_header h;
        if (!buf_->read(fd_, &h.name_len, 4)) { return {}; }
        if (h.name_len > (1u << 20)) { return {}; }  // not our protocol
        h.name.resize(h.name_len);
        uint32_t tail[2];
        if (!buf_->read(fd_, h.name.data(), h.name_len) || !buf_->read(fd_, tail, 8)) { return {}; }
        h.flags = tail[0];
        h.len = tail[1];
        len_ = h.len;
        return h;
    }

    bool read_body(void *data) override
    {
        STDML_COLLECTIVE_PROFILE_RATE("read_body", len_);
        return len_ == 0 || buf_->read(fd_, data, len_);
    }
};

class connection_impl final : public connection
{
    int fd_;
    conn_type type_;
    peer_id src_;
    std::mutex send_mu_;
    recv_buffer rbuf_;  // used by the (single) thread that reads this connection
    std::unique_ptr<shm_ring> ring_;  // dialler: written by send(); acceptor: read by next()

  public:
    connection_impl(int fd, conn_type type, peer_id src, std::unique_ptr<shm_ring> ring = nullptr)
        : fd_(fd), type_(type), src_(src), ring_(std::move(ring))
    {
        rbuf_.ring = ring_.get();
    }

    ~connection_impl() override
    {
        if (ring_) { ring_->close(); }
        if (fd_ >= 0) { ::close(fd_); }
    }

    int fd() const { return fd_; }

    void shutdown_now()
    {
        if (fd_ >= 0) { ::shutdown(fd_, SHUT_RDWR); }
    }

    conn_type type() const override { return type_; }
    peer_id src() const override { return src_; }

    std::unique_ptr<message_reader> next() override
    {
        return std::unique_ptr<message_reader>(new reader_impl(fd_, &rbuf_));
    }

    void send(const char *name, const void *data, size_t size, uint32_t flags) override
    {
        STDML_COLLECTIVE_PROFILE_RATE("send", size);
        if (size > 0xffffffffull) { throw std::length_error("rchan: message longer than 4 GiB"); }
        const uint32_t name_len = static_cast<uint32_t>(std::strlen(name));
        const uint32_t len = static_cast<uint32_t>(size);
        iovec iov[5];
        iov[0] = {&const_cast<uint32_t &>(name_len), 4};
        iov[1] = {const_cast<char *>(name), name_len};
        iov[2] = {&flags, 4};
        iov[3] = {&const_cast<uint32_t &>(len), 4};
        iov[4] = {const_cast<void *>(data), size};
        std::lock_guard<std::mutex> lk(send_mu_);
        if (ring_) {
            // header fields in one piece, so that a short message costs one wake-up
            char head[256];
            if (12 + static_cast<size_t>(name_len) <= sizeof(head)) {
                std::memcpy(head, &name_len, 4);
                std::memcpy(head + 4, name, name_len);
                std::memcpy(head + 4 + name_len, &flags, 4);
                std::memcpy(head + 8 + name_len, &len, 4);
                if (ring_->write(head, 12 + name_len) && (size == 0 || ring_->write(data, size))) {
                    return;
                }
            } else {
                bool ok = true;
                for (int i = 0; ok && i < (size > 0 ? 5 : 4); ++i) {
                    ok = ring_->write(iov[i].iov_base, iov[i].iov_len);
                }
                if (ok) { return; }
            }
            throw peer_failure(src_, "rchan: send to " + src_.str() + " failed: peer has gone");
        }
        if (!write_iov(fd_, iov, size > 0 ? 5 : 4)) {
            throw peer_failure(src_, "rchan: send to " + src_.str() + " failed: " +
                                          std::strerror(errno));
        }
    }
};

size_t ring_capacity()
{
    static const size_t v = [] {
        const auto mb = parse_env_int("STDML_COLLECTIVE_SHM_RING_MB").value_or(8);
        return static_cast<size_t>(std::min<int64_t>(std::max<int64_t>(mb, 1), 1024)) << 20;
    }();
    return v;
}

// dialler's side: create, map and hand over
std::unique_ptr<shm_ring> offer_ring(int sock)
{
    const size_t cap = ring_capacity();
    const int mfd = ::memfd_create("stdml-rchan-ring", MFD_CLOEXEC);
    if (mfd < 0) { return nullptr; }
    std::unique_ptr<shm_ring> ring(new shm_ring);
    const bool ok = ::ftruncate(mfd, static_cast<off_t>(shm_ring::bytes_for(cap))) == 0 &&
                    ring->open(mfd, cap, true, sock) && send_fd(sock, mfd, ring_offer{cap});
    ::close(mfd);  // the mapping and the receiver's copy keep the memory alive
    return ok ? std::move(ring) : nullptr;
}

// acceptor's side
std::unique_ptr<shm_ring> accept_ring(int sock)
{
    ring_offer offer{};
    const int mfd = recv_fd(sock, offer);
    if (mfd < 0) { return nullptr; }
    std::unique_ptr<shm_ring> ring(new shm_ring);
    struct stat st {};
    const bool ok = offer.capacity >= 4096 && offer.capacity <= (size_t(1) << 30) &&
                    ::fstat(mfd, &st) == 0 &&
                    static_cast<size_t>(st.st_size) >= shm_ring::bytes_for(offer.capacity) &&
                    ring->open(mfd, offer.capacity, false, sock);
    ::close(mfd);
    return ok ? std::move(ring) : nullptr;
}
}  // namespace

int64_t connect_timeout_ms()
{
    static const int64_t v =
        parse_env_int("STDML_COLLECTIVE_CONNECT_TIMEOUT_MS").value_or(120000);
    return v;
}

std::unique_ptr<connection> connection::dial(const peer_id remote, const conn_type type,
                                             const peer_id local, int64_t patience_ms)
{
    using clock = std::chrono::steady_clock;
    const auto t0 = clock::now();
    const int64_t limit = patience_ms >= 0 ? std::max<int64_t>(patience_ms, 1) : connect_timeout_ms();
    const sockaddr_in addr = to_sockaddr(remote);
    int wait_ms = 2;
    const bool same_host =
        remote.ipv4 == local.ipv4 || local.ipv4 == 0 || (remote.ipv4 >> 24) == 127u;
    const bool automatic = transport() == transport_mode::automatic;
    for (;;) {
        // one round: the UNIX socket of a peer of this host first, then TCP (a peer
        // elsewhere, or one that listens on TCP only)
        for (int attempt = 0; attempt < 2; ++attempt) {
            const bool local_peer = attempt == 0 && prefer_unix_sockets() && same_host;
            if (attempt == 0 && !local_peer) { continue; }              // nothing to try before TCP
            const int fd =
                ::socket(local_peer ? AF_UNIX : AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
            if (fd < 0) { throw std::runtime_error("rchan: socket() failed"); }
            mark_reusable(fd);
            int rc;
            if (local_peer) {
                sockaddr_un ua;
                const socklen_t ul = to_unix_addr(remote, ua);
                rc = ::connect(fd, reinterpret_cast<const sockaddr *>(&ua), ul);
            } else {
                rc = ::connect(fd, reinterpret_cast<const sockaddr *>(&addr), sizeof(addr));
            }
            if (rc == 0) {
                tune_socket(fd);
                const bool want_ring = local_peer && prefer_shared_memory();
                const uint16_t wire_type = static_cast<uint16_t>(type) |
                                           (want_ring ? conn_type_ring_bit : uint16_t(0));
                conn_header h{wire_type, local.port, local.ipv4};
                connection_ack ack{};
                iovec iov{&h, sizeof(h)};
                if (write_iov(fd, &iov, 1) && read_exact(fd, &ack, sizeof(ack))) {
                    if (!want_ring) {
                        return std::unique_ptr<connection>(new connection_impl(fd, type, remote));
                    }
                    if (auto ring = offer_ring(fd)) {
                        return std::unique_ptr<connection>(
                            new connection_impl(fd, type, remote, std::move(ring)));
                    }
                    ::close(fd);
                    if (automatic) {
                        // no shared memory to be had here: dial again, without a ring
                        g_ring_unavailable.store(true, std::memory_order_relaxed);
                        attempt = -1;
                        continue;
                    }
                    throw std::runtime_error("rchan: cannot set up a shared-memory ring to " +
                                             remote.str());
                }
            }
            ::close(fd);
        }
        const auto waited =
            std::chrono::duration_cast<std::chrono::milliseconds>(clock::now() - t0).count();
        if (limit > 0 && waited > limit) {
            throw peer_failure(remote, "rchan: could not reach " + remote.str() + " within " +
                                           std::to_string(limit) + " ms");
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(wait_ms));
        wait_ms = std::min(wait_ms * 2, 200);  // the peer may simply not be up yet
    }
}

namespace
{
// One TCP connect + handshake with a deadline; the socket is blocking again on
// return.  -1 if `remote` does not accept or acknowledge in time.
int handshake_with_deadline(const peer_id &remote, const peer_id &local, conn_type type,
                            int timeout_ms)
{
    using clock = std::chrono::steady_clock;
    const auto t0 = clock::now();
    const auto left = [&] {
        const auto spent =
            std::chrono::duration_cast<std::chrono::milliseconds>(clock::now() - t0).count();
        return static_cast<int>(std::max<int64_t>(0, timeout_ms - spent));
    };
    const int fd = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC | SOCK_NONBLOCK, 0);
    if (fd < 0) { return -1; }
    mark_reusable(fd);
    const auto fail = [&] {
        ::close(fd);
        return -1;
    };
    const sockaddr_in addr = to_sockaddr(remote);
    if (::connect(fd, reinterpret_cast<const sockaddr *>(&addr), sizeof(addr)) != 0) {
        if (errno != EINPROGRESS) { return fail(); }
        pollfd p{fd, POLLOUT, 0};
        if (::poll(&p, 1, left()) <= 0) { return fail(); }
        int err = 0;
        socklen_t len = sizeof(err);
        if (::getsockopt(fd, SOL_SOCKET, SO_ERROR, &err, &len) != 0 || err != 0) { return fail(); }
    }
    tune_socket(fd);
    const conn_header h{static_cast<uint16_t>(type), local.port, local.ipv4};
    if (::send(fd, &h, sizeof(h), MSG_NOSIGNAL) != static_cast<ssize_t>(sizeof(h))) { return fail(); }
    connection_ack ack{};
    size_t have = 0;
    while (have < sizeof(ack)) {
        pollfd p{fd, POLLIN, 0};
        if (::poll(&p, 1, left()) <= 0) { return fail(); }
        const ssize_t n = ::recv(fd, reinterpret_cast<char *>(&ack) + have, sizeof(ack) - have, 0);
        if (n <= 0) { return fail(); }
        have += static_cast<size_t>(n);
    }
    const int flags = ::fcntl(fd, F_GETFL, 0);
    if (flags < 0 || ::fcntl(fd, F_SETFL, flags & ~O_NONBLOCK) != 0) { return fail(); }
    return fd;
}
}  // namespace

double ping(const peer_id &remote, const peer_id &local, int timeout_ms)
{
    const auto t0 = std::chrono::steady_clock::now();
    const int fd = handshake_with_deadline(remote, local, conn_ping, timeout_ms);
    if (fd < 0) { return -1; }
    ::close(fd);
    return std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();
}

std::unique_ptr<connection> connection::dial_once(const peer_id remote, const conn_type type,
                                                  const peer_id local, int timeout_ms)
{
    const int fd = handshake_with_deadline(remote, local, type, timeout_ms);
    if (fd < 0) { return nullptr; }
    return std::unique_ptr<connection>(new connection_impl(fd, type, remote));
}

bool conn_handler::handle_next(connection *conn, msg_handler *h)
{
    auto reader = conn->next();
    const auto mh = reader->read_header();
    if (!mh) { return false; }
    return (*h)(*mh, reader.get(), conn->src());
}

size_t conn_handler::handle_to_end(connection *conn, msg_handler *h)
{
    size_t n = 0;
    while (handle_next(conn, h)) { ++n; }
    return n;
}

// ------------------------------------------------------------------- client
namespace
{
class client_impl final : public client
{
    const peer_id self_;
    const conn_type type_;
    std::mutex mu_;
    std::map<uint64_t, std::shared_ptr<connection>> conns_;
    std::atomic<int64_t> patience_ms_{-1};

    std::shared_ptr<connection> require(const peer_id &target)
    {
        std::lock_guard<std::mutex> lk(mu_);
        auto it = conns_.find(target.hash());
        if (it == conns_.end()) {
            // (nothing is stored when dial throws)
            it = conns_.emplace(target.hash(), connection::dial(target, type_, self_, patience_ms_.load())).first;
        }
        return it->second;
    }

  public:
    client_impl(peer_id self, conn_type type) : self_(self), type_(type) {}

    void send(const peer_id target, const char *name, const void *data, size_t size,
              uint32_t flags) override
    {
        require(target)->send(name, data, size, flags);
    }

    std::unique_ptr<connection> dial(peer_id target, conn_type type) override
    {
        return connection::dial(target, type, self_);
    }

    void reset_peers(const peer_list &ids) override
    {
        std::lock_guard<std::mutex> lk(mu_);
        for (const auto &id : ids) { conns_.erase(id.hash()); }
    }

    void set_dial_patience_ms(int64_t ms) override { patience_ms_.store(ms); }
};
}  // namespace

std::unique_ptr<client> client::New(peer_id self, conn_type type)
{
    return std::unique_ptr<client>(new client_impl(self, type));
}

client *client_pool::require(conn_type type)
{
    std::lock_guard<std::mutex> lk(mu_);
    auto &c = clients_[type];
    if (!c) {
        c = client::New(self_, type);
        c->set_dial_patience_ms(patience_ms_);
    }
    return c.get();
}

void client_pool::set_dial_patience_ms(int64_t ms)
{
    std::lock_guard<std::mutex> lk(mu_);
    patience_ms_ = ms;
    for (auto &kv : clients_) { kv.second->set_dial_patience_ms(ms); }
}

void client_pool::reset_peers(const peer_list &ids)
{
    std::lock_guard<std::mutex> lk(mu_);
    for (auto &kv : clients_) { kv.second->reset_peers(ids); }
}

// ------------------------------------------------------------------- server
namespace
{
class server_impl final : public server
{
    const peer_id self_;
    conn_handler *handler_;
    int listen_fd_ = -1;
    int unix_fd_ = -1;  // same service on an abstract UNIX socket
    std::atomic<bool> stopping_{false};
    std::thread accept_thread_;
    std::mutex mu_;
    struct session {
        std::thread th;
        int wake_fd = -1;  // dup of the connection's socket, to shut it down from stop()
        std::atomic<bool> finished{false};
    };
    std::list<session> sessions_;

    void open()
    {
        listen_fd_ = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
        if (listen_fd_ < 0) { throw std::runtime_error("rchan: socket() failed"); }
        int one = 1;
        setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
        sockaddr_in a = to_sockaddr(self_);
        a.sin_addr.s_addr = htonl(INADDR_ANY);
        // a loopback alias (127.0.0.x, x > 1) stands for a host of its own when
        // several hosts are emulated on one machine: bind the alias itself so
        // that the same port can be used by each of them
        if ((self_.ipv4 >> 24) == 127u && self_.ipv4 != ((127u << 24) | 1u)) {
            a.sin_addr.s_addr = htonl(self_.ipv4);
        }
        // a predecessor on the same port (a rank that was removed and is being
        // replaced, a previous job) may still be closing: give it a moment
        int rc = -1;
        for (int attempt = 0; attempt < 50; ++attempt) {
            rc = ::bind(listen_fd_, reinterpret_cast<sockaddr *>(&a), sizeof(a));
            if (rc == 0 || errno != EADDRINUSE) { break; }
            std::this_thread::sleep_for(std::chrono::milliseconds(100));
        }
        if (rc != 0) {
            const std::string why = std::strerror(errno);
            ::close(listen_fd_);
            listen_fd_ = -1;
            throw std::runtime_error("rchan: cannot bind " + self_.str() + ": " + why);
        }
        if (::listen(listen_fd_, 128) != 0) { throw std::runtime_error("rchan: listen() failed"); }
        // (a rank that is told to speak TCP only listens on TCP only, like a rank of
        // the reference; its peers' diallers then fall back to TCP)
        unix_fd_ = prefer_unix_sockets() ? ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0) : -1;
        if (unix_fd_ >= 0) {
            sockaddr_un ua;
            const socklen_t ul = to_unix_addr(self_, ua);
            if (::bind(unix_fd_, reinterpret_cast<sockaddr *>(&ua), ul) != 0 ||
                ::listen(unix_fd_, 128) != 0) {
                ::close(unix_fd_);  // TCP alone still serves everybody
                unix_fd_ = -1;
            }
        }
    }

    void reap()
    {
        for (auto it = sessions_.begin(); it != sessions_.end();) {
            if (it->finished.load()) {
                it->th.join();
                if (it->wake_fd >= 0) { ::close(it->wake_fd); }
                it = sessions_.erase(it);
            } else {
                ++it;
            }
        }
    }

    void accept_loop()
    {
        while (!stopping_.load()) {
            pollfd pfds[2] = {{listen_fd_, POLLIN, 0}, {unix_fd_, POLLIN, 0}};
            const int r = ::poll(pfds, unix_fd_ >= 0 ? 2 : 1, 100);
            if (r <= 0) { continue; }
            const int ready = (pfds[0].revents & POLLIN) ? listen_fd_ : unix_fd_;
            const int fd = ::accept4(ready, nullptr, nullptr, SOCK_CLOEXEC);
            if (fd < 0) { continue; }
            tune_socket(fd);
            conn_header h{};
            connection_ack ack{0};
            iovec iov{&ack, sizeof(ack)};
            if (!read_exact(fd, &h, sizeof(h)) || !write_iov(fd, &iov, 1)) {
                ::close(fd);
                continue;
            }
            std::unique_ptr<shm_ring> ring;
            if ((h.type & conn_type_ring_bit) != 0) {
                ring = accept_ring(fd);
                if (!ring) {
                    log(WARN) << "rchan: a peer offered a shared-memory ring that cannot be mapped";
                    ::close(fd);
                    continue;
                }
            }
            std::lock_guard<std::mutex> lk(mu_);
            if (stopping_.load()) {
                ::close(fd);
                break;
            }
            reap();
            sessions_.emplace_back();
            session &s = sessions_.back();
            auto *conn = new connection_impl(
                fd, static_cast<conn_type>(h.type & ~conn_type_ring_bit),
                peer_id{h.src_ipv4, h.src_port}, std::move(ring));
            s.wake_fd = ::dup(fd);
            s.th = std::thread([this, conn, &s] {
                try {
                    (*handler_)(std::unique_ptr<connection>(conn));
                } catch (const std::exception &e) {
                    log(WARN) << "rchan: connection handler failed:" << e.what();
                }
                s.finished.store(true);
            });
        }
    }

  public:
    server_impl(peer_id self, conn_handler *handler) : self_(self), handler_(handler) {}

    ~server_impl() override { stop(); }

    void serve() override
    {
        if (listen_fd_ < 0) { open(); }
        accept_loop();
    }

    void start() override
    {
        if (listen_fd_ < 0) { open(); }
        accept_thread_ = std::thread([this] { accept_loop(); });
    }

    void stop() override
    {
        if (stopping_.exchange(true)) { return; }
        if (accept_thread_.joinable()) { accept_thread_.join(); }
        {
            // wake every reader thread: they see end-of-stream and return
            std::lock_guard<std::mutex> lk(mu_);
            for (auto &s : sessions_) {
                if (s.wake_fd >= 0) { ::shutdown(s.wake_fd, SHUT_RDWR); }
            }
        }
        for (auto &s : sessions_) {
            if (s.th.joinable()) { s.th.join(); }
            if (s.wake_fd >= 0) { ::close(s.wake_fd); }
        }
        sessions_.clear();
        if (unix_fd_ >= 0) {
            ::close(unix_fd_);
            unix_fd_ = -1;
        }
        if (listen_fd_ >= 0) {
            ::close(listen_fd_);
            listen_fd_ = -1;
        }
    }
};
}  // namespace

std::unique_ptr<server> server::New(const peer_id self, conn_handler *handler)
{
    return std::unique_ptr<server>(new server_impl(self, handler));
}
}  // namespace stdml::collective::rchan
