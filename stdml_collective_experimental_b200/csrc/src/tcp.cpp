#include <cerrno>
#include <cstring>

#include <arpa/inet.h>
#include <fcntl.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <stdml/bits/collective/net/tcp.hpp>

namespace stdml::collective
{
InetAddr::InetAddr(uint16_t port, uint32_t host)
{
    std::memset(&addr_, 0, sizeof(addr_));
    addr_.sin_family = AF_INET;
    addr_.sin_port = htons(port);
    addr_.sin_addr.s_addr = htonl(host);
}

int InetAddr::bind(int sock) const { return ::bind(sock, get(), sizeof(addr_)); }
int InetAddr::connect(int sock) const { return ::connect(sock, get(), sizeof(addr_)); }

TcpSocket::TcpSocket() : fd_(::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0))
{
    if (fd_ < 0) { throw std::system_error(errno, std::generic_category(), "socket"); }
    int one = 1;  // keeps a client's TIME_WAIT entry from blocking a later bind of its local port
    setsockopt(fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
}

TcpSocket::TcpSocket(int fd) : fd_(fd) {}

TcpSocket::~TcpSocket()
{
    if (fd_ >= 0) { ::close(fd_); }
}

void TcpSocket::set_non_blocking(bool on)
{
    const int flags = ::fcntl(fd_, F_GETFL, 0);
    ::fcntl(fd_, F_SETFL, on ? (flags | O_NONBLOCK) : (flags & ~O_NONBLOCK));
}

long TcpSocket::recv_some(void *data, size_t size, std::error_code &ec)
{
    const ssize_t n = ::recv(fd_, data, size, 0);
    if (n > 0) { return n; }
    if (n == 0) {
        ec = std::make_error_code(std::errc::connection_reset);
        return -1;
    }
    if (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) { return 0; }
    ec = std::error_code(errno, std::generic_category());
    return -1;
}

long TcpSocket::send_some(const void *data, size_t size, std::error_code &ec)
{
    const ssize_t n = ::send(fd_, data, size, MSG_NOSIGNAL);
    if (n >= 0) { return n; }
    if (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) { return 0; }
    ec = std::error_code(errno, std::generic_category());
    return -1;
}

int TcpSocket::recv(void *data, size_t size)
{
    char *p = static_cast<char *>(data);
    while (size > 0) {
        std::error_code ec;
        const long n = recv_some(p, size, ec);
        if (n < 0) { return ec.value(); }
        if (n == 0) {  // non-blocking socket: wait until readable
            pollfd pfd{fd_, POLLIN, 0};
            ::poll(&pfd, 1, 100);
            continue;
        }
        p += n;
        size -= static_cast<size_t>(n);
    }
    return 0;
}

int TcpSocket::send(const void *data, size_t size)
{
    const char *p = static_cast<const char *>(data);
    while (size > 0) {
        std::error_code ec;
        const long n = send_some(p, size, ec);
        if (n < 0) { return ec.value(); }
        if (n == 0) {
            pollfd pfd{fd_, POLLOUT, 0};
            ::poll(&pfd, 1, 100);
            continue;
        }
        p += n;
        size -= static_cast<size_t>(n);
    }
    return 0;
}

TcpServer::TcpServer(uint16_t port, uint32_t host) : port_(port), host_(host) {}

TcpServer::~TcpServer()
{
    stop();
    if (sock_ >= 0) { ::close(sock_); }
}

void TcpServer::start()
{
    sock_ = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (sock_ < 0) { throw std::system_error(errno, std::generic_category(), "socket"); }
    int one = 1;
    ::setsockopt(sock_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    if (InetAddr(port_, host_).bind(sock_) != 0 || ::listen(sock_, 128) != 0) {
        throw std::system_error(errno, std::generic_category(), "bind/listen");
    }
    sockaddr_in a{};
    socklen_t len = sizeof(a);
    ::getsockname(sock_, reinterpret_cast<sockaddr *>(&a), &len);
    port_ = ntohs(a.sin_port);
}

std::unique_ptr<TcpSocket> TcpServer::wait_accept()
{
    while (!stopped_.load()) {
        pollfd pfd{sock_, POLLIN, 0};
        if (::poll(&pfd, 1, 100) <= 0) { continue; }
        const int fd = ::accept4(sock_, nullptr, nullptr, SOCK_CLOEXEC);
        if (fd >= 0) { return std::make_unique<TcpSocket>(fd); }
    }
    return nullptr;
}

void TcpServer::serve(const Handler &handle)
{
    while (auto s = wait_accept()) { handle(std::move(s)); }
}

void TcpServer::stop() { stopped_.store(true); }

TcpClient::TcpClient(uint16_t port, uint32_t host) : port_(port), host_(host) {}

void TcpClient::dial(int *code)
{
    const int rc = InetAddr(port_, host_).connect(sock_.fd());
    const int err = rc == 0 ? 0 : errno;
    if (code != nullptr) {
        *code = err;
        return;
    }
    if (err != 0) { throw std::system_error(err, std::generic_category(), "connect"); }
    int one = 1;
    ::setsockopt(sock_.fd(), IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
}

void TcpClient::write(const void *data, size_t size)
{
    const int err = sock_.send(data, size);
    if (err != 0) { throw std::system_error(err, std::generic_category(), "send"); }
}

std::vector<char> TcpClient::Talk(const void *data, size_t size)
{
    const uint32_t n = static_cast<uint32_t>(size);
    write(&n, sizeof(n));
    write(data, size);
    uint32_t m = 0;
    int err = sock_.recv(&m, sizeof(m));
    std::vector<char> reply(m);
    if (err == 0 && m > 0) { err = sock_.recv(reply.data(), m); }
    if (err != 0) { throw std::system_error(err, std::generic_category(), "recv"); }
    return reply;
}
}  // namespace stdml::collective
