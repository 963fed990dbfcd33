// Thin RAII wrappers over POSIX TCP sockets: the lowest public layer of the
// host transport.  Counterpart of include/stdml/bits/collective/net/tcp.hpp
// (TcpSocket / TcpServer / TcpClient / InetAddr); errors are exceptions or
// error codes here, never exit(1).
#pragma once
#include <atomic>
#include <cstddef>
#include <cstdint>
#include <functional>
#include <memory>
#include <system_error>
#include <vector>

#include <netinet/in.h>

namespace stdml::collective
{
constexpr uint32_t any_addr = 0;
constexpr uint32_t localhost = (127u << 24) | 1u;

class InetAddr
{
    sockaddr_in addr_;

  public:
    InetAddr(uint16_t port, uint32_t host);
    const sockaddr *get() const { return reinterpret_cast<const sockaddr *>(&addr_); }
    int bind(int sock) const;
    int connect(int sock) const;
};

class TcpSocket
{
    int fd_;

  public:
    TcpSocket();                 // a fresh socket
    explicit TcpSocket(int fd);  // adopts fd
    ~TcpSocket();
    TcpSocket(const TcpSocket &) = delete;
    TcpSocket &operator=(const TcpSocket &) = delete;

    int fd() const { return fd_; }
    void set_non_blocking(bool on);
    // exactly `size` bytes; 0 on success, else errno (ECONNRESET on end of stream)
    int recv(void *data, size_t size);
    int send(const void *data, size_t size);
    // at most `size` bytes, non-blocking friendly: bytes moved, 0 when it would
    // block, -1 with ec set on error / end of stream
    long recv_some(void *data, size_t size, std::error_code &ec);
    long send_some(const void *data, size_t size, std::error_code &ec);
};

class TcpServer
{
    uint16_t port_;
    uint32_t host_;
    int sock_ = -1;
    std::atomic<bool> stopped_{false};

  public:
    explicit TcpServer(uint16_t port, uint32_t host = any_addr);
    ~TcpServer();
    uint16_t port() const { return port_; }  // the bound port (port 0 picks one)
    void start();                            // bind + listen; throws std::system_error
    std::unique_ptr<TcpSocket> wait_accept();  // nullptr after stop()
    using Handler = std::function<void(std::unique_ptr<TcpSocket>)>;
    void serve(const Handler &handle);  // until stop()
    void stop();
};

class TcpClient
{
    uint16_t port_;
    uint32_t host_;
    TcpSocket sock_;

  public:
    explicit TcpClient(uint16_t port, uint32_t host = localhost);
    void dial(int *code = nullptr);  // throws unless `code` is given
    TcpSocket &socket() { return sock_; }
    void write(const void *data, size_t size);
    // request / response with a u32 length prefix in both directions
    std::vector<char> Talk(const void *data, size_t size);
    std::vector<char> Talk(const std::vector<char> &buf) { return Talk(buf.data(), buf.size()); }
};
}  // namespace stdml::collective
