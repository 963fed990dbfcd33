// Exact-size reads and writes over a socket-like object, blocking or as polled
// tasks.  `Socket` needs recv_some / send_some as in TcpSocket.  Counterpart of
// include/stdml/bits/collective/net/ioutil.hpp:73-239 (basic_ioutil,
// io_exact_task): with a non-blocking socket an io_exact_task makes progress on
// every poll() and never blocks, which lets one thread drive many transfers
// through the task runtime.
#pragma once
#include <cstddef>
#include <memory>
#include <stdexcept>
#include <system_error>
#include <type_traits>

#include <stdml/bits/collective/task.hpp>

namespace stdml::collective
{
enum io_type { io_read, io_write };

template <typename Socket, io_type iot>
class io_exact_task : public task
{
    Socket &socket_;
    char *ptr_;
    size_t left_;
    std::error_code ec_;

  public:
    io_exact_task(Socket &socket, std::conditional_t<iot == io_read, void *, const void *> ptr,
                  size_t n)
        : socket_(socket), ptr_(static_cast<char *>(const_cast<void *>(ptr))), left_(n)
    {
    }

    void poll() override
    {
        if (left_ == 0 || ec_) { return; }
        const long n = iot == io_read ? socket_.recv_some(ptr_, left_, ec_)
                                      : socket_.send_some(ptr_, left_, ec_);
        if (n > 0) {
            ptr_ += n;
            left_ -= static_cast<size_t>(n);
        }
    }

    bool finished() override { return left_ == 0 || static_cast<bool>(ec_); }
    const std::error_code &error() const { return ec_; }
    size_t remaining() const { return left_; }
};

template <typename Socket, bool non_blocking = false>
class basic_ioutil
{
  public:
    static void read(Socket &socket, void *ptr, size_t n, std::error_code &ec)
    {
        io_exact_task<Socket, io_read> t(socket, ptr, n);
        t.finish();
        ec = t.error();
    }

    static void read(Socket &socket, void *ptr, size_t n)
    {
        std::error_code ec;
        read(socket, ptr, n, ec);
        if (ec) { throw std::system_error(ec, "read"); }
    }

    static void write(Socket &socket, const void *ptr, size_t n)
    {
        io_exact_task<Socket, io_write> t(socket, ptr, n);
        t.finish();
        if (t.error()) { throw std::system_error(t.error(), "write"); }
    }

    static std::unique_ptr<task> new_read_task(Socket &socket, void *ptr, size_t n)
    {
        return std::unique_ptr<task>(new io_exact_task<Socket, io_read>(socket, ptr, n));
    }

    static std::unique_ptr<task> new_write_task(Socket &socket, const void *ptr, size_t n)
    {
        return std::unique_ptr<task>(new io_exact_task<Socket, io_write>(socket, ptr, n));
    }

    template <typename T>
    static void read(Socket &socket, T &t)
    {
        static_assert(std::is_standard_layout<T>::value, "plain data only");
        read(socket, &t, sizeof(T));
    }

    template <typename T>
    static void write(Socket &socket, const T &t)
    {
        static_assert(std::is_standard_layout<T>::value, "plain data only");
        write(socket, &t, sizeof(T));
    }
};
}  // namespace stdml::collective
