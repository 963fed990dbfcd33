#include <algorithm>
#include <cctype>
#include <cstring>
#include <stdexcept>

#include <arpa/inet.h>
#include <netdb.h>
#include <netinet/in.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <unistd.h>

#include <stdml/bits/collective/http.hpp>

namespace stdml::collective
{
std::optional<http_url> http_parse_url(const std::string &url)
{
    const std::string scheme = "http://";
    if (url.compare(0, scheme.size(), scheme) != 0) { return {}; }
    http_url u;
    const size_t host_begin = scheme.size();
    const size_t path_begin = url.find('/', host_begin);
    const std::string authority = url.substr(
        host_begin, path_begin == std::string::npos ? std::string::npos : path_begin - host_begin);
    if (authority.empty()) { return {}; }
    const size_t colon = authority.rfind(':');
    if (colon == std::string::npos) {
        u.host = authority;
    } else {
        u.host = authority.substr(0, colon);
        const std::string port = authority.substr(colon + 1);
        if (port.empty() || !std::all_of(port.begin(), port.end(), ::isdigit)) { return {}; }
        const long p = std::strtol(port.c_str(), nullptr, 10);
        if (p <= 0 || p > 65535) { return {}; }
        u.port = static_cast<uint16_t>(p);
    }
    if (u.host.empty()) { return {}; }
    u.path = path_begin == std::string::npos ? "/" : url.substr(path_begin);
    return u;
}

std::optional<size_t> http_content_length(const std::string &headers)
{
    std::string lower(headers);
    std::transform(lower.begin(), lower.end(), lower.begin(),
                   [](unsigned char c) { return static_cast<char>(std::tolower(c)); });
    const std::string key = "content-length:";
    const size_t pos = lower.find(key);
    if (pos == std::string::npos) { return {}; }
    size_t i = pos + key.size();
    while (i < lower.size() && (lower[i] == ' ' || lower[i] == '\t')) { ++i; }
    size_t n = 0;
    bool any = false;
    while (i < lower.size() && std::isdigit(static_cast<unsigned char>(lower[i]))) {
        n = n * 10 + static_cast<size_t>(lower[i] - '0');
        any = true;
        ++i;
    }
    if (!any) { return {}; }
    return n;
}

std::string http_make_request(const std::string &method, const http_url &u,
                              const std::string &body, const std::string &content_type)
{
    std::string r = method + " " + u.path + " HTTP/1.1\r\n";
    r += "Host: " + u.host + ":" + std::to_string(u.port) + "\r\n";
    r += "User-Agent: stdml-collective\r\nConnection: close\r\n";
    if (!body.empty() || method == "PUT" || method == "POST") {
        r += "Content-Type: " + content_type + "\r\n";
        r += "Content-Length: " + std::to_string(body.size()) + "\r\n";
    }
    r += "\r\n";
    r += body;
    return r;
}

namespace
{
void set_io_timeout(int fd, int timeout_ms)
{
    timeval tv;
    tv.tv_sec = timeout_ms / 1000;
    tv.tv_usec = (timeout_ms % 1000) * 1000;
    setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
    setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
}

bool send_all(int fd, const std::string &s)
{
    size_t off = 0;
    while (off < s.size()) {
        const ssize_t n = ::send(fd, s.data() + off, s.size() - off, MSG_NOSIGNAL);
        if (n <= 0) {
            if (n < 0 && errno == EINTR) { continue; }
            return false;
        }
        off += static_cast<size_t>(n);
    }
    return true;
}

// reads "head\r\n\r\nbody" with the body delimited by Content-Length or EOF
bool read_message(int fd, std::string &head, std::string &body, bool until_eof)
{
    std::string buf;
    char tmp[4096];
    size_t split = std::string::npos;
    while (split == std::string::npos) {
        const ssize_t n = ::recv(fd, tmp, sizeof(tmp), 0);
        if (n <= 0) {
            if (n < 0 && errno == EINTR) { continue; }
            return false;
        }
        buf.append(tmp, static_cast<size_t>(n));
        split = buf.find("\r\n\r\n");
        if (buf.size() > (16u << 20)) { return false; }
    }
    head = buf.substr(0, split);
    body = buf.substr(split + 4);
    const auto want = http_content_length(head);
    if (!want && !until_eof) {  // a request without a length has no body
        body.clear();
        return true;
    }
    while (!want || body.size() < *want) {
        const ssize_t n = ::recv(fd, tmp, sizeof(tmp), 0);
        if (n == 0) { break; }
        if (n < 0) {
            if (errno == EINTR) { continue; }
            return !want;
        }
        body.append(tmp, static_cast<size_t>(n));
        if (body.size() > (64u << 20)) { return false; }
    }
    if (want) {
        if (body.size() < *want) { return false; }
        body.resize(*want);
    }
    return true;
}

std::optional<http_response> roundtrip(const std::string &method, const std::string &url,
                                       const std::string &body, int timeout_ms)
{
    const auto u = http_parse_url(url);
    if (!u) { return {}; }
    addrinfo hints{}, *res = nullptr;
    hints.ai_family = AF_INET;
    hints.ai_socktype = SOCK_STREAM;
    if (getaddrinfo(u->host.c_str(), std::to_string(u->port).c_str(), &hints, &res) != 0 ||
        res == nullptr) {
        return {};
    }
    const int fd = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
    {
        int one = 1;  // see rchan.cpp: keeps this client's TIME_WAIT entry from blocking a later bind
        setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    }
    if (fd < 0) {
        freeaddrinfo(res);
        return {};
    }
    set_io_timeout(fd, timeout_ms);
    const bool connected = ::connect(fd, res->ai_addr, res->ai_addrlen) == 0;
    freeaddrinfo(res);
    std::optional<http_response> out;
    std::string head, payload;
    if (connected && send_all(fd, http_make_request(method, *u, body)) &&
        read_message(fd, head, payload, true)) {
        http_response r;
        if (std::sscanf(head.c_str(), "HTTP/%*d.%*d %d", &r.status) == 1) {
            r.body = std::move(payload);
            out = std::move(r);
        }
    }
    ::close(fd);
    return out;
}
}  // namespace

std::optional<http_response> http_get(const std::string &url, int timeout_ms)
{
    return roundtrip("GET", url, "", timeout_ms);
}

std::optional<http_response> http_put(const std::string &url, const std::string &body,
                                      int timeout_ms)
{
    return roundtrip("PUT", url, body, timeout_ms);
}

http_server::http_server(uint16_t port, handler h) : handler_(std::move(h))
{
    fd_ = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (fd_ < 0) { throw std::runtime_error("http_server: socket() failed"); }
    int one = 1;
    setsockopt(fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in a{};
    a.sin_family = AF_INET;
    a.sin_addr.s_addr = htonl(INADDR_ANY);
    a.sin_port = htons(port);
    if (::bind(fd_, reinterpret_cast<sockaddr *>(&a), sizeof(a)) != 0 || ::listen(fd_, 64) != 0) {
        ::close(fd_);
        fd_ = -1;
        throw std::runtime_error("http_server: cannot listen on port " + std::to_string(port));
    }
    socklen_t len = sizeof(a);
    getsockname(fd_, reinterpret_cast<sockaddr *>(&a), &len);
    port_ = ntohs(a.sin_port);
}

http_server::~http_server()
{
    stop();
    if (fd_ >= 0) { ::close(fd_); }
}

void http_server::start()
{
    thread_ = std::thread([this] { loop(); });
}

void http_server::stop()
{
    stopping_.store(true);
    if (thread_.joinable()) { thread_.join(); }
}

void http_server::loop()
{
    while (!stopping_.load()) {
        pollfd pfd{fd_, POLLIN, 0};
        if (::poll(&pfd, 1, 100) <= 0) { continue; }
        const int c = ::accept4(fd_, nullptr, nullptr, SOCK_CLOEXEC);
        if (c < 0) { continue; }
        set_io_timeout(c, 5000);
        std::string head, body;
        if (read_message(c, head, body, false)) {
            request rq;
            char method[16] = {0}, path[1024] = {0};
            if (std::sscanf(head.c_str(), "%15s %1023s", method, path) == 2) {
                rq.method = method;
                rq.path = path;
                rq.body = std::move(body);
                http_response rs;
                try {
                    rs = handler_(rq);
                } catch (const std::exception &e) {
                    rs.status = 500;
                    rs.body = e.what();
                }
                const char *reason = rs.status == 200 ? "OK" : (rs.status == 404 ? "Not Found" : "Error");
                std::string out = "HTTP/1.1 " + std::to_string(rs.status) + " " + reason +
                                  "\r\nContent-Type: application/json\r\nContent-Length: " +
                                  std::to_string(rs.body.size()) + "\r\nConnection: close\r\n\r\n" +
                                  rs.body;
                send_all(c, out);
            }
        }
        ::close(c);
    }
}
}  // namespace stdml::collective
