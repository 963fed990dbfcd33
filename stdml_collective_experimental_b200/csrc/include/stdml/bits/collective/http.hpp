// Minimal HTTP/1.1 client (GET, PUT) and a tiny single-threaded server, enough
// for the elastic config service.  The reference has the request helpers
// (include/stdml/bits/collective/http.hpp, src/stdml/collective/http.cpp:29-103)
// and a client only in its Networking-TS back-end; the server side comes from
// KungFu's Go launcher there.
#pragma once
#include <atomic>
#include <cstdint>
#include <functional>
#include <map>
#include <optional>
#include <string>
#include <thread>

namespace stdml::collective
{
struct http_url {
    std::string host;
    uint16_t port = 80;
    std::string path = "/";
};

std::optional<http_url> http_parse_url(const std::string &url);
// value of Content-Length in a header block; nullopt when absent
std::optional<size_t> http_content_length(const std::string &headers);
std::string http_make_request(const std::string &method, const http_url &u,
                              const std::string &body = "",
                              const std::string &content_type = "application/json");

struct http_response {
    int status = 0;
    std::string body;
};

// nullopt: could not connect or malformed answer
std::optional<http_response> http_get(const std::string &url, int timeout_ms = 5000);
std::optional<http_response> http_put(const std::string &url, const std::string &body,
                                      int timeout_ms = 5000);

class http_server
{
  public:
    struct request {
        std::string method, path, body;
    };
    using handler = std::function<http_response(const request &)>;

    // port 0 picks a free port (see port())
    http_server(uint16_t port, handler h);
    ~http_server();
    uint16_t port() const { return port_; }
    void start();
    void stop();

  private:
    void loop();
    int fd_ = -1;
    uint16_t port_ = 0;
    handler handler_;
    std::atomic<bool> stopping_{false};
    std::thread thread_;
};
}  // namespace stdml::collective
