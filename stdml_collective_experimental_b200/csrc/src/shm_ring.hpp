// Single-producer / single-consumer byte ring in shared memory: the data path
// of the third host back-end (STDML_COLLECTIVE_TRANSPORT=shm) between ranks of
// one host.  The sender creates the ring (memfd), passes the descriptor over
// the UNIX-domain connection it dialled, and both sides map it; message
// framing is the same byte stream as on a socket.  Sleeping is done with
// futexes on two sequence words; the socket stays open next to the ring and is
// what tells either side that the other one has gone.
// (The reference lists shared memory as a TODO: TODO:3,5 there.)
#pragma once
#include <atomic>
#include <cerrno>
#include <climits>
#include <cstddef>
#include <cstdint>
#include <cstring>

#include <linux/futex.h>
#include <sys/mman.h>
#include <sys/socket.h>
#include <sys/syscall.h>
#include <time.h>
#include <unistd.h>

namespace stdml::collective::rchan
{
struct shm_ring_header {
    alignas(64) std::atomic<uint64_t> head;  // bytes ever written
    alignas(64) std::atomic<uint64_t> tail;  // bytes ever read
    alignas(64) std::atomic<uint32_t> data_seq;   // bumped after every write
    std::atomic<uint32_t> consumer_waiting;
    alignas(64) std::atomic<uint32_t> space_seq;  // bumped after every read
    std::atomic<uint32_t> producer_waiting;
    alignas(64) std::atomic<uint32_t> closed;
    uint64_t capacity;
};

class shm_ring
{
    shm_ring_header *h_ = nullptr;
    char *data_ = nullptr;
    size_t map_bytes_ = 0;
    int liveness_fd_ = -1;  // the connection's socket: readable/closed when the peer died

    static long futex(std::atomic<uint32_t> *addr, int op, uint32_t val, const timespec *ts)
    {
        return ::syscall(SYS_futex, reinterpret_cast<uint32_t *>(addr), op, val, ts, nullptr, 0);
    }

    bool peer_gone() const
    {
        if (h_->closed.load(std::memory_order_acquire) != 0) { return true; }
        if (liveness_fd_ < 0) { return false; }
        char c;
        const ssize_t n = ::recv(liveness_fd_, &c, 1, MSG_PEEK | MSG_DONTWAIT);
        return n == 0 || (n < 0 && errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR);
    }

    static void nap(std::atomic<uint32_t> *seq, std::atomic<uint32_t> *flag, uint32_t seen)
    {
        flag->store(1, std::memory_order_seq_cst);
        if (seq->load(std::memory_order_seq_cst) == seen) {
            timespec ts{0, 100 * 1000 * 1000};  // re-check liveness every 100 ms
            futex(seq, FUTEX_WAIT, seen, &ts);
        }
        flag->store(0, std::memory_order_relaxed);
    }

    static void bump(std::atomic<uint32_t> *seq, std::atomic<uint32_t> *flag)
    {
        seq->fetch_add(1, std::memory_order_seq_cst);
        if (flag->load(std::memory_order_seq_cst) != 0) { futex(seq, FUTEX_WAKE, INT_MAX, nullptr); }
    }

  public:
    static constexpr size_t default_capacity = 8u << 20;

    static size_t bytes_for(size_t capacity) { return sizeof(shm_ring_header) + capacity; }

    // maps `fd` (which holds bytes_for(capacity) bytes); create = initialise it
    bool open(int fd, size_t capacity, bool create, int liveness_fd)
    {
        map_bytes_ = bytes_for(capacity);
        void *p = ::mmap(nullptr, map_bytes_, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
        if (p == MAP_FAILED) { return false; }
        h_ = static_cast<shm_ring_header *>(p);
        data_ = static_cast<char *>(p) + sizeof(shm_ring_header);
        liveness_fd_ = liveness_fd;
        if (create) {
            new (h_) shm_ring_header();
            h_->head.store(0);
            h_->tail.store(0);
            h_->data_seq.store(0);
            h_->space_seq.store(0);
            h_->consumer_waiting.store(0);
            h_->producer_waiting.store(0);
            h_->closed.store(0);
            h_->capacity = capacity;
        }
        return h_->capacity == capacity;
    }

    ~shm_ring()
    {
        if (h_ != nullptr) { ::munmap(h_, map_bytes_); }
    }

    bool valid() const { return h_ != nullptr; }

    void close()
    {
        if (h_ == nullptr) { return; }
        h_->closed.store(1, std::memory_order_release);
        bump(&h_->data_seq, &h_->consumer_waiting);
        bump(&h_->space_seq, &h_->producer_waiting);
    }

    // producer: all n bytes, in pieces as space frees up; false if the consumer is gone
    bool write(const void *src, size_t n)
    {
        const char *p = static_cast<const char *>(src);
        const uint64_t cap = h_->capacity;
        while (n > 0) {
            const uint64_t head = h_->head.load(std::memory_order_relaxed);
            const uint32_t seen = h_->space_seq.load(std::memory_order_seq_cst);
            const uint64_t tail = h_->tail.load(std::memory_order_acquire);
            const uint64_t room = cap - (head - tail);
            if (room == 0) {
                if (peer_gone()) { return false; }
                nap(&h_->space_seq, &h_->producer_waiting, seen);
                continue;
            }
            const size_t k = static_cast<size_t>(room < n ? room : n);
            const size_t at = static_cast<size_t>(head % cap);
            const size_t first = k < cap - at ? k : static_cast<size_t>(cap - at);
            std::memcpy(data_ + at, p, first);
            std::memcpy(data_, p + first, k - first);
            h_->head.store(head + k, std::memory_order_release);
            bump(&h_->data_seq, &h_->consumer_waiting);
            p += k;
            n -= k;
        }
        return true;
    }

    // consumer: exactly n bytes; false if the producer has gone before that
    bool read(void *dst, size_t n)
    {
        char *p = static_cast<char *>(dst);
        const uint64_t cap = h_->capacity;
        while (n > 0) {
            const uint64_t tail = h_->tail.load(std::memory_order_relaxed);
            const uint32_t seen = h_->data_seq.load(std::memory_order_seq_cst);
            const uint64_t head = h_->head.load(std::memory_order_acquire);
            const uint64_t avail = head - tail;
            if (avail == 0) {
                if (peer_gone()) {
                    // the producer may have written and closed in one go: look once more
                    if (h_->head.load(std::memory_order_acquire) == tail) { return false; }
                    continue;
                }
                nap(&h_->data_seq, &h_->consumer_waiting, seen);
                continue;
            }
            const size_t k = static_cast<size_t>(avail < n ? avail : n);
            const size_t at = static_cast<size_t>(tail % cap);
            const size_t first = k < cap - at ? k : static_cast<size_t>(cap - at);
            std::memcpy(p, data_ + at, first);
            std::memcpy(p + first, data_, k - first);
            h_->tail.store(tail + k, std::memory_order_release);
            bump(&h_->space_seq, &h_->producer_waiting);
            p += k;
            n -= k;
        }
        return true;
    }
};
}  // namespace stdml::collective::rchan
