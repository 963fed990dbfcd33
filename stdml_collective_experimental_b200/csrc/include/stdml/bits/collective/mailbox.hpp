// Rendezvous tables keyed by (source peer, message name).
//   mailbox : eager messages.  The network thread allocates, reads the body and
//             queues it; the receiver may come later.
//   slotbox : rendezvous messages.  The receiver posts its destination pointer
//             and blocks; the network thread reads the body straight into it.
// Counterpart of include/stdml/bits/collective/mailbox.hpp:15-62.  Unlike the
// reference, a slot is a FIFO of any depth on both sides and a body whose
// destination is not posted yet is parked in a temporary buffer, so a network
// thread never blocks behind one unposted buffer while it holds other tensors'
// messages (the head-of-line blocking that deadlocks the reference's
// group_all_reduce when ranks submit tensors in different orders).
#pragma once
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <utility>

#include <stdml/bits/collective/address.hpp>
#include <stdml/bits/collective/buffer.hpp>
#include <stdml/bits/collective/channel.hpp>

namespace stdml::collective
{
// One rendezvous point.  The receiver posts a destination (pointer + capacity);
// the network thread delivers a message body with put().  If a destination is
// already posted the body is read straight into it (zero-copy); if not, the
// body is read into a temporary buffer and handed over when the receiver
// arrives, so the network thread never waits for the receiver.  A body longer
// than the posted capacity is rejected (the reference trusts the sender's
// length, src/stdml/collective/send_recv.cpp:6-12).
class slot
{
    struct ticket {
        void *ptr = nullptr;
        size_t cap = 0;
        // written under the slot's mutex; atomic so that the holder of a pending can
        // ask "is there anything left to withdraw?" without touching the slot, which
        // may be gone by the time a finished operation's handle is destroyed
        std::atomic<bool> done{false};
        bool ok = false;
        std::atomic<bool> withdrawn{false};  // cancelled before any body was matched to it
    };
    std::mutex mu_;
    std::condition_variable finished_;
    std::deque<std::shared_ptr<ticket>> waiting_;
    std::deque<buffer> early_;

    static bool deliver(ticket &t, const buffer &b)
    {
        if (b.len > t.cap) { return false; }
        if (b.len > 0) { std::memcpy(t.ptr, b.data.get(), b.len); }
        return true;
    }

    std::shared_ptr<ticket> post_ticket(void *ptr, size_t cap)
    {
        auto t = std::make_shared<ticket>();
        t->ptr = ptr;
        t->cap = cap;
        std::lock_guard<std::mutex> lk(mu_);
        if (!early_.empty()) {
            t->ok = deliver(*t, early_.front());
            t->done = true;
            early_.pop_front();
        } else {
            waiting_.push_back(t);
        }
        return t;
    }

  public:
    // Blocks until a body has been written into ptr; false if it did not fit.
    bool get(void *ptr, size_t cap)
    {
        auto t = post_ticket(ptr, cap);
        std::unique_lock<std::mutex> lk(mu_);
        finished_.wait(lk, [&] { return t->done.load(); });
        return t->ok;
    }

    // Like get(), but gives up after `ms` milliseconds (ms <= 0: never): returns
    // -1 on timeout, else 1 (delivered) or 0 (did not fit).  A ticket that
    // timed out is withdrawn, so a late body is parked for the next receiver.
    int get_for(void *ptr, size_t cap, long long ms)
    {
        if (ms <= 0) { return get(ptr, cap) ? 1 : 0; }
        auto t = post_ticket(ptr, cap);
        std::unique_lock<std::mutex> lk(mu_);
        if (!finished_.wait_for(lk, std::chrono::milliseconds(ms), [&] { return t->done.load(); })) {
            for (auto it = waiting_.begin(); it != waiting_.end(); ++it) {
                if (*it == t) {
                    waiting_.erase(it);
                    return -1;
                }
            }
            // a network thread has taken the ticket and is filling it right now
            finished_.wait(lk, [&] { return t->done.load(); });
        }
        return t->ok ? 1 : 0;
    }

    // A posted destination.  wait(ms) returns 1 (delivered), 0 (did not fit) or
    // -1 (not yet; ms <= 0 waits without limit).  A pending that is given up
    // must be cancel()led, or a late body would be written through a pointer
    // that its owner no longer holds; cancel() itself waits if a network
    // thread is filling the destination at that moment.
    class pending
    {
        friend class slot;
        slot *s_ = nullptr;
        std::shared_ptr<ticket> t_;

      public:
        pending() = default;
        explicit operator bool() const { return s_ != nullptr; }

        int wait(long long ms)
        {
            std::unique_lock<std::mutex> lk(s_->mu_);
            if (ms <= 0) {
                s_->finished_.wait(lk, [&] { return t_->done.load(); });
            } else if (!s_->finished_.wait_for(lk, std::chrono::milliseconds(ms),
                                               [&] { return t_->done.load(); })) {
                return -1;
            }
            return t_->ok ? 1 : 0;
        }

        // true when nothing can be written through this post any more (delivered or
        // withdrawn); does not touch the slot
        bool settled() const { return !t_ || t_->done.load() || t_->withdrawn.load(); }

        // wait() without waiting
        int ready()
        {
            std::lock_guard<std::mutex> lk(s_->mu_);
            return !t_->done ? -1 : (t_->ok ? 1 : 0);
        }

        // true: withdrawn, nothing will be written; false: it was (being) delivered
        bool cancel()
        {
            std::unique_lock<std::mutex> lk(s_->mu_);
            if (t_->done) { return false; }
            if (t_->withdrawn) { return true; }  // cancelled before: still nothing will be written
            for (auto it = s_->waiting_.begin(); it != s_->waiting_.end(); ++it) {
                if (*it == t_) {
                    s_->waiting_.erase(it);
                    t_->withdrawn = true;
                    return true;
                }
            }
            s_->finished_.wait(lk, [&] { return t_->done.load(); });
            return false;
        }
    };

    pending post_pending(void *ptr, size_t cap)
    {
        pending p;
        p.s_ = this;
        p.t_ = post_ticket(ptr, cap);
        return p;
    }

    // Posts now; the returned function waits for the body.
    std::function<bool()> post(void *ptr, size_t cap)
    {
        auto t = post_ticket(ptr, cap);
        return [this, t] {
            std::unique_lock<std::mutex> lk(mu_);
            finished_.wait(lk, [&] { return t->done.load(); });
            return t->ok;
        };
    }

    // Posts now; the returned function tells, without blocking, whether the
    // body has arrived (for the polled task runtime).
    std::function<bool()> post_polled(void *ptr, size_t cap)
    {
        auto t = post_ticket(ptr, cap);
        return [this, t] {
            std::lock_guard<std::mutex> lk(mu_);
            return t->done.load();
        };
    }

    // Network side: `read_body(dst)` must read exactly `len` bytes into dst.
    void put(size_t len, const std::function<bool(void *)> &read_body)
    {
        std::shared_ptr<ticket> t;
        {
            std::lock_guard<std::mutex> lk(mu_);
            if (!waiting_.empty()) {
                t = waiting_.front();
                waiting_.pop_front();
            }
        }
        if (t && len <= t->cap) {
            const bool ok = read_body(t->ptr);
            std::lock_guard<std::mutex> lk(mu_);
            t->ok = ok;
            t->done = true;
            finished_.notify_all();
            return;
        }
        buffer b = alloc_buffer(len);
        const bool ok = read_body(b.data.get());
        std::lock_guard<std::mutex> lk(mu_);
        if (t) {  // posted, but too small: drained above, report failure
            t->ok = false;
            t->done = true;
            finished_.notify_all();
            return;
        }
        if (!ok) { return; }
        if (!waiting_.empty()) {
            t = waiting_.front();
            waiting_.pop_front();
            t->ok = deliver(*t, b);
            t->done = true;
            finished_.notify_all();
        } else {
            early_.push_back(std::move(b));
        }
    }
};

template <typename Box>
class basic_mailbox
{
    using key = std::pair<uint64_t, std::string>;
    std::mutex mu_;
    std::map<key, std::unique_ptr<Box>> boxes_;

  public:
    Box *require(const peer_id &src, const std::string &name)
    {
        std::lock_guard<std::mutex> lk(mu_);
        auto &b = boxes_[key(src.hash(), name)];
        if (!b) { b.reset(new Box); }
        return b.get();
    }

    size_t size()
    {
        std::lock_guard<std::mutex> lk(mu_);
        return boxes_.size();
    }
};

struct eager_box : channel<buffer> {
    eager_box() : channel<buffer>(1u << 16) {}
};

using mailbox = basic_mailbox<eager_box>;
using slotbox = basic_mailbox<slot>;
}  // namespace stdml::collective
