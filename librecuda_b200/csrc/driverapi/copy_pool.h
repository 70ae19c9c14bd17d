// Worker pool that spreads one host memcpy over several threads (used by the pageable-copy staging ring).
// Pure C++, no CUDA: tests/test_host_cpp.py builds it with the address and thread sanitizers.
#pragma once

#include <condition_variable>
#include <cstddef>
#include <cstring>
#include <mutex>
#include <thread>
#include <vector>

namespace lcu {

// Fixed pool; copy() splits [0, n) into one slice per worker and returns when all slices are copied.
// One caller at a time (the libreCu* API is single-threaded by contract).
class CopyPool {
public:
    explicit CopyPool(int workers) : n_(workers) {
        for (int i = 0; i < n_; ++i) threads_.emplace_back([this, i] { loop(i); });
    }
    ~CopyPool() {
        {
            std::lock_guard<std::mutex> lk(m_);
            stop_ = true;
            ++generation_;
        }
        cv_.notify_all();
        for (auto &t : threads_) t.join();
    }
    void copy(void *dst, const void *src, size_t n) {
        if (n < ((size_t)1 << 20) || n_ <= 1) {
            std::memcpy(dst, src, n);
            return;
        }
        std::unique_lock<std::mutex> lk(m_);
        dst_ = static_cast<unsigned char *>(dst);
        src_ = static_cast<const unsigned char *>(src);
        bytes_ = n;
        pending_ = n_;
        ++generation_;
        cv_.notify_all();
        done_.wait(lk, [this] { return pending_ == 0; });
    }

private:
    void loop(int idx) {
        unsigned long long seen = 0;
        for (;;) {
            unsigned char *d;
            const unsigned char *s;
            size_t n;
            {
                std::unique_lock<std::mutex> lk(m_);
                cv_.wait(lk, [&] { return generation_ != seen; });
                seen = generation_;
                if (stop_) return;
                d = dst_;
                s = src_;
                n = bytes_;
            }
            const size_t per = ((n / (size_t)n_) + 4095) & ~(size_t)4095;
            size_t lo = per * (size_t)idx, hi = lo + per;
            if (lo > n) lo = n;
            if (hi > n || idx == n_ - 1) hi = n;
            if (hi > lo) std::memcpy(d + lo, s + lo, hi - lo);
            {
                std::lock_guard<std::mutex> lk(m_);
                if (--pending_ == 0) done_.notify_all();
            }
        }
    }
    int n_;
    std::vector<std::thread> threads_;
    std::mutex m_;
    std::condition_variable cv_, done_;
    unsigned long long generation_ = 0;
    bool stop_ = false;
    unsigned char *dst_ = nullptr;
    const unsigned char *src_ = nullptr;
    size_t bytes_ = 0;
    int pending_ = 0;
};


}  // namespace lcu
