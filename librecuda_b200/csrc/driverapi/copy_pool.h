// Worker pool that spreads one host memcpy over several threads (used by the pageable-copy staging ring).
// Pure C++, no CUDA: tests/test_host_cpp.py builds it with the address and thread sanitizers.
#pragma once

#include <condition_variable>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <thread>
#include <vector>

#if defined(__x86_64__) || defined(_M_X64)
#include <emmintrin.h>
#define LCU_HAVE_SSE2_STREAM 1
#endif

namespace lcu {

// memcpy whose stores bypass the cache (non-temporal).  For a destination that will not be read again soon
// -- the user's buffer at the end of a device-to-host copy -- this avoids reading every destination line
// into the cache before overwriting it, which costs a third of the memory traffic of the copy.
inline void stream_copy(void *dst, const void *src, size_t n) {
#ifdef LCU_HAVE_SSE2_STREAM
    unsigned char *d = static_cast<unsigned char *>(dst);
    const unsigned char *s = static_cast<const unsigned char *>(src);
    if (n < 4096) {
        std::memcpy(d, s, n);
        return;
    }
    const size_t head = (16 - (reinterpret_cast<uintptr_t>(d) & 15)) & 15;
    std::memcpy(d, s, head);
    d += head;
    s += head;
    n -= head;
    const size_t blocks = n / 64;
    for (size_t i = 0; i < blocks; ++i) {
        const __m128i a = _mm_loadu_si128(reinterpret_cast<const __m128i *>(s));
        const __m128i b = _mm_loadu_si128(reinterpret_cast<const __m128i *>(s + 16));
        const __m128i c = _mm_loadu_si128(reinterpret_cast<const __m128i *>(s + 32));
        const __m128i e = _mm_loadu_si128(reinterpret_cast<const __m128i *>(s + 48));
        _mm_stream_si128(reinterpret_cast<__m128i *>(d), a);
        _mm_stream_si128(reinterpret_cast<__m128i *>(d + 16), b);
        _mm_stream_si128(reinterpret_cast<__m128i *>(d + 32), c);
        _mm_stream_si128(reinterpret_cast<__m128i *>(d + 48), e);
        s += 64;
        d += 64;
    }
    _mm_sfence();
    std::memcpy(d, s, n - blocks * 64);
#else
    std::memcpy(dst, src, n);
#endif
}

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
    // streaming = true: the destination is written with non-temporal stores (see stream_copy)
    void copy(void *dst, const void *src, size_t n, bool streaming = false) {
        if (n < ((size_t)1 << 20) || n_ <= 1) {
            if (streaming) stream_copy(dst, src, n);
            else std::memcpy(dst, src, n);
            return;
        }
        std::unique_lock<std::mutex> lk(m_);
        streaming_ = streaming;
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
            bool streaming;
            {
                std::unique_lock<std::mutex> lk(m_);
                cv_.wait(lk, [&] { return generation_ != seen; });
                seen = generation_;
                if (stop_) return;
                d = dst_;
                s = src_;
                n = bytes_;
                streaming = streaming_;
            }
            const size_t per = ((n / (size_t)n_) + 4095) & ~(size_t)4095;
            size_t lo = per * (size_t)idx, hi = lo + per;
            if (lo > n) lo = n;
            if (hi > n || idx == n_ - 1) hi = n;
            if (hi > lo) {
                if (streaming) stream_copy(d + lo, s + lo, hi - lo);
                else std::memcpy(d + lo, s + lo, hi - lo);
            }
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
    bool streaming_ = false;
    unsigned char *dst_ = nullptr;
    const unsigned char *src_ = nullptr;
    size_t bytes_ = 0;
    int pending_ = 0;
};


}  // namespace lcu
