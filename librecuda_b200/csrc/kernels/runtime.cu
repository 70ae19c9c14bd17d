// Process-wide state of the kernel layer: tunables, cached device properties, the sticky device error
// word, and the small timing helpers the benchmark uses on raw CUDA streams.
#include <cstdlib>
#include <cstring>
#include <string>

#include "common.cuh"
#include "lcb200_kernels.h"

extern "C" int lcb_tune(const char *name, int value);

namespace lcb {

static const Tuning kDefaults = {
        /*copy_vec_threads*/ 0,
        /*copy_vec_unroll*/ 0,
        /*copy_vec_ctas_sm*/ 0,
        /*copy_cache_mode*/ 2,
        /*tma_chunk*/ 32768,
        /*tma_stages*/ 2,
        /*tma_lookahead*/ 1,
        /*tma_ctas_sm*/ 0,
        /*tma_cache_hint*/ 0,
        /*auto_tma_min_mib*/ 2048,
        /*memset_path*/ 0,
        /*memset_unroll*/ 8,
        /*memset_threads*/ 256,
        /*memset_ctas_sm*/ 4096,
        /*memset_chunk*/ 32768,
        /*memset_issuers*/ 4,
        /*memset_bulk_ctas_sm*/ 2,
        /*memset_cache_hint*/ 0,
        /*pdl*/ 1,
        /*copy_vec_smem_pad*/ 0,
        /*tma_smem_pad*/ 0,
        /*memset_smem_pad*/ 0,
        /*fill_ctas_sm*/ 4096,
        /*axpb_ctas_sm*/ 16384,
        /*a2a_ctas_sm*/ 4096,
        /*tma2_depth*/ 2,
        /*tma2_stages*/ 8,
        /*tma2_chunk*/ 8192,
        /*peer_copy_engine*/ 64,
        /*bcast_piece_mib*/ 64,
        /*bcast_pull_ctas*/ 74,
        /*bcast_engine_piece_mib*/ 0,
};

Tuning &tuning() {
    static Tuning t = kDefaults;
    static bool env_read = false;
    if (!env_read) {  // LCB_TUNE="knob=value,knob=value": overrides for experiments, applied once
        env_read = true;
        if (const char *e = std::getenv("LCB_TUNE")) {
            std::string all(e);
            size_t pos = 0;
            while (pos < all.size()) {
                size_t end = all.find(',', pos);
                if (end == std::string::npos) end = all.size();
                const std::string item = all.substr(pos, end - pos);
                const size_t eq = item.find('=');
                if (eq != std::string::npos) lcb_tune(item.substr(0, eq).c_str(), std::atoi(item.c_str() + eq + 1));
                pos = end + 1;
            }
        }
    }
    return t;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

int check_launch() { return (int)cudaGetLastError(); }

}  // namespace lcb

extern "C" int lcb_tune(const char *name, int value) {
    using lcb::tuning;
    if (name == nullptr) return 1;
    if (std::strcmp(name, "reset") == 0) {  // back to the shipped configuration
        tuning() = lcb::kDefaults;
        return 0;
    }
#define LCB_KNOB(field)                  \
    if (std::strcmp(name, #field) == 0) { \
        tuning().field = value;          \
        return 0;                        \
    }
    LCB_KNOB(copy_vec_threads)
    LCB_KNOB(copy_vec_unroll)
    LCB_KNOB(copy_vec_ctas_sm)
    LCB_KNOB(copy_cache_mode)
    LCB_KNOB(tma_chunk)
    LCB_KNOB(tma_stages)
    LCB_KNOB(tma_lookahead)
    LCB_KNOB(tma_ctas_sm)
    LCB_KNOB(tma_cache_hint)
    LCB_KNOB(auto_tma_min_mib)
    LCB_KNOB(memset_path)
    LCB_KNOB(memset_unroll)
    LCB_KNOB(memset_threads)
    LCB_KNOB(memset_ctas_sm)
    LCB_KNOB(memset_chunk)
    LCB_KNOB(memset_issuers)
    LCB_KNOB(memset_bulk_ctas_sm)
    LCB_KNOB(memset_cache_hint)
    LCB_KNOB(pdl)
    LCB_KNOB(copy_vec_smem_pad)
    LCB_KNOB(tma_smem_pad)
    LCB_KNOB(memset_smem_pad)
    LCB_KNOB(fill_ctas_sm)
    LCB_KNOB(axpb_ctas_sm)
    LCB_KNOB(a2a_ctas_sm)
    LCB_KNOB(tma2_depth)
    LCB_KNOB(tma2_stages)
    LCB_KNOB(tma2_chunk)
    LCB_KNOB(peer_copy_engine)
    LCB_KNOB(bcast_piece_mib)
    LCB_KNOB(bcast_pull_ctas)
    LCB_KNOB(bcast_engine_piece_mib)
#undef LCB_KNOB
    return 1;
}

extern "C" int lcb_tune_get(const char *name) {
    using lcb::tuning;
    if (name == nullptr) return -1;
#define LCB_KNOB(field) \
    if (std::strcmp(name, #field) == 0) return tuning().field;
    LCB_KNOB(bcast_piece_mib)
    LCB_KNOB(bcast_pull_ctas)
    LCB_KNOB(bcast_engine_piece_mib)
    LCB_KNOB(peer_copy_engine)
    LCB_KNOB(a2a_ctas_sm)
    LCB_KNOB(pdl)
    LCB_KNOB(auto_tma_min_mib)
#undef LCB_KNOB
    return -1;
}

extern "C" int lcb_preload(void) {
    int rc = lcb::preload_copy_kernels();
    if (rc == 0) rc = lcb::preload_fill_kernels();
    return rc;
}

extern "C" const char *lcb_version(void) { return "lcb200 0.1 sm_100a"; }

// ---- event timers on a raw stream ---------------------------------------------------------------
struct lcbTimer_ {
    cudaEvent_t start, stop;
};

extern "C" int lcb_timer_create(void **timer_out) {
    if (timer_out == nullptr) return 1;
    lcbTimer_ *t = new lcbTimer_();
    cudaError_t err = cudaEventCreate(&t->start);
    if (err == cudaSuccess) err = cudaEventCreate(&t->stop);
    if (err != cudaSuccess) {
        delete t;
        return (int)err;
    }
    *timer_out = t;
    return 0;
}

extern "C" int lcb_timer_start(void *timer, lcbStream stream) {
    if (timer == nullptr) return 1;
    return (int)cudaEventRecord(static_cast<lcbTimer_ *>(timer)->start, static_cast<cudaStream_t>(stream));
}

extern "C" int lcb_timer_stop(void *timer, lcbStream stream) {
    if (timer == nullptr) return 1;
    return (int)cudaEventRecord(static_cast<lcbTimer_ *>(timer)->stop, static_cast<cudaStream_t>(stream));
}

extern "C" int lcb_timer_elapsed_ms(void *timer, float *ms_out) {
    if (timer == nullptr || ms_out == nullptr) return 1;
    lcbTimer_ *t = static_cast<lcbTimer_ *>(timer);
    cudaError_t err = cudaEventSynchronize(t->stop);
    if (err != cudaSuccess) return (int)err;
    return (int)cudaEventElapsedTime(ms_out, t->start, t->stop);
}

extern "C" int lcb_timer_destroy(void *timer) {
    if (timer == nullptr) return 1;
    lcbTimer_ *t = static_cast<lcbTimer_ *>(timer);
    cudaEventDestroy(t->start);
    cudaEventDestroy(t->stop);
    delete t;
    return 0;
}

extern "C" int lcb_stream_synchronize(lcbStream stream) {
    return (int)cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
}

extern "C" int lcb_stream_wait_stream(lcbStream waiter, lcbStream signaller) {
    cudaEvent_t ev = nullptr;
    cudaError_t err = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    if (err != cudaSuccess) return (int)err;
    err = cudaEventRecord(ev, static_cast<cudaStream_t>(signaller));
    if (err == cudaSuccess) err = cudaStreamWaitEvent(static_cast<cudaStream_t>(waiter), ev, 0);
    (void)cudaEventDestroy(ev);  // released by the runtime once the wait has consumed it
    return (int)err;
}

// ---- vendor paths, for side-by-side measurement only (never used by the library's own data path) ---------
extern "C" int lcb_vendor_memcpy_d2d(void *dst, const void *src, size_t bytes, lcbStream stream) {
    return (int)cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream));
}

extern "C" int lcb_vendor_memset_d8(void *dst, unsigned char value, size_t bytes, lcbStream stream) {
    return (int)cudaMemsetAsync(dst, value, bytes, static_cast<cudaStream_t>(stream));
}
