// Process-wide state of the kernel layer: tunables, cached device properties, the sticky device error
// word, and the small timing helpers the benchmark uses on raw CUDA streams.
#include <cstdio>
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
        /*tma_chunk*/ 0,
        /*tma_stages*/ 2,
        /*tma_lookahead*/ 1,
        /*tma_ctas_sm*/ 0,
        /*tma_cache_hint*/ 0,
        /*auto_tma_min_mib*/ 96,
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
        /*phase_chunk*/ 32768,
        /*phase_stages*/ 6,
        /*phase_ns*/ 4000,
        /*bcast_ring_chunk_kib*/ 0,
        /*bcast_ring_ctas*/ 0,
        /*bcast_mc_piece_mib*/ 256,
        /*bcast_mc_slots*/ 2,
        /*bcast_mc_ctas*/ 64,
        /*bcast_ring_warp*/ 1,
        /*bcast_ring_tickets*/ 1,
};

static void apply_env_overrides() {  // LCB_TUNE="knob=value,knob=value": overrides for experiments
    const char *e = std::getenv("LCB_TUNE");
    if (e == nullptr) return;
    std::string all(e);
    size_t pos = 0;
    while (pos < all.size()) {
        size_t end = all.find(',', pos);
        if (end == std::string::npos) end = all.size();
        const std::string item = all.substr(pos, end - pos);
        const size_t eq = item.find('=');
        if (eq != std::string::npos && lcb_tune(item.substr(0, eq).c_str(), std::atoi(item.c_str() + eq + 1)) != 0)
            fprintf(stderr, "LCB_TUNE: '%s' refused (unknown knob or value out of range)\n", item.c_str());
        pos = end + 1;
    }
}

Tuning &tuning() {
    static Tuning t = kDefaults;
    static bool env_read = false;
    if (!env_read) {  // applied once at first use, and again after lcb_tune("reset", 0)
        env_read = true;
        apply_env_overrides();
    }
    return t;
}

// Accepted range of every knob.  A value outside it is refused and the previous value stays: a CTA of one
// warp has nobody to copy the tail bytes, a thread count of 0 divides by zero, more than 512 threads breaks
// the kernels' launch bounds, and ring shapes exist only as the instantiated (stages, lookahead) pairs.
static bool knob_value_ok(const char *name, int v) {
    auto is = [&](const char *n) { return std::strcmp(name, n) == 0; };
    auto threads_ok = [&](int lo) { return v >= lo && v <= 512 && (v % 32) == 0; };
    if (is("copy_vec_threads")) return v == 0 || threads_ok(64);
    if (is("copy_vec_unroll")) return v == 0 || v == 1 || v == 2 || v == 4 || v == 8;
    if (is("memset_threads")) return threads_ok(64);
    if (is("memset_unroll")) return v == 1 || v == 2 || v == 4 || v == 8;
    if (is("copy_cache_mode")) return v >= 0 && v <= 4;
    if (is("tma_chunk") && v == 0) return true;  // 0: chunk, stages and lookahead chosen by size
    if (is("phase_stages")) return v == 2 || v == 3 || v == 4 || v == 6 || v == 12 || v == 24;
    if (is("phase_ns")) return v >= 0 && v <= 1000000;
    if (is("tma_chunk") || is("tma2_chunk") || is("memset_chunk") || is("phase_chunk")) return v >= 1024 && v <= 65536 && (v & 127) == 0;
    if (is("tma_stages")) return v >= 2 && v <= 16;
    if (is("tma_lookahead")) return v >= 1 && v <= 12;
    if (is("tma2_stages")) return v >= 4 && v <= 24;
    if (is("tma2_depth")) return v >= 1 && v <= 8;
    if (is("memset_path")) return v >= 0 && v <= 2;
    if (is("memset_issuers")) return v >= 1 && v <= 8;
    if (is("memset_bulk_ctas_sm")) return v >= 1 && v <= 32;
    if (is("tma_cache_hint") || is("memset_cache_hint") || is("pdl") || is("bcast_ring_warp") || is("bcast_ring_tickets")) return v == 0 || v == 1;
    if (is("auto_tma_min_mib")) return v >= -1;
    if (is("copy_vec_smem_pad") || is("tma_smem_pad") || is("memset_smem_pad")) return v >= 0 && v <= 200 * 1024;
    if (is("bcast_pull_ctas")) return v >= 0 && v <= 65536;
    if (is("bcast_mc_piece_mib")) return v >= 1 && v <= 1024;
    if (is("bcast_ring_chunk_kib")) return v == 0 || (v >= 4 && v <= 65536 && (v & (v - 1)) == 0);
    if (is("bcast_ring_ctas")) return v >= 0 && v <= 4096;
    if (is("bcast_mc_slots")) return v >= 2 && v <= 16;
    return v >= 0;  // grid caps, thresholds and piece sizes: any non-negative value
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

#define LCB_ALL_KNOBS(X) \
    X(copy_vec_threads) \
    X(copy_vec_unroll) \
    X(copy_vec_ctas_sm) \
    X(copy_cache_mode) \
    X(tma_chunk) \
    X(tma_stages) \
    X(tma_lookahead) \
    X(tma_ctas_sm) \
    X(tma_cache_hint) \
    X(auto_tma_min_mib) \
    X(memset_path) \
    X(memset_unroll) \
    X(memset_threads) \
    X(memset_ctas_sm) \
    X(memset_chunk) \
    X(memset_issuers) \
    X(memset_bulk_ctas_sm) \
    X(memset_cache_hint) \
    X(pdl) \
    X(copy_vec_smem_pad) \
    X(tma_smem_pad) \
    X(memset_smem_pad) \
    X(fill_ctas_sm) \
    X(axpb_ctas_sm) \
    X(a2a_ctas_sm) \
    X(tma2_depth) \
    X(tma2_stages) \
    X(tma2_chunk) \
    X(peer_copy_engine) \
    X(bcast_piece_mib) \
    X(bcast_pull_ctas) \
    X(bcast_engine_piece_mib) \
    X(phase_chunk) \
    X(phase_stages) \
    X(phase_ns) \
    X(bcast_ring_chunk_kib) \
    X(bcast_ring_ctas) \
    X(bcast_mc_piece_mib) \
    X(bcast_mc_slots) \
    X(bcast_mc_ctas) \
    X(bcast_ring_warp) \
    X(bcast_ring_tickets)

extern "C" int lcb_tune(const char *name, int value) {
    using lcb::tuning;
    if (name == nullptr) return 1;
    if (std::strcmp(name, "reset") == 0) {  // back to the configuration the process started with
        tuning() = lcb::kDefaults;
        lcb::apply_env_overrides();
        return 0;
    }
    if (!lcb::knob_value_ok(name, value)) return 1;
#define LCB_KNOB(field)                  \
    if (std::strcmp(name, #field) == 0) { \
        tuning().field = value;          \
        return 0;                        \
    }
    LCB_ALL_KNOBS(LCB_KNOB)
#undef LCB_KNOB
    return 1;
}

extern "C" int lcb_tune_get(const char *name) {
    using lcb::tuning;
    if (name == nullptr) return -1;
#define LCB_KNOB(field) \
    if (std::strcmp(name, #field) == 0) return tuning().field;
    LCB_ALL_KNOBS(LCB_KNOB)
#undef LCB_KNOB
    return -1;
}

extern "C" int lcb_preload(void) {
    int rc = lcb::preload_copy_kernels();
    if (rc == 0) rc = lcb::preload_fill_kernels();
    if (rc == 0) rc = lcb::setup_error_mirror();
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
