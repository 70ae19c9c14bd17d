// Host-to-device / device-to-host copies whose host side is ordinary pageable memory (stack arrays, new[],
// malloc -- what every program written for the reference passes to libreCuMemCpy, e.g.
// tests/dma_chronological_consistency/main.cpp:33-39).
//
// The copy engines can only reach page-locked memory, so a pageable transfer has to bounce through a pinned
// buffer.  Left to the CUDA runtime that bounce runs on one thread (11 GB/s HtoD, 21 GB/s DtoH measured on
// the B200 hosts).  Here each stream owns a small ring of pinned slots; a pool of worker threads copies the
// next slot while the copy engine is busy with the previous one, so the host copy and the DMA overlap and the
// host copy itself is spread over several cores.  The reference hands the raw pointer to the DMA engine
// (driverapi/src/cmdqueue.cpp:746-774), which only works with HMM-capable kernel modules.
#include <cstdlib>
#include <cstring>

#include "copy_pool.h"
#include "internal.h"

namespace lcu {
namespace {

CopyPool &pool() {
    static CopyPool *p = [] {
        int n = 8;
        if (const char *e = std::getenv("LIBRECUDA_STAGING_THREADS")) n = std::atoi(e);
        const int hw = (int)std::thread::hardware_concurrency();
        if (hw > 0 && n > hw) n = hw;
        if (n < 1) n = 1;
        return new CopyPool(n);  // lives until process exit
    }();
    return *p;
}

}  // namespace

// bit 0: non-temporal stores when draining a slot into the user's buffer (DtoH); bit 1: when filling a slot (HtoD)
static int nt_mode() {
    static int mode = [] {
        const char *e = std::getenv("LIBRECUDA_STAGING_NT");
        return e ? std::atoi(e) : 1;
    }();
    return mode;
}

bool is_pageable_host(const void *p) {
    cudaPointerAttributes attr{};
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return true;
    }
    return attr.type == cudaMemoryTypeUnregistered;
}

static libreCudaStatus_t ensure_ring(LibreCUstream st) {
    if (st->stage[0] != nullptr) LIBRECUDA_SUCCEED();
    for (int i = 0; i < kStageSlots; ++i) {
        LCU_CUDA(cudaHostAlloc(&st->stage[i], kStageBytes, cudaHostAllocDefault));
        LCU_CUDA(cudaEventCreateWithFlags(&st->stage_done[i], cudaEventDisableTiming));
    }
    LIBRECUDA_SUCCEED();
}

// Pageable host -> device on `lane`.  Returns once the whole source has been read (the DMA of the last
// slots may still be in flight; the ring's events protect their reuse).
libreCudaStatus_t staged_h2d(LibreCUstream st, cudaStream_t lane, void *dst, const void *src, size_t bytes) {
    LIBRECUDA_ERR_PROPAGATE(ensure_ring(st));
    const unsigned char *s = static_cast<const unsigned char *>(src);
    unsigned char *d = static_cast<unsigned char *>(dst);
    for (size_t off = 0; off < bytes; off += kStageBytes) {
        const size_t n = bytes - off < kStageBytes ? bytes - off : kStageBytes;
        const int slot = st->stage_next;
        st->stage_next = (slot + 1) % kStageSlots;
        if (st->stage_busy[slot]) LCU_CUDA(cudaEventSynchronize(st->stage_done[slot]));
        pool().copy(st->stage[slot], s + off, n, /*streaming=*/(nt_mode() & 2) != 0);
        LCU_CUDA(cudaMemcpyAsync(d + off, st->stage[slot], n, cudaMemcpyHostToDevice, lane));
        LCU_CUDA(cudaEventRecord(st->stage_done[slot], lane));
        st->stage_busy[slot] = true;
    }
    LIBRECUDA_SUCCEED();
}

// Device -> pageable host on `lane`.  Blocks until the destination holds the data (as a runtime copy into
// pageable memory would): the DMA of slot k+1 runs while the workers empty slot k.
libreCudaStatus_t staged_d2h(LibreCUstream st, cudaStream_t lane, void *dst, const void *src, size_t bytes) {
    LIBRECUDA_ERR_PROPAGATE(ensure_ring(st));
    const unsigned char *s = static_cast<const unsigned char *>(src);
    unsigned char *d = static_cast<unsigned char *>(dst);
    struct Pending {
        int slot;
        size_t off, n;
    };
    Pending q[kStageSlots];
    int head = 0, count = 0;
    auto drain_one = [&]() -> libreCudaStatus_t {
        const Pending p = q[head];
        head = (head + 1) % kStageSlots;
        --count;
        LCU_CUDA(cudaEventSynchronize(st->stage_done[p.slot]));
        pool().copy(d + p.off, st->stage[p.slot], p.n, /*streaming=*/(nt_mode() & 1) != 0);
        st->stage_busy[p.slot] = false;
        LIBRECUDA_SUCCEED();
    };
    for (size_t off = 0; off < bytes; off += kStageBytes) {
        const size_t n = bytes - off < kStageBytes ? bytes - off : kStageBytes;
        if (count == kStageSlots) LIBRECUDA_ERR_PROPAGATE(drain_one());
        const int slot = st->stage_next;
        st->stage_next = (slot + 1) % kStageSlots;
        if (st->stage_busy[slot]) LCU_CUDA(cudaEventSynchronize(st->stage_done[slot]));  // left over from an HtoD
        LCU_CUDA(cudaMemcpyAsync(st->stage[slot], s + off, n, cudaMemcpyDeviceToHost, lane));
        LCU_CUDA(cudaEventRecord(st->stage_done[slot], lane));
        st->stage_busy[slot] = true;
        q[(head + count) % kStageSlots] = Pending{slot, off, n};
        ++count;
    }
    while (count > 0) LIBRECUDA_ERR_PROPAGATE(drain_one());
    LIBRECUDA_SUCCEED();
}

void free_ring(LibreCUstream st) {
    for (int i = 0; i < kStageSlots; ++i) {
        if (st->stage[i]) {
            (void)cudaFreeHost(st->stage[i]);
            (void)cudaEventDestroy(st->stage_done[i]);
            st->stage[i] = nullptr;
        }
    }
}

}  // namespace lcu
