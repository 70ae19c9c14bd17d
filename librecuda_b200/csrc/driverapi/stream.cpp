// Stream / event ordering layer and the stream-recorded operations (copies, memset, launches).
//
// Semantics kept from the reference's NvCommandQueue (driverapi/src/cmdqueue.cpp):
//  * operations are recorded and reach the GPU at Commence (:200-218, :821-868); Await blocks until the
//    submitted work is complete (:272-277, :334-357);
//  * async=false orders an operation after everything recorded before it, async=true lets it overlap
//    earlier operations of the same stream (:480-487, :715-727);
//  * events are timestamped markers in the stream (:896-955).
// What changed: ordering is resolved on the GPU.  An ordered operation runs on the stream's main CUDA
// stream; an async operation is forked onto one of a few side streams that start at the last ordered point,
// and the next ordered operation (or event, or Await) joins them back with CUDA events.  Copies that touch
// host memory go to the copy engines, device-to-device copies to this library's copy kernel, and neither
// switch costs a CPU round trip (the reference replays every compute<->DMA switch with a CPU wait, :826-844).
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <iterator>
#include <thread>

#include "internal.h"

using namespace lcu;

namespace lcu {

libreCudaStatus_t record(LibreCUstream stream, Command &&cmd) {
    stream->pending.push_back(std::move(cmd));
    LIBRECUDA_SUCCEED();
}

// Limit of a host wait in milliseconds, from LIBRECUDA_WAIT_TIMEOUT_MS (unset or 0: wait for ever, like the
// reference's signalWaitCpu, cmdqueue.cpp:346-352).  With a limit, a wait that runs out returns NOT_READY and
// the work stays submitted: the caller may wait again.
static uint64_t wait_limit_ms() {
    static const uint64_t limit = [] {
        const char *e = std::getenv("LIBRECUDA_WAIT_TIMEOUT_MS");
        const long long v = e ? std::atoll(e) : 0;
        return v > 0 ? (uint64_t)v : (uint64_t)0;
    }();
    return limit;
}

// A kernel of this library that gave up a bounded wait leaves its copy incomplete and raises the device's
// sticky error word; the stream itself finishes without a CUDA error.  Checked after every host wait, so a
// program written for the reference (which only ever looks at the status of Await) cannot take a partial
// copy for a finished one.  The word is reported once and cleared.
static libreCudaStatus_t check_device_error_word() {
    unsigned int w = 0;
    if (lcb_device_error_peek(&w) != 0 || w == 0) LIBRECUDA_SUCCEED();
    unsigned int cleared = 0;
    (void)lcb_device_error_word(&cleared);
    LIBRECUDA_DEBUG("device error word " << (w | cleared) << ": a kernel of this library gave up a bounded wait; its operation is incomplete");
    LIBRECUDA_FAIL(LIBRECUDA_ERROR_UNKNOWN);
}

// Host-side wait in the style chosen at context creation (reference cmdqueue.cpp:337-355).
template <typename QueryFn, typename BlockFn>
static libreCudaStatus_t host_wait(LibreCUcontext ctx, QueryFn query, BlockFn block) {
    const int flags = ctx ? ctx->flags : 0;
    const uint64_t limit = wait_limit_ms();
    if ((flags & CU_CTX_SCHED_BLOCKING_SYNC) && limit == 0) {
        LCU_CUDA(block());
        return check_device_error_word();
    }
    // blocking contexts with a limit poll and yield: a blocking CUDA wait cannot be given a deadline
    const bool yield = (flags & CU_CTX_SCHED_BLOCKING_SYNC) || (!(flags & CU_CTX_SCHED_SPIN) && (flags & CU_CTX_SCHED_YIELD));
    cudaError_t failure = cudaSuccess;
    const WaitOutcome out = poll_until(
        [&] {
            const cudaError_t q = query();
            if (q == cudaSuccess) return PollResult::Done;
            if (q == cudaErrorNotReady) return PollResult::Pending;
            failure = q;
            return PollResult::Failed;
        },
        steady_ms, limit, yield);
    if (out == WaitOutcome::Failed) LCU_CUDA(failure);
    if (out == WaitOutcome::TimedOut) {
        LIBRECUDA_DEBUG("host wait gave up after " << limit << " ms (LIBRECUDA_WAIT_TIMEOUT_MS)");
        LIBRECUDA_FAIL(LIBRECUDA_ERROR_NOT_READY);
    }
    return check_device_error_word();
}

libreCudaStatus_t host_wait_stream(LibreCUcontext ctx, cudaStream_t s) {
    return host_wait(ctx, [&] { return cudaStreamQuery(s); }, [&] { return cudaStreamSynchronize(s); });
}

libreCudaStatus_t host_wait_event(LibreCUcontext ctx, cudaEvent_t e) {
    return host_wait(ctx, [&] { return cudaEventQuery(e); }, [&] { return cudaEventSynchronize(e); });
}

libreCudaStatus_t join_sides(LibreCUstream st) {
    for (int i = 0; i < kSideLanes; ++i) {
        if (!st->side_dirty[i]) continue;
        LCU_CUDA(cudaEventRecord(st->side_done[i], st->side[i]));
        LCU_CUDA(cudaStreamWaitEvent(st->main, st->side_done[i], 0));
        st->side_dirty[i] = false;
    }
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t fork_side(LibreCUstream st, int i, cudaStream_t *lane) {
    if (st->side[i] == nullptr) {
        LCU_CUDA(cudaStreamCreateWithFlags(&st->side[i], cudaStreamNonBlocking));
        LCU_CUDA(cudaEventCreateWithFlags(&st->side_done[i], cudaEventDisableTiming));
    }
    LCU_CUDA(cudaEventRecord(st->fork, st->main));
    LCU_CUDA(cudaStreamWaitEvent(st->side[i], st->fork, 0));
    st->side_dirty[i] = true;
    *lane = st->side[i];
    LIBRECUDA_SUCCEED();
}

// Lane an operation runs on: the main stream after a join for ordered operations, a side stream forked
// from the main stream's current tail for async ones.
static libreCudaStatus_t pick_lane(LibreCUstream st, bool async, cudaStream_t *lane) {
    if (!async) {
        LIBRECUDA_ERR_PROPAGATE(join_sides(st));
        *lane = st->main;
        LIBRECUDA_SUCCEED();
    }
    const int i = st->next_side;
    st->next_side = (i + 1) % kSideLanes;
    return fork_side(st, i, lane);
}

static libreCudaStatus_t submit(LibreCUstream st, Command &c) {
    cudaStream_t lane = nullptr;
    switch (c.kind) {
        case Command::CopyKernel: {
            LIBRECUDA_ERR_PROPAGATE(pick_lane(st, c.async, &lane));
            // An ordered copy whose source no library kernel still in flight on the main lane writes may load
            // before the previous kernel has drained (its stores still wait).  Async copies run on side lanes
            // that start behind an event, where there is nothing to overlap with.
            int path = LCB_COPY_AUTO;
            if (!c.async) {
                if (!st->main_writes.may_be_written(c.src, c.bytes)) path |= LCB_COPY_SRC_STABLE;
                st->main_writes.add(c.dst, c.bytes);
            }
            LCU_LCB(lcb_copy_d2d_ex(c.dst, c.src, c.bytes, path, 0, lane));
            break;
        }
        case Command::CopyEngine:
            LIBRECUDA_ERR_PROPAGATE(pick_lane(st, c.async, &lane));
            // a copy-engine transfer starts after, and the next kernel after it starts behind, everything before it
            if (!c.async) st->main_writes.clear();
            if (c.bytes >= kStageMinBytes && c.copy_kind == cudaMemcpyHostToDevice && is_pageable_host(c.src)) {
                LIBRECUDA_ERR_PROPAGATE(staged_h2d(st, lane, c.dst, c.src, c.bytes));
            } else if (c.bytes >= kStageMinBytes && c.copy_kind == cudaMemcpyDeviceToHost && is_pageable_host(c.dst)) {
                LIBRECUDA_ERR_PROPAGATE(staged_d2h(st, lane, c.dst, c.src, c.bytes));
            } else {
                LCU_CUDA(cudaMemcpyAsync(c.dst, c.src, c.bytes, c.copy_kind, lane));
            }
            break;
        case Command::Memset:
            LIBRECUDA_ERR_PROPAGATE(pick_lane(st, c.async, &lane));
            if (!c.async) st->main_writes.add(c.dst, c.bytes);
            LCU_LCB(lcb_memset_ex(c.dst, c.value, c.elem, c.bytes / (size_t)c.elem, 0, 0, lane));
            break;
        case Command::AllToAllPush:
            LIBRECUDA_ERR_PROPAGATE(pick_lane(st, c.async, &lane));
            if (!c.async) st->main_writes.add_unknown();  // writes into every peer's buffer
            LCU_LCB(lcb_alltoall_push(c.peers.data(), c.src, c.bytes, (int)c.peers.size(), c.rank, lane));
            break;
        case Command::AllToAllPull:
            LIBRECUDA_ERR_PROPAGATE(pick_lane(st, c.async, &lane));
            if (!c.async) st->main_writes.add(c.dst, c.bytes * c.peers.size());
            LCU_LCB(lcb_alltoall_pull(c.peers.data(), c.dst, c.bytes, (int)c.peers.size(), c.rank, lane));
            break;
        case Command::AllToAllEngines: {
            // engine copies on the main lane, the local chunk as a kernel on a side lane beside them
            LIBRECUDA_ERR_PROPAGATE(pick_lane(st, false, &lane));
            st->main_writes.clear();  // copy-engine transfers serialise the lane
            cudaStream_t local = nullptr;
            LIBRECUDA_ERR_PROPAGATE(fork_side(st, 0, &local));
            LCU_LCB(lcb_alltoall_engines(c.peers.data(), c.src, c.bytes, (int)c.peers.size(), c.rank,
                                         c.peer_flags.empty() ? nullptr : c.peer_flags[(size_t)c.rank],
                                         c.peer_flags.empty() ? nullptr : c.peer_flags.data(), c.epoch, c.timeout_ms, lane, local));
            st->main_writes.add_unknown();
            break;
        }
        case Command::Launch: {
            LIBRECUDA_ERR_PROPAGATE(pick_lane(st, c.async, &lane));
            // what a user kernel writes is unknown, and a library kernel behind it may become resident as soon as the
            // user kernel's last block has exited: no loads ahead of the wait until the lane has fully serialised
            if (!c.async) st->main_writes.add_unknown();
            LibreCUFunction f = c.fn;
            std::vector<void *> argv(f->param_size.size());
            for (size_t i = 0; i < argv.size(); ++i) argv[i] = c.params.data() + f->param_offset[i];
            LCU_CU(driver()->LaunchKernel(f->fn, c.grid[0], c.grid[1], c.grid[2], c.block[0], c.block[1], c.block[2],
                                          c.smem, lane, argv.empty() ? nullptr : argv.data(), nullptr));
            break;
        }
        case Command::EventRecord: {
            LIBRECUDA_ERR_PROPAGATE(join_sides(st));
            LibreCUEvent e = c.event;
            if (e->ev != nullptr && e->device != st->ctx->device->ordinal) {
                (void)cudaEventDestroy(e->ev);
                e->ev = nullptr;
            }
            if (e->ev == nullptr) {
                LCU_CUDA(cudaEventCreate(&e->ev));
                e->device = st->ctx->device->ordinal;
            }
            {   // a fresh epoch in front of the event when the newest one is getting old (see LibreCUcontext_)
                LibreCUcontext ctx = st->ctx;
                const uint64_t now = steady_ms();
                if (now - ctx->epochs.back().host_ms >= kEpochRollMs) {
                    LibreCUcontext_::Epoch ep;
                    LCU_CUDA(cudaEventCreate(&ep.ev));
                    LCU_CUDA(cudaEventRecord(ep.ev, st->main));
                    ep.host_ms = now;
                    ctx->epochs.push_back(ep);
                    ctx->epoch_base_ns.push_back(0);
                }
                e->epoch_idx = ctx->epochs.size() - 1;
            }
            LCU_CUDA(cudaEventRecord(e->ev, st->main));
            e->state = LibreCUEvent_::Submitted;
            break;
        }
        case Command::WaitEvent:
            // later operations fork from / run on the main stream, so they all observe the wait
            LCU_CUDA(cudaStreamWaitEvent(st->main, c.event->ev, 0));
            break;
    }
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t commence(LibreCUstream st) {
    LIBRECUDA_ERR_PROPAGATE(bind(st->ctx));
    // a wait on an event whose record has not been submitted anywhere cannot be honoured: refuse the whole
    // batch before anything is submitted
    for (size_t i = 0; i < st->pending.size(); ++i) {
        const Command &c = st->pending[i];
        if (c.kind != Command::WaitEvent) continue;
        LibreCUEvent e = c.event;
        if (e->state == LibreCUEvent_::Submitted) continue;
        bool earlier_here = false;
        for (size_t j = 0; j < i; ++j)
            if (st->pending[j].kind == Command::EventRecord && st->pending[j].event == e) earlier_here = true;
        LIBRECUDA_VALIDATE(earlier_here, LIBRECUDA_ERROR_NOT_READY);
    }
    std::vector<Command> batch;
    batch.swap(st->pending);
    libreCudaStatus_t status = LIBRECUDA_SUCCESS;
    for (size_t i = 0; i < batch.size(); ++i) {
        status = submit(st, batch[i]);
        if (status != LIBRECUDA_SUCCESS) {
            // the failed operation is dropped; what was recorded after it stays recorded for a later Commence
            st->pending.insert(st->pending.begin(), std::make_move_iterator(batch.begin() + (long)i + 1),
                               std::make_move_iterator(batch.end()));
            break;
        }
    }
    LibreCUcontext cur = globals().current;
    if (cur != nullptr && cur != st->ctx) LIBRECUDA_ERR_PROPAGATE(bind(cur));
    return status;
}

}  // namespace lcu

// ---- streams ----------------------------------------------------------------------------------------------

libreCudaStatus_t libreCuStreamCreate(LibreCUstream *pStreamOut, uint32_t flags) {
    return lcu_guarded([&]() -> libreCudaStatus_t {
        (void)flags;
        LIBRECUDA_VALIDATE(pStreamOut != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        LCU_ENSURE_CTX();
        LibreCUcontext ctx = globals().current;
        LIBRECUDA_ERR_PROPAGATE(bind(ctx));
        auto st = std::make_unique<LibreCUstream_>();
        st->ctx = ctx;
        LCU_CUDA(cudaStreamCreateWithFlags(&st->main, cudaStreamNonBlocking));
        LCU_CUDA(cudaEventCreateWithFlags(&st->fork, cudaEventDisableTiming));
        // The side lanes of async operations are made here, not at their first use: creating a CUDA stream while
        // kernels are running can wait for them, which cost the first burst of async launches most of its overlap.
        for (int i = 0; i < kSideLanes; ++i) {
            LCU_CUDA(cudaStreamCreateWithFlags(&st->side[i], cudaStreamNonBlocking));
            LCU_CUDA(cudaEventCreateWithFlags(&st->side_done[i], cudaEventDisableTiming));
        }
        *pStreamOut = st.release();
        LIBRECUDA_SUCCEED();
    });
}

libreCudaStatus_t libreCuStreamDestroy(LibreCUstream stream) {
    LIBRECUDA_VALIDATE(stream != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    if (cudaSetDevice(stream->ctx->device->ordinal) == cudaSuccess) {
        for (int i = 0; i < kSideLanes; ++i) {
            if (stream->side[i]) {
                (void)cudaStreamSynchronize(stream->side[i]);
                (void)cudaStreamDestroy(stream->side[i]);
                (void)cudaEventDestroy(stream->side_done[i]);
            }
        }
        (void)cudaStreamSynchronize(stream->main);
        free_ring(stream);
        (void)cudaStreamDestroy(stream->main);
        (void)cudaEventDestroy(stream->fork);
    }
    (void)cudaGetLastError();
    LibreCUcontext cur = globals().current;
    delete stream;
    if (cur != nullptr) (void)cudaSetDevice(cur->device->ordinal);
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t libreCuStreamCommence(LibreCUstream stream) {
    return lcu_guarded([&]() -> libreCudaStatus_t {
        LIBRECUDA_VALIDATE(stream != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        return commence(stream);
    });
}

libreCudaStatus_t libreCuStreamAwait(LibreCUstream stream) {
    LIBRECUDA_VALIDATE(stream != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_ERR_PROPAGATE(bind(stream->ctx));
    LIBRECUDA_ERR_PROPAGATE(join_sides(stream));
    const libreCudaStatus_t waited = host_wait_stream(stream->ctx, stream->main);
    if (waited == LIBRECUDA_SUCCESS) stream->main_writes.clear();  // nothing is in flight any more
    LibreCUcontext cur = globals().current;
    if (cur != nullptr && cur != stream->ctx) LIBRECUDA_ERR_PROPAGATE(bind(cur));
    return waited;
}

libreCudaStatus_t libreCuStreamGetNativeHandle(void **pNativeStreamOut, LibreCUstream stream) {
    LIBRECUDA_VALIDATE(pNativeStreamOut != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(stream != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    *pNativeStreamOut = stream->main;
    LIBRECUDA_SUCCEED();
}

// ---- copies -----------------------------------------------------------------------------------------------

static libreCudaStatus_t record_copy(void *dst, const void *src, size_t n, LibreCUstream stream, bool async,
                                     PtrClass dc, PtrClass sc) {
    if (n == 0) LIBRECUDA_SUCCEED();
    Command c;
    c.async = async;
    c.dst = dst;
    c.src = src;
    c.bytes = n;
    if (dc == PtrClass::Device && sc == PtrClass::Device) {
        // the copy kernel runs on the stream's GPU: both buffers must be its own or a peer's it was given
        // access to (libreCuCtxEnablePeerAccess); refusing here is what keeps a bad pointer from faulting the GPU
        for (const void *p : {static_cast<const void *>(dst), src}) {
            const int owner = owner_device(p);
            LIBRECUDA_VALIDATE(owner < 0 || stream->ctx->peers.count(owner) != 0, LIBRECUDA_ERROR_INVALID_VALUE);
        }
        c.kind = Command::CopyKernel;  // reference: memcpyD2D, memcopy.cpp:77
        // Between two different GPUs the copy engines move 775-782 GB/s per direction, also with every link busy
        // both ways, where SM-issued stores reach 707-716 and loads 645 (NVLink write packets from the SMs carry
        // half the payload of the engines'); but every engine peer copy costs 7.7 us on top of its transfer
        // (measured: 4 GiB cut into 16 ... 2048 back-to-back copies), a kernel launch about 2.5.  The engines
        // win from about 44 MB up: a cross-device copy of 64 MiB and more goes to them (knob, in MiB; 0 = never).
        const int od = owner_device(dst), os = owner_device(src);
        const int engine_mib = (od >= 0 && os >= 0 && od != os) ? lcb_tune_get("peer_copy_engine") : 0;
        if (od >= 0 && os >= 0 && od != os && engine_mib > 0 && n >= ((size_t)engine_mib << 20)) {
            c.kind = Command::CopyEngine;
            c.copy_kind = cudaMemcpyDefault;
        }
    } else {
        c.kind = Command::CopyEngine;  // reference: gpuMemcpy, cmdqueue.cpp:732
        c.copy_kind = dc == PtrClass::Device ? cudaMemcpyHostToDevice
                      : sc == PtrClass::Device ? cudaMemcpyDeviceToHost
                                               : cudaMemcpyHostToHost;
    }
    return record(stream, std::move(c));
}

libreCudaStatus_t libreCuMemCpy(void *dst, void *src, size_t byteCount, LibreCUstream stream, bool async) {
    return lcu_guarded([&]() -> libreCudaStatus_t {
        LIBRECUDA_VALIDATE(dst != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        LIBRECUDA_VALIDATE(src != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        LIBRECUDA_VALIDATE(stream != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        LCU_ENSURE_CTX();
        return record_copy(dst, src, byteCount, stream, async, classify(dst), classify(src));
    });
}

static libreCudaStatus_t directional(void *dst, const void *src, size_t n, LibreCUstream stream, bool async,
                                     PtrClass want_dst, PtrClass want_src) {
    LIBRECUDA_VALIDATE(dst != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(src != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(stream != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LCU_ENSURE_CTX();
    const PtrClass dc = classify(dst), sc = classify(src);
    LIBRECUDA_VALIDATE(dc == want_dst, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(sc == want_src, LIBRECUDA_ERROR_INVALID_VALUE);
    return record_copy(dst, src, n, stream, async, dc, sc);
}

libreCudaStatus_t libreCuMemcpyHtoD(void *d, const void *s, size_t n, LibreCUstream st) {
    return directional(d, s, n, st, false, PtrClass::Device, PtrClass::Host);
}
libreCudaStatus_t libreCuMemcpyHtoDAsync(void *d, const void *s, size_t n, LibreCUstream st) {
    return directional(d, s, n, st, true, PtrClass::Device, PtrClass::Host);
}
libreCudaStatus_t libreCuMemcpyDtoH(void *d, const void *s, size_t n, LibreCUstream st) {
    return directional(d, s, n, st, false, PtrClass::Host, PtrClass::Device);
}
libreCudaStatus_t libreCuMemcpyDtoHAsync(void *d, const void *s, size_t n, LibreCUstream st) {
    return directional(d, s, n, st, true, PtrClass::Host, PtrClass::Device);
}
libreCudaStatus_t libreCuMemcpyDtoD(void *d, const void *s, size_t n, LibreCUstream st) {
    return directional(d, s, n, st, false, PtrClass::Device, PtrClass::Device);
}
libreCudaStatus_t libreCuMemcpyDtoDAsync(void *d, const void *s, size_t n, LibreCUstream st) {
    return directional(d, s, n, st, true, PtrClass::Device, PtrClass::Device);
}

libreCudaStatus_t libreCuMemcpyPeer(void *dstDevice, const void *srcDevice, size_t byteCount, LibreCUstream stream,
                                    bool async) {
    return directional(dstDevice, srcDevice, byteCount, stream, async, PtrClass::Device, PtrClass::Device);
}

// ---- memset -----------------------------------------------------------------------------------------------

static libreCudaStatus_t record_memset(void *dst, unsigned int value, int elem, size_t count, LibreCUstream stream,
                                       bool async) {
    LIBRECUDA_VALIDATE(dst != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(stream != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LCU_ENSURE_CTX();
    LIBRECUDA_VALIDATE((reinterpret_cast<uintptr_t>(dst) & (uintptr_t)(elem - 1)) == 0, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(classify(dst) == PtrClass::Device, LIBRECUDA_ERROR_INVALID_VALUE);
    {
        const int owner = owner_device(dst);  // same rule as for kernel copies
        LIBRECUDA_VALIDATE(owner < 0 || stream->ctx->peers.count(owner) != 0, LIBRECUDA_ERROR_INVALID_VALUE);
    }
    if (count == 0) LIBRECUDA_SUCCEED();
    Command c;
    c.kind = Command::Memset;
    c.async = async;
    c.dst = dst;
    c.value = value;
    c.elem = elem;
    c.bytes = count * (size_t)elem;
    return record(stream, std::move(c));
}

libreCudaStatus_t libreCuMemsetD8(void *d, unsigned char v, size_t n, LibreCUstream st) { return record_memset(d, v, 1, n, st, false); }
libreCudaStatus_t libreCuMemsetD8Async(void *d, unsigned char v, size_t n, LibreCUstream st) { return record_memset(d, v, 1, n, st, true); }
libreCudaStatus_t libreCuMemsetD16(void *d, unsigned short v, size_t n, LibreCUstream st) { return record_memset(d, v, 2, n, st, false); }
libreCudaStatus_t libreCuMemsetD16Async(void *d, unsigned short v, size_t n, LibreCUstream st) { return record_memset(d, v, 2, n, st, true); }
libreCudaStatus_t libreCuMemsetD32(void *d, unsigned int v, size_t n, LibreCUstream st) { return record_memset(d, v, 4, n, st, false); }
libreCudaStatus_t libreCuMemsetD32Async(void *d, unsigned int v, size_t n, LibreCUstream st) { return record_memset(d, v, 4, n, st, true); }

// ---- events -----------------------------------------------------------------------------------------------

libreCudaStatus_t libreCuEventCreate(LibreCUEvent *pEventOut, uint32_t flags) {
    return lcu_guarded([&]() -> libreCudaStatus_t {
        (void)flags;
        LIBRECUDA_VALIDATE(pEventOut != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        *pEventOut = new LibreCUEvent_();
        LIBRECUDA_SUCCEED();
    });
}

libreCudaStatus_t libreCuEventRecord(LibreCUEvent event, LibreCUstream stream) {
    return lcu_guarded([&]() -> libreCudaStatus_t {
        LIBRECUDA_VALIDATE(event != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        LIBRECUDA_VALIDATE(stream != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        event->stream = stream;
        event->ctx = stream->ctx;
        event->state = LibreCUEvent_::Pending;
        Command c;
        c.kind = Command::EventRecord;
        c.event = event;
        return record(stream, std::move(c));
    });
}

libreCudaStatus_t libreCuEventSynchronize(LibreCUEvent event) {
    LIBRECUDA_VALIDATE(event != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(event->state != LibreCUEvent_::Never, LIBRECUDA_ERROR_INVALID_VALUE);  // reference librecuda.cpp:1633
    // recorded but its stream never commenced: the reference would spin forever (cmdqueue.cpp:928-940)
    LIBRECUDA_VALIDATE(event->state == LibreCUEvent_::Submitted, LIBRECUDA_ERROR_NOT_READY);
    LIBRECUDA_ERR_PROPAGATE(bind(event->ctx));  // the error word consulted after the wait is the event's device's
    const libreCudaStatus_t waited = host_wait_event(event->ctx, event->ev);
    LibreCUcontext cur = globals().current;
    if (cur != nullptr && cur != event->ctx) LIBRECUDA_ERR_PROPAGATE(bind(cur));
    return waited;
}

libreCudaStatus_t libreCuEventQuery(LibreCUEvent event) {
    LIBRECUDA_VALIDATE(event != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(event->state != LibreCUEvent_::Never, LIBRECUDA_ERROR_INVALID_VALUE);
    if (event->state != LibreCUEvent_::Submitted) LIBRECUDA_FAIL(LIBRECUDA_ERROR_NOT_READY);
    cudaError_t q = cudaEventQuery(event->ev);
    if (q == cudaErrorNotReady) LIBRECUDA_FAIL(LIBRECUDA_ERROR_NOT_READY);
    LCU_CUDA(q);
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t libreCuEventElapsedTime(float *pMillisecondsOut, LibreCUEvent start, LibreCUEvent end) {
    LIBRECUDA_VALIDATE(pMillisecondsOut != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(start != nullptr && end != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(start->state != LibreCUEvent_::Never && end->state != LibreCUEvent_::Never, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(start->stream == end->stream, LIBRECUDA_ERROR_INVALID_VALUE);  // reference librecuda.cpp:1641-1643
    if (start->state != LibreCUEvent_::Submitted || end->state != LibreCUEvent_::Submitted) LIBRECUDA_FAIL(LIBRECUDA_ERROR_NOT_READY);
    cudaError_t e = cudaEventElapsedTime(pMillisecondsOut, start->ev, end->ev);
    if (e == cudaErrorNotReady) {
        (void)cudaGetLastError();
        LIBRECUDA_FAIL(LIBRECUDA_ERROR_NOT_READY);
    }
    LCU_CUDA(e);
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t libreCuEventGetTimestamp(uint64_t *pNanosecondsOut, LibreCUEvent event) {
    LIBRECUDA_VALIDATE(pNanosecondsOut != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(event != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(event->state != LibreCUEvent_::Never, LIBRECUDA_ERROR_INVALID_VALUE);
    if (event->state != LibreCUEvent_::Submitted) LIBRECUDA_FAIL(LIBRECUDA_ERROR_NOT_READY);
    LibreCUcontext ctx = event->ctx;
    // offsets of the epochs up to the event's own, as far as the GPU has reached them
    (void)resolve_epochs(ctx->epoch_base_ns, ctx->epochs_resolved, event->epoch_idx, [&](size_t a, size_t b, float *ms) {
        const cudaError_t e = cudaEventElapsedTime(ms, ctx->epochs[a].ev, ctx->epochs[b].ev);
        if (e != cudaSuccess) (void)cudaGetLastError();
        return e == cudaSuccess;
    });
    // measure from the newest resolved epoch at or before the event's (an epoch recorded on another stream may
    // not have been reached yet although the event has: fall back to an older one)
    size_t k = event->epoch_idx < ctx->epochs_resolved ? event->epoch_idx : ctx->epochs_resolved - 1;
    for (;; --k) {
        float ms = 0.f;
        const cudaError_t e = cudaEventElapsedTime(&ms, ctx->epochs[k].ev, event->ev);
        if (e == cudaSuccess) {
            const int64_t t = (int64_t)ctx->epoch_base_ns[k] + (int64_t)((double)ms * 1.0e6);
            *pNanosecondsOut = t > 0 ? (uint64_t)t : 0;
            LIBRECUDA_SUCCEED();
        }
        (void)cudaGetLastError();
        if (e != cudaErrorNotReady) LCU_CUDA(e);
        if (k == 0) LIBRECUDA_FAIL(LIBRECUDA_ERROR_NOT_READY);
    }
}

libreCudaStatus_t libreCuEventDestroy(LibreCUEvent event) {
    LIBRECUDA_VALIDATE(event != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    if (event->ev) {
        (void)cudaEventDestroy(event->ev);
        (void)cudaGetLastError();
    }
    delete event;
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t libreCuStreamWaitEvent(LibreCUstream stream, LibreCUEvent event) {
    return lcu_guarded([&]() -> libreCudaStatus_t {
        LIBRECUDA_VALIDATE(stream != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        LIBRECUDA_VALIDATE(event != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        LIBRECUDA_VALIDATE(event->state != LibreCUEvent_::Never, LIBRECUDA_ERROR_INVALID_VALUE);
        Command c;
        c.kind = Command::WaitEvent;
        c.event = event;
        return record(stream, std::move(c));
    });
}
