// Multi-GPU entry points: peer access, the shard partitioner, partitioned / all-to-all / broadcast data
// movement over NVLink, and inter-process buffer sharing.  The reference is single-GPU (one process-global
// context, driverapi/src/librecuda.cpp:61), so everything here is additive.
//
// Own-kernel paths read straight from (or write straight into) peer memory with the library's copy kernels
// (plain vector accesses or non-multicast bulk copies).  Measured on NVLink 5: when only one direction of a
// link carries data (scatter from a root) remote LOADS are faster (786 vs 716 GB/s per GPU); when both
// directions are busy (all-to-all, ring shift) remote STORES are (704 vs 665), and the copy engines beat both
// (775) at the price of 7.7 us per copy, so the collectives also have a copy-engine form.  NCCL is used only
// for the broadcast and all-to-all collectives and is loaded lazily with dlopen so that programs that never
// call them do not need it.
#include <dlfcn.h>
#include <nccl.h>

#include <cmath>
#include <cstring>

#include "internal.h"
#include "multicast.h"

using namespace lcu;

libreCudaStatus_t libreCuDeviceCanAccessPeer(int *pCanAccess, LibreCUdevice device, LibreCUdevice peerDevice) {
    LIBRECUDA_VALIDATE(pCanAccess != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(device != nullptr && peerDevice != nullptr, LIBRECUDA_ERROR_INVALID_DEVICE);
    if (device == peerDevice) {
        *pCanAccess = 1;
        LIBRECUDA_SUCCEED();
    }
    LCU_CUDA(cudaDeviceCanAccessPeer(pCanAccess, device->ordinal, peerDevice->ordinal));
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t libreCuCtxEnablePeerAccess(LibreCUcontext peerCtx, unsigned int flags) {
    LIBRECUDA_VALIDATE(peerCtx != nullptr, LIBRECUDA_ERROR_INVALID_CONTEXT);
    LIBRECUDA_VALIDATE(flags == 0, LIBRECUDA_ERROR_INVALID_VALUE);
    LCU_ENSURE_CTX();
    LibreCUcontext cur = globals().current;
    const int peer = peerCtx->device->ordinal;
    if (cur->peers.count(peer)) LIBRECUDA_SUCCEED();
    LIBRECUDA_ERR_PROPAGATE(bind(cur));
    cudaError_t err = cudaDeviceEnablePeerAccess(peer, 0);
    if (err == cudaErrorPeerAccessAlreadyEnabled) {
        (void)cudaGetLastError();
        err = cudaSuccess;
    }
    LCU_CUDA(err);
    cur->peers.insert(peer);
    LIBRECUDA_SUCCEED();
}

// ---- partitioner ------------------------------------------------------------------------------------------

libreCudaStatus_t libreCuPartitionPlan(size_t totalBytes, int parts, size_t alignBytes, size_t *offsetsOut) {
    LIBRECUDA_VALIDATE(offsetsOut != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(parts >= 1, LIBRECUDA_ERROR_INVALID_VALUE);
    if (alignBytes == 0) alignBytes = (size_t)2 << 20;
    LIBRECUDA_VALIDATE((alignBytes & (alignBytes - 1)) == 0, LIBRECUDA_ERROR_INVALID_VALUE);
    // equal shares rounded up to the alignment; trailing shards may be short or empty
    const size_t share = (totalBytes + (size_t)parts - 1) / (size_t)parts;
    const size_t per = (share + alignBytes - 1) / alignBytes * alignBytes;
    for (int g = 0; g <= parts; ++g) {
        const size_t o = per * (size_t)g;
        offsetsOut[g] = (g == parts || o > totalBytes) ? totalBytes : o;
    }
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t libreCuMemcpyPartitioned(void *const *dsts, const void *src, size_t totalBytes, int parts,
                                           size_t alignBytes, const LibreCUstream *streams) {
    return lcu_guarded([&]() -> libreCudaStatus_t {
        LIBRECUDA_VALIDATE(dsts != nullptr && src != nullptr && streams != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        LIBRECUDA_VALIDATE(parts >= 1 && parts <= 64, LIBRECUDA_ERROR_INVALID_VALUE);
        size_t off[65];
        LIBRECUDA_ERR_PROPAGATE(libreCuPartitionPlan(totalBytes, parts, alignBytes, off));
        for (int g = 0; g < parts; ++g) {
            LIBRECUDA_VALIDATE(dsts[g] != nullptr && streams[g] != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        }
        for (int g = 0; g < parts; ++g) {
            if (off[g + 1] == off[g]) continue;
            LIBRECUDA_ERR_PROPAGATE(libreCuMemcpyPeer(dsts[g], static_cast<const uint8_t *>(src) + off[g], off[g + 1] - off[g],
                                                      streams[g], false));
        }
        LIBRECUDA_SUCCEED();
    });
}

// ---- all-to-all ---------------------------------------------------------------------------------------------

static libreCudaStatus_t record_alltoall(bool pull, void *const *peerBufs, void *mine, size_t chunkBytes, int nRanks,
                                         int rank, LibreCUstream stream) {
    LIBRECUDA_VALIDATE(peerBufs != nullptr && mine != nullptr && stream != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(nRanks >= 1 && nRanks <= 16 && rank >= 0 && rank < nRanks, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE((chunkBytes & 15) == 0, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE((reinterpret_cast<uintptr_t>(mine) & 15) == 0, LIBRECUDA_ERROR_INVALID_VALUE);
    for (int j = 0; j < nRanks; ++j) {
        LIBRECUDA_VALIDATE(peerBufs[j] != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        LIBRECUDA_VALIDATE((reinterpret_cast<uintptr_t>(peerBufs[j]) & 15) == 0, LIBRECUDA_ERROR_INVALID_VALUE);
    }
    {   // every buffer must be reachable from the GPU that runs the kernel
        const int own = owner_device(mine);
        LIBRECUDA_VALIDATE(own < 0 || stream->ctx->peers.count(own) != 0, LIBRECUDA_ERROR_INVALID_VALUE);
        for (int j = 0; j < nRanks; ++j) {
            const int owner = owner_device(peerBufs[j]);
            LIBRECUDA_VALIDATE(owner < 0 || stream->ctx->peers.count(owner) != 0, LIBRECUDA_ERROR_INVALID_VALUE);
        }
    }
    if (chunkBytes == 0) LIBRECUDA_SUCCEED();
    Command c;
    c.kind = pull ? Command::AllToAllPull : Command::AllToAllPush;
    c.src = pull ? nullptr : mine;
    c.dst = pull ? mine : nullptr;
    c.bytes = chunkBytes;
    c.rank = rank;
    c.peers.assign(peerBufs, peerBufs + nRanks);
    return record(stream, std::move(c));
}

libreCudaStatus_t libreCuAllToAllPush(void *const *peerRecvBufs, const void *sendBuf, size_t chunkBytes, int nRanks,
                                      int rank, LibreCUstream stream) {
    return record_alltoall(false, peerRecvBufs, const_cast<void *>(sendBuf), chunkBytes, nRanks, rank, stream);
}

libreCudaStatus_t libreCuAllToAllPull(void *const *peerSendBufs, void *recvBuf, size_t chunkBytes, int nRanks, int rank,
                                      LibreCUstream stream) {
    return record_alltoall(true, peerSendBufs, recvBuf, chunkBytes, nRanks, rank, stream);
}

libreCudaStatus_t libreCuAllToAllEngines(void *const *peerRecvBufs, const void *sendBuf, size_t chunkBytes, int nRanks, int rank,
                                         void *const *peerFlags, unsigned int epoch, unsigned int timeoutMs, LibreCUstream stream) {
    return lcu_guarded([&]() -> libreCudaStatus_t {
        LIBRECUDA_VALIDATE(peerRecvBufs != nullptr && sendBuf != nullptr && stream != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        LIBRECUDA_VALIDATE(nRanks >= 1 && nRanks <= 16 && rank >= 0 && rank < nRanks, LIBRECUDA_ERROR_INVALID_VALUE);
        LIBRECUDA_VALIDATE(timeoutMs >= 1 && timeoutMs <= 10000, LIBRECUDA_ERROR_INVALID_VALUE);
        if (nRanks > 2) {
            LIBRECUDA_VALIDATE(peerFlags != nullptr && epoch >= 1, LIBRECUDA_ERROR_INVALID_VALUE);
            for (int j = 0; j < nRanks; ++j) {
                LIBRECUDA_VALIDATE(peerFlags[j] != nullptr && (reinterpret_cast<uintptr_t>(peerFlags[j]) & 3) == 0, LIBRECUDA_ERROR_INVALID_VALUE);
                const int owner = owner_device(peerFlags[j]);
                LIBRECUDA_VALIDATE(owner < 0 || stream->ctx->peers.count(owner) != 0, LIBRECUDA_ERROR_INVALID_VALUE);
            }
        }
        for (int j = 0; j < nRanks; ++j) {
            LIBRECUDA_VALIDATE(peerRecvBufs[j] != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
            const int owner = owner_device(peerRecvBufs[j]);
            LIBRECUDA_VALIDATE(owner < 0 || stream->ctx->peers.count(owner) != 0, LIBRECUDA_ERROR_INVALID_VALUE);
        }
        if (chunkBytes == 0) LIBRECUDA_SUCCEED();
        Command c;
        c.kind = Command::AllToAllEngines;
        c.src = sendBuf;
        c.bytes = chunkBytes;
        c.rank = rank;
        c.peers.assign(peerRecvBufs, peerRecvBufs + nRanks);
        if (nRanks > 2) c.peer_flags.assign(peerFlags, peerFlags + nRanks);
        c.epoch = epoch;
        c.timeout_ms = timeoutMs;
        return record(stream, std::move(c));
    });
}

// ---- NCCL, loaded on first use ------------------------------------------------------------------------------
namespace {

struct Nccl {
    void *lib = nullptr;
    ncclResult_t (*CommInitAll)(ncclComm_t *, int, const int *) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    ncclResult_t (*Send)(const void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Broadcast)(const void *, void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    std::vector<int> devs;           // devices of the cached communicator group
    std::vector<ncclComm_t> comms;
};

Nccl *nccl() {
    static Nccl n;
    static int state = 0;
    if (state == 0) {
        state = -1;
        n.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
        if (n.lib == nullptr) {
            LIBRECUDA_DEBUG("NCCL unavailable: " << dlerror());
            return nullptr;
        }
        bool ok = true;
        auto sym = [&](const char *name, void **out) {
            *out = dlsym(n.lib, name);
            if (*out == nullptr) ok = false;
        };
        sym("ncclCommInitAll", reinterpret_cast<void **>(&n.CommInitAll));
        sym("ncclCommDestroy", reinterpret_cast<void **>(&n.CommDestroy));
        sym("ncclGroupStart", reinterpret_cast<void **>(&n.GroupStart));
        sym("ncclGroupEnd", reinterpret_cast<void **>(&n.GroupEnd));
        sym("ncclSend", reinterpret_cast<void **>(&n.Send));
        sym("ncclRecv", reinterpret_cast<void **>(&n.Recv));
        sym("ncclBroadcast", reinterpret_cast<void **>(&n.Broadcast));
        sym("ncclGetErrorString", reinterpret_cast<void **>(&n.GetErrorString));
        if (ok) state = 1;
    }
    return state == 1 ? &n : nullptr;
}

#define LCU_NCCL(n, expr)                                                                                    \
    do {                                                                                                     \
        ncclResult_t lcu_nr_ = (expr);                                                                       \
        if (lcu_nr_ != ncclSuccess) {                                                                        \
            LIBRECUDA_DEBUG(__FILE__ ":" LIBRECUDA_STR_(__LINE__) ": " #expr " -> " << (n)->GetErrorString(lcu_nr_)); \
            return LIBRECUDA_ERROR_UNKNOWN;                                                                  \
        }                                                                                                    \
    } while (0)

libreCudaStatus_t nccl_group_for(Nccl *n, const std::vector<int> &devs) {
    if (n->devs == devs) LIBRECUDA_SUCCEED();
    for (ncclComm_t c : n->comms) n->CommDestroy(c);
    n->comms.assign(devs.size(), nullptr);
    n->devs.clear();
    LCU_NCCL(n, n->CommInitAll(n->comms.data(), (int)devs.size(), devs.data()));
    n->devs = devs;
    LIBRECUDA_SUCCEED();
}

// every buffer of a collective must be reachable from every participating GPU's context
libreCudaStatus_t check_reachable(int nDev, const LibreCUstream *streams, void *const *bufs) {
    for (int r = 0; r < nDev; ++r) {
        for (int j = 0; j < nDev; ++j) {
            const int owner = owner_device(bufs[j]);
            LIBRECUDA_VALIDATE(owner < 0 || streams[r]->ctx->peers.count(owner) != 0, LIBRECUDA_ERROR_INVALID_VALUE);
        }
    }
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t check_group(int nDev, const LibreCUstream *streams, std::vector<int> *devs) {
    LIBRECUDA_VALIDATE(streams != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(nDev >= 1 && nDev <= 16, LIBRECUDA_ERROR_INVALID_VALUE);
    for (int r = 0; r < nDev; ++r) {
        LIBRECUDA_VALIDATE(streams[r] != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        const int d = streams[r]->ctx->device->ordinal;
        for (int q : *devs) LIBRECUDA_VALIDATE(q != d, LIBRECUDA_ERROR_INVALID_VALUE);  // one stream per device
        devs->push_back(d);
    }
    LIBRECUDA_SUCCEED();
}

// Every stream waits for everything submitted so far on all the others -- async operations on their side lanes
// included -- so a collective starts after all earlier work of the group and an operation recorded later on
// any of the streams sees the complete result.
libreCudaStatus_t cross_join(int nDev, const LibreCUstream *streams) {
    std::vector<cudaEvent_t> done(nDev);
    for (int r = 0; r < nDev; ++r) {
        LIBRECUDA_ERR_PROPAGATE(bind(streams[r]->ctx));
        LIBRECUDA_ERR_PROPAGATE(join_sides(streams[r]));
        streams[r]->main_writes.add_unknown();  // the collectives' kernels write buffers this record does not follow
        LCU_CUDA(cudaEventCreateWithFlags(&done[r], cudaEventDisableTiming));
        LCU_CUDA(cudaEventRecord(done[r], streams[r]->main));
    }
    for (int r = 0; r < nDev; ++r) {
        LIBRECUDA_ERR_PROPAGATE(bind(streams[r]->ctx));
        for (int q = 0; q < nDev; ++q)
            if (q != r) LCU_CUDA(cudaStreamWaitEvent(streams[r]->main, done[q], 0));
    }
    for (int r = 0; r < nDev; ++r) (void)cudaEventDestroy(done[r]);  // released once the waits have consumed it
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t rebind_current() {
    LibreCUcontext cur = globals().current;
    if (cur != nullptr) return bind(cur);
    LIBRECUDA_SUCCEED();
}

}  // namespace

// Collectives over several streams of this process submit what those streams have recorded so far and are
// then enqueued at once (eager submission is within the Commence contract); they are complete after
// libreCuStreamAwait on the participating streams.
libreCudaStatus_t libreCuAllToAll(void *const *recvBufs, void *const *sendBufs, size_t chunkBytes, int nDev,
                                  const LibreCUstream *streams, int useNccl) {
    return lcu_guarded([&]() -> libreCudaStatus_t {
        LIBRECUDA_VALIDATE(recvBufs != nullptr && sendBufs != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        std::vector<int> devs;
        LIBRECUDA_ERR_PROPAGATE(check_group(nDev, streams, &devs));
        for (int r = 0; r < nDev; ++r) LIBRECUDA_VALIDATE(recvBufs[r] != nullptr && sendBufs[r] != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        LIBRECUDA_VALIDATE(useNccl >= 0 && useNccl <= 2, LIBRECUDA_ERROR_INVALID_VALUE);
        if (useNccl != 1) {
            LIBRECUDA_ERR_PROPAGATE(check_reachable(nDev, streams, recvBufs));
            LIBRECUDA_ERR_PROPAGATE(check_reachable(nDev, streams, sendBufs));
        }
        for (int r = 0; r < nDev; ++r) LIBRECUDA_ERR_PROPAGATE(commence(streams[r]));
        if (chunkBytes == 0) LIBRECUDA_SUCCEED();
        if (useNccl == 2) {
            // copy engines: rank r sends chunk (r+s) mod n to rank (r+s) mod n at step s, so that at every step
            // each GPU receives from exactly one sender; its own chunk goes through the local copy kernel.
            // Two engine copies that land on one GPU at the same time, or leave one GPU at the same time, fall to
            // about half the rate each AND idle another port meanwhile (measured: 500 GB/s per GPU instead of
            // 700-750 with 2-3 concurrent copies per GPU), so the schedule must stay in lock-step: the receiver of
            // rank r's step s was served by rank r+1 at step s-1, and rank r's copy waits for that one (one event
            // per copy).  Nothing then depends on the ranks running at the same speed.
            LIBRECUDA_ERR_PROPAGATE(cross_join(nDev, streams));
            std::vector<cudaEvent_t> landed((size_t)nDev, nullptr), landed_prev((size_t)nDev, nullptr);
            for (int r = 0; r < nDev; ++r) {
                // the local chunk runs as a kernel on a side lane, beside the engine copies of the main lane
                LibreCUstream sr = streams[r];
                LIBRECUDA_ERR_PROPAGATE(bind(sr->ctx));
                cudaStream_t lane = nullptr;
                LIBRECUDA_ERR_PROPAGATE(fork_side(sr, 0, &lane));
                LCU_LCB(lcb_copy_d2d(static_cast<uint8_t *>(recvBufs[r]) + (size_t)r * chunkBytes,
                                     static_cast<const uint8_t *>(sendBufs[r]) + (size_t)r * chunkBytes, chunkBytes, lane));
            }
            for (int step = 1; step < nDev; ++step) {
                landed_prev.swap(landed);
                for (int r = 0; r < nDev; ++r) {
                    const int j = (r + step) % nDev;
                    LIBRECUDA_ERR_PROPAGATE(bind(streams[r]->ctx));
                    uint8_t *d = static_cast<uint8_t *>(recvBufs[j]) + (size_t)r * chunkBytes;
                    const uint8_t *s = static_cast<const uint8_t *>(sendBufs[r]) + (size_t)j * chunkBytes;
                    if (step > 1 && nDev > 2) LCU_CUDA(cudaStreamWaitEvent(streams[r]->main, landed_prev[(size_t)((r + 1) % nDev)], 0));
                    LCU_CUDA(cudaMemcpyAsync(d, s, chunkBytes, cudaMemcpyDefault, streams[r]->main));
                    if (step + 1 < nDev && nDev > 2) {
                        LCU_CUDA(cudaEventCreateWithFlags(&landed[(size_t)r], cudaEventDisableTiming));
                        LCU_CUDA(cudaEventRecord(landed[(size_t)r], streams[r]->main));
                    }
                }
                for (cudaEvent_t e : landed_prev)
                    if (e != nullptr) (void)cudaEventDestroy(e);  // released once the waits have consumed it
                std::fill(landed_prev.begin(), landed_prev.end(), nullptr);
            }
            for (cudaEvent_t e : landed)
                if (e != nullptr) (void)cudaEventDestroy(e);
            LIBRECUDA_ERR_PROPAGATE(cross_join(nDev, streams));  // takes the side lanes in first
        } else if (useNccl == 1) {
            Nccl *n = nccl();
            LIBRECUDA_VALIDATE(n != nullptr, LIBRECUDA_ERROR_NOT_FOUND);
            LIBRECUDA_ERR_PROPAGATE(nccl_group_for(n, devs));
            for (int r = 0; r < nDev; ++r) {  // NCCL runs on the main lanes: they first absorb async work
                LIBRECUDA_ERR_PROPAGATE(bind(streams[r]->ctx));
                LIBRECUDA_ERR_PROPAGATE(join_sides(streams[r]));
            }
            LCU_NCCL(n, n->GroupStart());
            for (int r = 0; r < nDev; ++r) {
                const uint8_t *s = static_cast<const uint8_t *>(sendBufs[r]);
                uint8_t *d = static_cast<uint8_t *>(recvBufs[r]);
                for (int j = 0; j < nDev; ++j) {
                    LCU_NCCL(n, n->Send(s + (size_t)j * chunkBytes, chunkBytes, ncclUint8, j, n->comms[r], streams[r]->main));
                    LCU_NCCL(n, n->Recv(d + (size_t)j * chunkBytes, chunkBytes, ncclUint8, j, n->comms[r], streams[r]->main));
                }
            }
            LCU_NCCL(n, n->GroupEnd());
        } else {
            LIBRECUDA_VALIDATE((chunkBytes & 15) == 0, LIBRECUDA_ERROR_INVALID_VALUE);
            // rank r must not overwrite a receive slot its peer may still be using: start after everything
            // submitted so far on every stream.  Stores, not loads: with every link busy in both directions remote
            // stores are the faster form (704 vs 665 GB/s per GPU measured).
            LIBRECUDA_ERR_PROPAGATE(cross_join(nDev, streams));
            for (int r = 0; r < nDev; ++r) {
                LIBRECUDA_ERR_PROPAGATE(bind(streams[r]->ctx));
                LCU_LCB(lcb_alltoall_push(recvBufs, sendBufs[r], chunkBytes, nDev, r, streams[r]->main));
            }
            LIBRECUDA_ERR_PROPAGATE(cross_join(nDev, streams));
        }
        return rebind_current();
    });
}

namespace {

// Copy-engine chain over bytes [lo, hi) of the buffers: root -> d1 -> d2 -> ... in device order, piece by piece,
// on lanes[k] of device k.  The lane of chain member h pushes piece p to member h+1 as soon as member h-1 has
// delivered it (one event per piece and hop), so every GPU receives and sends at the engines' rate at once.
// Time = bytes / rate + pieces * c + (members - 2) * piece / rate, where c, the cost of one dependent peer copy,
// measured 7-12 us (4 GPUs, 4 GiB: 571 / 623 / 671 / 686 GB/s with 16 / 32 / 64 / 128 MiB pieces; alternating
// the pieces over two lanes per member changed nothing, so the cost sits in the engine, not in the lane).  The
// piece that minimises it is sqrt(bytes * c * rate / (members - 2)), c * rate = 7.75 MB.
libreCudaStatus_t bcast_chain(void *const *bufs, int root, size_t lo, size_t hi, int nDev, const LibreCUstream *streams,
                              const std::vector<cudaStream_t> &lanes) {
    if (hi <= lo) LIBRECUDA_SUCCEED();
    const size_t bytes = hi - lo;
    std::vector<int> chain;
    for (int k = 0; k < nDev; ++k) chain.push_back((root + k) % nDev);
    size_t piece = bytes;
    if (nDev > 2) {
        const int piece_mib = lcb_tune_get("bcast_engine_piece_mib");
        if (piece_mib > 0) {
            piece = (size_t)piece_mib << 20;
        } else {
            const double best = std::sqrt((double)bytes * 7.75e6 / (double)(nDev - 2));
            piece = ((size_t)(best / 1048576.0) + 1) << 20;
        }
    }
    std::vector<cudaEvent_t> arrived(nDev, nullptr);  // arrived[h]: the current piece has reached member h
    for (size_t p = lo; p < hi; p += piece) {
        const size_t n = hi - p < piece ? hi - p : piece;
        for (int h = 0; h + 1 < nDev; ++h) {
            const int dev = chain[h];
            LIBRECUDA_ERR_PROPAGATE(bind(streams[dev]->ctx));
            if (h > 0) {
                LCU_CUDA(cudaStreamWaitEvent(lanes[dev], arrived[h], 0));
                (void)cudaEventDestroy(arrived[h]);  // released once the wait has consumed it
                arrived[h] = nullptr;
            }
            LCU_CUDA(cudaMemcpyAsync(static_cast<uint8_t *>(bufs[chain[h + 1]]) + p,
                                     static_cast<const uint8_t *>(bufs[dev]) + p, n, cudaMemcpyDefault, lanes[dev]));
            if (h + 2 < nDev) {
                LCU_CUDA(cudaEventCreateWithFlags(&arrived[h + 1], cudaEventDisableTiming));
                LCU_CUDA(cudaEventRecord(arrived[h + 1], lanes[dev]));
            }
        }
    }
    LIBRECUDA_SUCCEED();
}

// Multicast through NVSwitch over bytes [lo, hi) (lo a multiple of 16; the caller has checked that the root
// buffer is 16-byte aligned).  The root's kernel reads its buffer once and writes it with multimem stores to a
// multicast address: every byte leaves the root's port once and the switch puts a copy into a staging slab on
// every GPU of the group; each GPU then moves the piece from its own slab into the caller's buffer with a local
// copy (HBM speed, a small fraction of the link time).  Nobody forwards anything, so the rate does not fall
// with the number of GPUs: 550 / 543 GB/s at 2 / 4 GPUs, whatever the kernel's shape (16 ... 1184 CTAs, 1-8
// vectors per thread, weak or relaxed stores) -- the fabric's rate for multicast writes from one GPU, below the
// 690-780 GB/s of the copy-engine chain there, which is why this form is not the default recommendation.  The
// slabs are a ring of `slots` pieces; the root reuses a slot once every GPU has copied the piece out of it (one
// event per GPU and slot), and a GPU starts its local copy when the root's kernel for that piece has finished.
libreCudaStatus_t bcast_multicast(void *const *bufs, int root, size_t lo, size_t hi, int nDev, const LibreCUstream *streams,
                                  const std::vector<cudaStream_t> &lanes, const McWindow *win, size_t piece, int slots) {
    if (hi <= lo) LIBRECUDA_SUCCEED();
    const uint8_t *src = static_cast<const uint8_t *>(bufs[root]);
    uint8_t *mc = static_cast<uint8_t *>(win->mc);
    std::vector<cudaEvent_t> filled((size_t)slots, nullptr);
    std::vector<cudaEvent_t> consumed((size_t)slots * (size_t)nDev, nullptr);
    std::vector<cudaEvent_t> retired;
    const size_t body_end = lo + ((hi - lo) & ~(size_t)15);  // multimem stores move whole 16-byte vectors
    const int ctas = lcb_tune_get("bcast_mc_ctas");
    size_t idx = 0;
    for (size_t p = lo; p < body_end; p += piece, ++idx) {
        const size_t n = body_end - p < piece ? body_end - p : piece;
        const size_t slot = idx % (size_t)slots;
        LIBRECUDA_ERR_PROPAGATE(bind(streams[root]->ctx));
        for (int g = 0; g < nDev; ++g) {  // the slot is free again once every GPU has emptied it
            cudaEvent_t &c = consumed[slot * (size_t)nDev + (size_t)g];
            if (c == nullptr) continue;
            LCU_CUDA(cudaStreamWaitEvent(lanes[root], c, 0));
            retired.push_back(c);
            c = nullptr;
        }
        LCU_LCB(lcb_multicast_store(mc + slot * piece, src + p, n, ctas, lanes[root]));
        if (filled[slot] != nullptr) retired.push_back(filled[slot]);
        LCU_CUDA(cudaEventCreateWithFlags(&filled[slot], cudaEventDisableTiming));
        LCU_CUDA(cudaEventRecord(filled[slot], lanes[root]));
        for (int g = 0; g < nDev; ++g) {
            if (g == root) continue;
            LIBRECUDA_ERR_PROPAGATE(bind(streams[g]->ctx));
            LCU_CUDA(cudaStreamWaitEvent(lanes[g], filled[slot], 0));
            LCU_LCB(lcb_copy_d2d(static_cast<uint8_t *>(bufs[g]) + p, static_cast<const uint8_t *>(win->local[g]) + slot * piece, n,
                                 lanes[g]));
            cudaEvent_t &c = consumed[slot * (size_t)nDev + (size_t)g];
            LCU_CUDA(cudaEventCreateWithFlags(&c, cudaEventDisableTiming));
            LCU_CUDA(cudaEventRecord(c, lanes[g]));
        }
    }
    if (body_end < hi) {  // the last few bytes: plain stores from the root into every buffer
        LIBRECUDA_ERR_PROPAGATE(bind(streams[root]->ctx));
        for (int g = 0; g < nDev; ++g)
            if (g != root) LCU_LCB(lcb_copy_d2d(static_cast<uint8_t *>(bufs[g]) + body_end, src + body_end, hi - body_end, lanes[root]));
    }
    for (cudaEvent_t e : filled)
        if (e != nullptr) (void)cudaEventDestroy(e);
    for (cudaEvent_t e : consumed)
        if (e != nullptr) (void)cudaEventDestroy(e);
    for (cudaEvent_t e : retired) (void)cudaEventDestroy(e);
    LIBRECUDA_SUCCEED();
}

}  // namespace

namespace {
int g_last_broadcast_form = -1;  // the form the most recent libreCuBroadcast really ran (after any fall-back)

// Per-device flag words of the ring broadcast (one per chunk), allocated on first use, grown on demand, kept
// until the process exits (128 KiB per GPU for a 4 GiB broadcast in 128 KiB chunks).  They start at zero and
// every call writes its own epoch, so they are never cleared.
struct RingFlags {
    unsigned int *ptr = nullptr;
    size_t words = 0;
};
RingFlags g_ring_flags[64];
unsigned int g_ring_epoch = 0;

libreCudaStatus_t ring_flags_for(int device, size_t words, unsigned int **out) {
    LIBRECUDA_VALIDATE(device >= 0 && device < 64, LIBRECUDA_ERROR_INVALID_DEVICE);
    RingFlags &f = g_ring_flags[device];
    if (f.words < words) {
        LCU_CUDA(cudaSetDevice(device));
        if (f.ptr != nullptr) {
            LCU_CUDA(cudaDeviceSynchronize());
            LCU_CUDA(cudaFree(f.ptr));
            f.ptr = nullptr;
            f.words = 0;
        }
        const size_t want = words < 65536 ? 65536 : words * 2;
        LCU_CUDA(cudaMalloc(reinterpret_cast<void **>(&f.ptr), want * sizeof(unsigned int)));
        LCU_CUDA(cudaMemset(f.ptr, 0, want * sizeof(unsigned int)));
        LCU_CUDA(cudaDeviceSynchronize());
        f.words = want;
        // a fresh array is all zero: earlier epochs must not look "already delivered", and they do not, because
        // every call uses a larger epoch than any before it
    }
    *out = f.ptr;
    LIBRECUDA_SUCCEED();
}
}

libreCudaStatus_t libreCuBroadcastLastForm(int *pFormOut) {
    LIBRECUDA_VALIDATE(pFormOut != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    *pFormOut = g_last_broadcast_form;
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t libreCuBroadcast(void *const *bufs, int root, size_t byteCount, int nDev, const LibreCUstream *streams,
                                   int useNccl) {
    return lcu_guarded([&]() -> libreCudaStatus_t {
        LIBRECUDA_VALIDATE(bufs != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        std::vector<int> devs;
        LIBRECUDA_ERR_PROPAGATE(check_group(nDev, streams, &devs));
        LIBRECUDA_VALIDATE(root >= 0 && root < nDev, LIBRECUDA_ERROR_INVALID_VALUE);
        for (int r = 0; r < nDev; ++r) LIBRECUDA_VALIDATE(bufs[r] != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        LIBRECUDA_VALIDATE(useNccl >= 0 && useNccl <= 5, LIBRECUDA_ERROR_INVALID_VALUE);
        if (useNccl != 1) LIBRECUDA_ERR_PROPAGATE(check_reachable(nDev, streams, bufs));
        for (int r = 0; r < nDev; ++r) LIBRECUDA_ERR_PROPAGATE(commence(streams[r]));
        if (byteCount == 0 || nDev == 1) LIBRECUDA_SUCCEED();
        std::vector<cudaStream_t> mains((size_t)nDev);
        for (int r = 0; r < nDev; ++r) mains[(size_t)r] = streams[r]->main;
        if (useNccl == 5) {
            // Two complementary binary trees of fused kernels (tree_bcast_kernel, lcb_bcast_tree_plan): half of the
            // chunks per tree, one launch per GPU, 8 KiB chunks by ticket, one CTA per SM.  Same requirements and
            // fall-back as the ring.  Measured, 4 GiB / 1 GiB: 683 / 637 GB/s at 8 GPUs (ring 678 / 612, NCCL 668 /
            // 633), 694 / 669 at 4 (ring 693 / 663, NCCL 673 / 649); time = bytes / 690 GB/s + 0.18 ms at 8 GPUs.  More
            // than one CTA per SM is slower here (577-589 with 222 / 296 CTAs).
            bool aligned = true;
            for (int r = 0; r < nDev; ++r) aligned = aligned && (reinterpret_cast<uintptr_t>(bufs[r]) & 15) == 0;
            const size_t body = byteCount & ~(size_t)15;
            if (aligned && body > 0) {
                const int chunk_kib = lcb_tune_get("bcast_ring_chunk_kib") > 0 ? lcb_tune_get("bcast_ring_chunk_kib") : 8;
                const size_t chunk = (size_t)chunk_kib << 10;
                const size_t words = (body + chunk - 1) / chunk;
                std::vector<unsigned int *> flags((size_t)nDev, nullptr);
                for (int r = 0; r < nDev; ++r) LIBRECUDA_ERR_PROPAGATE(ring_flags_for(devs[(size_t)r], words, &flags[(size_t)r]));
                LIBRECUDA_ERR_PROPAGATE(cross_join(nDev, streams));  // nobody may still be reading or writing the buffers
                const unsigned int epoch = ++g_ring_epoch;
                const int ctas = lcb_tune_get("bcast_ring_ctas");
                for (int k = 0; k < nDev; ++k) {  // the root first, then in chain order: parents come before children
                    const int d = (root + k) % nDev;
                    int parents[2], kids[4];
                    LIBRECUDA_VALIDATE(lcb_bcast_tree_plan(nDev, root, d, parents, kids) == 0, LIBRECUDA_ERROR_UNKNOWN);
                    void *kid_bufs[4], *kid_flags[4];
                    for (int c = 0; c < 4; ++c) {
                        kid_bufs[c] = kids[c] < 0 ? nullptr : bufs[kids[c]];
                        kid_flags[c] = kids[c] < 0 ? nullptr : flags[(size_t)kids[c]];
                    }
                    LIBRECUDA_ERR_PROPAGATE(bind(streams[d]->ctx));
                    LCU_LCB(lcb_bcast_tree_node(bufs[d], d == root ? nullptr : flags[(size_t)d], kid_bufs, kid_flags, body, chunk,
                                                words / 2, epoch, 2000, ctas, streams[d]->main));
                }
                if (body < byteCount) {  // the last few bytes: plain stores from the root into every buffer
                    LIBRECUDA_ERR_PROPAGATE(bind(streams[root]->ctx));
                    const uint8_t *src = static_cast<const uint8_t *>(bufs[root]);
                    for (int g = 0; g < nDev; ++g)
                        if (g != root)
                            LCU_LCB(lcb_copy_d2d(static_cast<uint8_t *>(bufs[g]) + body, src + body, byteCount - body, streams[root]->main));
                }
                LIBRECUDA_ERR_PROPAGATE(cross_join(nDev, streams));
                g_last_broadcast_form = 5;
                return rebind_current();
            }
            useNccl = nDev == 2 ? 0 : 2;
        }
        if (useNccl == 4) {
            // Ring of kernels: one launch per GPU that receives and forwards in small chunks through flags in peer
            // memory.  All buffers must be 16-byte aligned; otherwise the engine chain runs.  Two kernels:
            //   one chunk per warp (ring_bcast_warp_kernel, the default): 8 KiB chunks handed out by ticket, one CTA
            //     per SM.  Measured, 4 GiB: 693 GB/s at 4 GPUs (NCCL 673, engine chain 689), 676-678 at 8 (NCCL 668);
            //     with a fixed stride instead of tickets 671-687 / 641-673 and a strong dependence on the grid.
            //     Time = bytes / 705 GB/s + 0.15 ms at 4 GPUs, + 0.25-0.30 ms at 8: every hop adds about the time
            //     the chunks in flight take to drain, which is what the two trees of form 5 shorten.
            //   one chunk per CTA (ring_bcast_kernel, tunable bcast_ring_warp = 0): 128 KiB chunks x 296 CTAs, 676 at 4
            //     GPUs and 654 at 8 (+ 0.22 / 0.47 ms); 590 with 64 KiB, 369 with 32 KiB chunks, because the whole CTA
            //     idles while one thread's release waits for the remote stores to be acknowledged.
            bool aligned = true;
            for (int r = 0; r < nDev; ++r) aligned = aligned && (reinterpret_cast<uintptr_t>(bufs[r]) & 15) == 0;
            const size_t body = byteCount & ~(size_t)15;
            if (aligned && body > 0) {
                const bool per_warp = lcb_tune_get("bcast_ring_warp") != 0;
                const int chunk_kib = lcb_tune_get("bcast_ring_chunk_kib") > 0 ? lcb_tune_get("bcast_ring_chunk_kib") : (per_warp ? 8 : 128);
                const size_t chunk = (size_t)chunk_kib << 10;
                const size_t words = (body + chunk - 1) / chunk;
                std::vector<unsigned int *> flags((size_t)nDev, nullptr);
                for (int r = 0; r < nDev; ++r) LIBRECUDA_ERR_PROPAGATE(ring_flags_for(devs[(size_t)r], words, &flags[(size_t)r]));
                LIBRECUDA_ERR_PROPAGATE(cross_join(nDev, streams));  // nobody may still be reading or writing the buffers
                const unsigned int epoch = ++g_ring_epoch;
                const int ctas = lcb_tune_get("bcast_ring_ctas");  // 0: one CTA per SM with a chunk per warp, two per CTA
                for (int k = 0; k < nDev; ++k) {
                    const int d = (root + k) % nDev, nx = (root + k + 1) % nDev;
                    const bool last = k + 1 == nDev;
                    LIBRECUDA_ERR_PROPAGATE(bind(streams[d]->ctx));
                    LCU_LCB(lcb_bcast_ring_hop(bufs[d], last ? nullptr : bufs[nx], k == 0 ? nullptr : flags[(size_t)d],
                                               last ? nullptr : flags[(size_t)nx], body, chunk, epoch, 2000, ctas, streams[d]->main));
                }
                if (body < byteCount) {  // the last few bytes: plain stores from the root into every buffer
                    LIBRECUDA_ERR_PROPAGATE(bind(streams[root]->ctx));
                    const uint8_t *src = static_cast<const uint8_t *>(bufs[root]);
                    for (int g = 0; g < nDev; ++g)
                        if (g != root)
                            LCU_LCB(lcb_copy_d2d(static_cast<uint8_t *>(bufs[g]) + body, src + body, byteCount - body, streams[root]->main));
                }
                LIBRECUDA_ERR_PROPAGATE(cross_join(nDev, streams));
                g_last_broadcast_form = 4;
                return rebind_current();
            }
            useNccl = nDev == 2 ? 0 : 2;
        }
        if (useNccl == 3) {
            // Multicast (see bcast_multicast).  Needs multicast support on every GPU and a 16-byte aligned root
            // buffer; otherwise the call falls back to the copy-engine chain (form 2; form 0 with two GPUs).
            // Running the chain beside it on a share of the bytes does not add the two rates up: the mix measured
            // 410-505 GB/s at 4 GPUs for every split, below either path alone (543 and 689).
            const int piece_mib = lcb_tune_get("bcast_mc_piece_mib") > 0 ? lcb_tune_get("bcast_mc_piece_mib") : 256;
            const int slots = lcb_tune_get("bcast_mc_slots") >= 2 ? lcb_tune_get("bcast_mc_slots") : 2;
            const size_t piece = (size_t)piece_mib << 20;
            const McWindow *win = nullptr;
            int rc = -1;
            if ((reinterpret_cast<uintptr_t>(bufs[root]) & 15) == 0) rc = mc_window_acquire(devs.data(), nDev, piece * (size_t)slots, &win);
            if (rc > 0) {
                LIBRECUDA_DEBUG("multicast window could not be created (CUresult " << rc << "); using the copy-engine chain");
                rc = -1;
            }
            if (rc == 0) {
                LIBRECUDA_ERR_PROPAGATE(cross_join(nDev, streams));
                LIBRECUDA_ERR_PROPAGATE(bcast_multicast(bufs, root, 0, byteCount, nDev, streams, mains, win, piece, slots));
                LIBRECUDA_ERR_PROPAGATE(cross_join(nDev, streams));
                g_last_broadcast_form = 3;
                return rebind_current();
            }
            useNccl = nDev == 2 ? 0 : 2;
        }
        if (useNccl == 2) {
            LIBRECUDA_ERR_PROPAGATE(cross_join(nDev, streams));
            LIBRECUDA_ERR_PROPAGATE(bcast_chain(bufs, root, 0, byteCount, nDev, streams, mains));
            LIBRECUDA_ERR_PROPAGATE(cross_join(nDev, streams));
            g_last_broadcast_form = 2;
            return rebind_current();
        }
        if (useNccl == 1) {
            Nccl *n = nccl();
            LIBRECUDA_VALIDATE(n != nullptr, LIBRECUDA_ERROR_NOT_FOUND);
            LIBRECUDA_ERR_PROPAGATE(nccl_group_for(n, devs));
            for (int r = 0; r < nDev; ++r) {  // NCCL runs on the main lanes: they first absorb async work
                LIBRECUDA_ERR_PROPAGATE(bind(streams[r]->ctx));
                LIBRECUDA_ERR_PROPAGATE(join_sides(streams[r]));
            }
            LCU_NCCL(n, n->GroupStart());
            for (int r = 0; r < nDev; ++r)
                LCU_NCCL(n, n->Broadcast(bufs[root], bufs[r], byteCount, ncclUint8, root, n->comms[r], streams[r]->main));
            LCU_NCCL(n, n->GroupEnd());
            g_last_broadcast_form = 1;
            return rebind_current();
        }
        g_last_broadcast_form = 0;
        // Own path.  The buffer is cut into one shard per non-root device, each shard into pieces.
        //   pull lane of device g : loads piece after piece of shard g from the root (every byte leaves the root
        //                           exactly once; remote loads are the faster direction while the root only sends);
        //   push lane of device g : as soon as a piece has landed, stores it to every other non-root device (with
        //                           all those links busy in both directions, stores are the faster form).
        // The two lanes are separate CUDA streams tied by one event per piece, so forwarding piece p overlaps the
        // arrival of piece p+1 and the whole broadcast takes about one buffer's worth of link time.
        std::vector<int> owners;
        for (int g = 0; g < nDev; ++g)
            if (g != root) owners.push_back(g);
        const int parts = (int)owners.size();
        size_t off[17];
        LIBRECUDA_ERR_PROPAGATE(libreCuPartitionPlan(byteCount, parts, 0, off));
        LIBRECUDA_ERR_PROPAGATE(cross_join(nDev, streams));
        const uint8_t *src = static_cast<const uint8_t *>(bufs[root]);
        // one piece when there is nobody to forward to; otherwise pipelined pieces (64 MiB by default)
        const int piece_mib = lcb_tune_get("bcast_piece_mib") > 0 ? lcb_tune_get("bcast_piece_mib") : 64;
        const int pull_ctas = lcb_tune_get("bcast_pull_ctas") > 0 ? lcb_tune_get("bcast_pull_ctas") : 74;
        // Programmatic dependent launch parks the next kernel's CTAs on the SMs while they wait; good for one
        // stream of back-to-back copies, bad here, where two lanes of every device must share the SMs (measured:
        // 8.7 ms with it, 7.2 ms without at 4 GPUs).  Every launch of this call asks for a plain launch.
        constexpr int kPlain = LCB_COPY_NO_PDL;
        const size_t kPiece = parts > 1 ? ((size_t)piece_mib << 20) : ~(size_t)0;
        std::vector<cudaEvent_t> to_destroy;
        std::vector<cudaStream_t> push_lane(parts, nullptr);
        if (parts > 1) {
            for (int k = 0; k < parts; ++k) {
                LibreCUstream sg = streams[owners[k]];
                if (off[k + 1] == off[k]) continue;
                LIBRECUDA_ERR_PROPAGATE(bind(sg->ctx));
                LIBRECUDA_ERR_PROPAGATE(fork_side(sg, 0, &push_lane[k]));  // starts where the stream stands now
            }
        }
        // pieces outermost, devices innermost: every device gets its first work within microseconds of the call
        bool more = true;
        for (size_t piece = 0; more; ++piece) {
            more = false;
            for (int k = 0; k < parts; ++k) {
                const size_t shard = off[k + 1] - off[k];
                if (kPiece != ~(size_t)0 ? piece * kPiece >= shard : piece > 0 || shard == 0) continue;
                const size_t p = off[k] + (kPiece != ~(size_t)0 ? piece * kPiece : 0);
                const size_t n = (kPiece == ~(size_t)0 || off[k + 1] - p < kPiece) ? off[k + 1] - p : kPiece;
                if (p + n < off[k + 1]) more = true;
                const int g = owners[k];
                LibreCUstream sg = streams[g];
                LIBRECUDA_ERR_PROPAGATE(bind(sg->ctx));
                uint8_t *mine = static_cast<uint8_t *>(bufs[g]);
                // The pull shares the root's port with all the other devices, so it is slow by construction; with a
                // full grid its waiting CTAs would fill every SM and starve the forwarding kernels of this device
                // (measured: the broadcast took twice as long).  74 looping CTAs carry the pull's share comfortably.
                if (push_lane[k] == nullptr) LCU_LCB(lcb_copy_d2d_ex(mine + p, src + p, n, LCB_COPY_AUTO | kPlain, 0, sg->main));
                else LCU_LCB(lcb_copy_d2d_ex(mine + p, src + p, n, LCB_COPY_VEC | kPlain, pull_ctas, sg->main));
                if (push_lane[k] == nullptr) continue;
                cudaEvent_t landed;
                LCU_CUDA(cudaEventCreateWithFlags(&landed, cudaEventDisableTiming));
                to_destroy.push_back(landed);
                LCU_CUDA(cudaEventRecord(landed, sg->main));
                LCU_CUDA(cudaStreamWaitEvent(push_lane[k], landed, 0));
                for (int step = 1; step < parts; ++step) {  // rotate the targets so the stores spread over the peers
                    const int q = owners[(k + step) % parts];
                    LCU_LCB(lcb_copy_d2d_ex(static_cast<uint8_t *>(bufs[q]) + p, mine + p, n, LCB_COPY_AUTO | kPlain, 0, push_lane[k]));
                }
            }
        }
        for (cudaEvent_t e : to_destroy) (void)cudaEventDestroy(e);
        LIBRECUDA_ERR_PROPAGATE(cross_join(nDev, streams));  // takes the push lanes in first
        return rebind_current();
    });
}

// ---- inter-process sharing -------------------------------------------------------------------------------------
// handle layout: cudaIpcMemHandle_t (64 bytes) followed by the 8-byte offset of the pointer inside the
// underlying CUDA allocation.

libreCudaStatus_t libreCuIpcGetMemHandle(void *handle, void *devicePointer) {
    LIBRECUDA_VALIDATE(handle != nullptr && devicePointer != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LCU_ENSURE_CTX();
    auto &allocs = globals().allocations;
    auto it = allocs.find(reinterpret_cast<uintptr_t>(devicePointer));
    LIBRECUDA_VALIDATE(it != allocs.end(), LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(!it->second.mapped && !it->second.ipc, LIBRECUDA_ERROR_INVALID_VALUE);
    LCU_CUDA(cudaSetDevice(it->second.device));
    cudaIpcMemHandle_t h;
    LCU_CUDA(cudaIpcGetMemHandle(&h, it->second.raw));
    const uint64_t offset = reinterpret_cast<uintptr_t>(devicePointer) - reinterpret_cast<uintptr_t>(it->second.raw);
    std::memcpy(handle, &h, sizeof(h));
    std::memcpy(static_cast<uint8_t *>(handle) + sizeof(h), &offset, sizeof(offset));
    return rebind_current();
}

libreCudaStatus_t libreCuIpcOpenMemHandle(void **pDevicePointer, const void *handle) {
    LIBRECUDA_VALIDATE(pDevicePointer != nullptr && handle != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LCU_ENSURE_CTX();
    LIBRECUDA_ERR_PROPAGATE(bind(globals().current));
    cudaIpcMemHandle_t h;
    uint64_t offset = 0;
    std::memcpy(&h, handle, sizeof(h));
    std::memcpy(&offset, static_cast<const uint8_t *>(handle) + sizeof(h), sizeof(offset));
    void *raw = nullptr;
    LCU_CUDA(cudaIpcOpenMemHandle(&raw, h, cudaIpcMemLazyEnablePeerAccess));
    void *p = static_cast<uint8_t *>(raw) + offset;
    // opening with cudaIpcMemLazyEnablePeerAccess gave this context access to the exporting GPU's memory
    const int opener = globals().current->device->ordinal;
    int owner = opener;
    cudaPointerAttributes attr{};
    if (cudaPointerGetAttributes(&attr, raw) == cudaSuccess && attr.type == cudaMemoryTypeDevice) {
        globals().current->peers.insert(attr.device);
        owner = attr.device;
    } else {
        (void)cudaGetLastError();
    }
    // size unknown on this side: register the page that holds the pointer so classification sees device memory;
    // the CUDA driver answers for the rest of the range.  The recorded owner is the exporting GPU, which is also
    // what the driver reports beyond this page, so every offset into the mapping has the same owner.
    globals().allocations[reinterpret_cast<uintptr_t>(p)] = Allocation{raw, 4096, owner, false, true, opener};
    *pDevicePointer = p;
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t libreCuIpcCloseMemHandle(void *devicePointer) {
    LIBRECUDA_VALIDATE(devicePointer != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    auto &allocs = globals().allocations;
    auto it = allocs.find(reinterpret_cast<uintptr_t>(devicePointer));
    LIBRECUDA_VALIDATE(it != allocs.end() && it->second.ipc, LIBRECUDA_ERROR_INVALID_VALUE);
    LCU_CUDA(cudaSetDevice(it->second.opener >= 0 ? it->second.opener : it->second.device));
    void *raw = it->second.raw;
    allocs.erase(it);
    LCU_CUDA(cudaIpcCloseMemHandle(raw));
    return rebind_current();
}
