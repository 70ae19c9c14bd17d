// librecuda.h -- public C API of the B200-native data-movement library.
//
// Part 1 is the drop-in boundary: the 30 `libreCu*` entry points, handle typedefs, context flags
// and attribute enums of the reference header (driverapi/include/librecuda.h:9-114), with identical
// names, parameter types, default arguments and `extern "C"` linkage, so programs written against
// the reference (its tests/*/main.cpp) compile and link unchanged.  Each declaration cites the
// reference declaration (header line) and implementation (driverapi/src/librecuda.cpp lines) it
// stands in for.
//
// Part 2 is additive: memset, direction-checked copies, cross-stream event waits and the multi-GPU
// (peer / partitioned / all-to-all / broadcast / IPC) entry points.  The reference has no counterpart
// for any of them; they follow the same conventions (status return, stream-recorded execution,
// validation line on stderr, no exceptions across the ABI).
//
// Execution contract (reference: librecuda.h:98-112, driverapi/src/cmdqueue.cpp:821-868):
// every stream operation is *recorded*; recorded work is submitted to the GPU by
// libreCuStreamCommence and is complete -- results visible to the host -- after libreCuStreamAwait
// (or libreCuEventSynchronize for work recorded before that event).  `async=false` orders an
// operation after everything recorded earlier on its stream; `async=true` lets it overlap earlier
// operations of the same stream (cmdqueue.cpp:480-487,715-727).
#ifndef LIBRECUDA_B200_H
#define LIBRECUDA_B200_H

#include <cstddef>
#include <cstdint>

#include "librecuda_status.h"

#define LIBRECUDA_EXPORT extern "C"

// ---------------------------------------------------------------------------------------------
// Part 1 -- reference surface
// ---------------------------------------------------------------------------------------------

// Opaque handles (reference librecuda.h:9-21).  Device handles are owned by the library; contexts,
// modules, streams and events are released by their Destroy / Unload call.
struct LibreCUdevice_;
struct LibreCUcontext_;
struct LibreCUmodule_;
struct LibreCUFunction_;
struct LibreCUstream_;
struct LibreCUEvent_;
typedef LibreCUdevice_ *LibreCUdevice;
typedef LibreCUcontext_ *LibreCUcontext;
typedef LibreCUmodule_ *LibreCUmodule;
typedef LibreCUFunction_ *LibreCUFunction;
typedef LibreCUstream_ *LibreCUstream;
typedef LibreCUEvent_ *LibreCUEvent;

// Host wait style used by libreCuStreamAwait / libreCuEventSynchronize (reference librecuda.h:23-25,
// cmdqueue.cpp:334-357).  BLOCKING_SYNC, which throws in the reference, blocks in the driver here.
#define CU_CTX_SCHED_SPIN 0x01
#define CU_CTX_SCHED_YIELD 0x02
#define CU_CTX_SCHED_BLOCKING_SYNC 0x04

// Numeric values follow the CUDA driver API (reference librecuda.h:27-35).
enum LibreCuDeviceAttribute {
    CU_DEVICE_ATTRIBUTE_MAX_SHARED_MEMORY_PER_BLOCK = 8,
    CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR = 75,
    CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR = 76,
    CU_DEVICE_ATTRIBUTE_MAX_SHARED_MEMORY_PER_BLOCK_OPTIN = 97
};
enum LibreCuFunctionAttribute {
    CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES = 8,
};

// --- initialisation, devices, contexts ---------------------------------------------------------

// ref librecuda.h:37, librecuda.cpp:80-210.  Idempotent; `flags` unused.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuInit(int flags);
// ref librecuda.h:39, librecuda.cpp:216-221.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuDeviceGetCount(int *pDeviceCount);
// ref librecuda.h:41, librecuda.cpp:223-229.  Out-of-range ordinal -> INVALID_DEVICE.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuDeviceGet(LibreCUdevice *device, int deviceOrdinal);
// ref librecuda.h:43, librecuda.cpp:232-241.  Unknown code -> *pStatusName = nullptr, SUCCESS.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuGetErrorString(libreCudaStatus_t status, const char **pStatusName);
// ref librecuda.h:45, librecuda.cpp:393-625.  The new context becomes the process-wide current one.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuCtxCreate_v2(LibreCUcontext *pCtx, int flags, LibreCUdevice device);
// ref librecuda.h:47, librecuda.cpp:627-641.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuCtxDestroy(LibreCUcontext ctx);
// ref librecuda.h:49, librecuda.cpp:643-647.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuCtxSetCurrent(LibreCUcontext ctx);
// ref librecuda.h:51, librecuda.cpp:1511-1515.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuCtxGetCurrent(LibreCUcontext *pCtxOut);
// ref librecuda.h:63, librecuda.cpp:1499-1509.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuDeviceGetName(char *pDeviceName, int length, LibreCUdevice device);
// ref librecuda.h:65, librecuda.cpp:1517-1586.  Only the four LibreCuDeviceAttribute values.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuDeviceGetAttribute(int *pValOut, LibreCuDeviceAttribute attribute, LibreCUdevice device);

// --- memory ---------------------------------------------------------------------------------------

// ref librecuda.h:53, librecuda.cpp:738-750 (gpuAlloc :688-736).  bytesize 0 / null -> INVALID_VALUE.
// Pointers are at least 4 KiB aligned.  mapToCpu=true returns memory the host may dereference at the
// same address.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuMemAlloc(void **pDevicePointer, size_t bytesize, bool mapToCpu = false);
// ref librecuda.h:55, librecuda.cpp:873-885.  Direction is inferred from the pointers: device->device
// runs the copy kernels of this library (reference: memcpyD2D, driverapi/src/memcopy.cpp:77-158),
// anything touching host memory goes to the copy engines (reference: gpuMemcpy, cmdqueue.cpp:732-786).
LIBRECUDA_EXPORT libreCudaStatus_t libreCuMemCpy(void *dst, void *src, size_t byteCount, LibreCUstream stream, bool async = false);
// ref librecuda.h:57, librecuda.cpp:864-871.  Pointer must be an allocation base.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuMemFree(void *devicePointer);

// --- streams ----------------------------------------------------------------------------------------

// ref librecuda.h:59, librecuda.cpp:1462-1473.  Bound to the context current at creation.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuStreamCreate(LibreCUstream *pStreamOut, uint32_t flags);
// ref librecuda.h:61, librecuda.cpp:1489-1497.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuStreamDestroy(LibreCUstream stream);
// ref librecuda.h:111, librecuda.cpp:1476-1480 -> cmdqueue.cpp:821-868.  Submits everything recorded so far.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuStreamCommence(LibreCUstream stream);
// ref librecuda.h:112, librecuda.cpp:1483-1487 -> cmdqueue.cpp:272-277.  Blocks until submitted work is done.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuStreamAwait(LibreCUstream stream);

// --- modules, functions, launches ---------------------------------------------------------------------

// ref librecuda.h:67, librecuda.cpp:1588-1609.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuFuncSetAttribute(LibreCUFunction function, LibreCuFunctionAttribute attribute, int value);
// ref librecuda.h:69-70, librecuda.cpp:944-1379.  The image is copied; the caller keeps its buffer.
LIBRECUDA_EXPORT libreCudaStatus_t
libreCuModuleLoadData(LibreCUmodule *pModuleOut, const void *image, size_t imageSize);
// ref librecuda.h:72, librecuda.cpp:1382-1387.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuModuleGetFunctionCount(uint32_t *count, LibreCUmodule mod);
// ref librecuda.h:74-75, librecuda.cpp:1389-1397.  numFunctions must be >= the function count.
LIBRECUDA_EXPORT libreCudaStatus_t
libreCuModuleEnumerateFunctions(LibreCUFunction *functionsOut, uint32_t numFunctions, LibreCUmodule mod);
// ref librecuda.h:77, librecuda.cpp:1456-1460.  Library-owned string.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuFuncGetName(const char **pNameOut, LibreCUFunction func);
// ref librecuda.h:79-80, librecuda.cpp:1399-1417.  Unknown name -> NOT_FOUND.
LIBRECUDA_EXPORT libreCudaStatus_t
libreCuModuleGetFunction(LibreCUFunction *pFunc, LibreCUmodule module, const char *name);
// ref librecuda.h:82-90, librecuda.cpp:1419-1441 -> cmdqueue.cpp:459-729.  kernelParams[i] points at
// the i-th argument value; the values are captured when this call returns.  numParams must equal the
// kernel's parameter count.  `extra` is ignored.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuLaunchKernel(LibreCUFunction function,
                                                       uint32_t gridDimX, uint32_t gridDimY,
                                                       uint32_t gridDimZ,
                                                       uint32_t blockDimX, uint32_t blockDimY,
                                                       uint32_t blockDimZ,
                                                       uint32_t sharedMemBytes, LibreCUstream stream,
                                                       void **kernelParams, size_t numParams,
                                                       void **extra,
                                                       bool async = false);
// ref librecuda.h:114, librecuda.cpp:1443-1454.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuModuleUnload(LibreCUmodule module);

// --- events (ref librecuda.h:92-96, librecuda.cpp:1617-1655, cmdqueue.cpp:896-955) -----------------------

LIBRECUDA_EXPORT libreCudaStatus_t libreCuEventCreate(LibreCUEvent *pEventOut, uint32_t flags);
// Recorded into the stream; takes effect once the stream is commenced.  Unlike the reference's
// one-shot events, an event may be recorded again.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuEventRecord(LibreCUEvent event, LibreCUstream stream);
// Never recorded -> INVALID_VALUE.  Recorded but its stream not commenced yet -> NOT_READY (the
// reference would spin forever).
LIBRECUDA_EXPORT libreCudaStatus_t libreCuEventSynchronize(LibreCUEvent event);
// Both events must belong to the same stream (else INVALID_VALUE); NOT_READY until both were reached.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuEventElapsedTime(float *pMillisecondsOut, LibreCUEvent start, LibreCUEvent end);
LIBRECUDA_EXPORT libreCudaStatus_t libreCuEventDestroy(LibreCUEvent event);

// ---------------------------------------------------------------------------------------------
// Part 2 -- additive entry points (no counterpart in the reference)
// ---------------------------------------------------------------------------------------------

// Direction-checked copies.  The pointer classes must match the name, else INVALID_VALUE.  The plain
// form is ordered like libreCuMemCpy(..., async=false); the *Async form is async=true.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuMemcpyHtoD(void *dstDevice, const void *srcHost, size_t byteCount, LibreCUstream stream);
LIBRECUDA_EXPORT libreCudaStatus_t libreCuMemcpyHtoDAsync(void *dstDevice, const void *srcHost, size_t byteCount, LibreCUstream stream);
LIBRECUDA_EXPORT libreCudaStatus_t libreCuMemcpyDtoH(void *dstHost, const void *srcDevice, size_t byteCount, LibreCUstream stream);
LIBRECUDA_EXPORT libreCudaStatus_t libreCuMemcpyDtoHAsync(void *dstHost, const void *srcDevice, size_t byteCount, LibreCUstream stream);
LIBRECUDA_EXPORT libreCudaStatus_t libreCuMemcpyDtoD(void *dstDevice, const void *srcDevice, size_t byteCount, LibreCUstream stream);
LIBRECUDA_EXPORT libreCudaStatus_t libreCuMemcpyDtoDAsync(void *dstDevice, const void *srcDevice, size_t byteCount, LibreCUstream stream);

// Page-locked host memory (copies to and from it run at full PCIe rate and do not block the host).
LIBRECUDA_EXPORT libreCudaStatus_t libreCuMemAllocHost(void **pHostPointer, size_t bytesize);
LIBRECUDA_EXPORT libreCudaStatus_t libreCuMemFreeHost(void *hostPointer);

// Memset on device memory.  D16 / D32 destinations must be 2 / 4 byte aligned; counts are elements.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuMemsetD8(void *dstDevice, unsigned char value, size_t count, LibreCUstream stream);
LIBRECUDA_EXPORT libreCudaStatus_t libreCuMemsetD8Async(void *dstDevice, unsigned char value, size_t count, LibreCUstream stream);
LIBRECUDA_EXPORT libreCudaStatus_t libreCuMemsetD16(void *dstDevice, unsigned short value, size_t count, LibreCUstream stream);
LIBRECUDA_EXPORT libreCudaStatus_t libreCuMemsetD16Async(void *dstDevice, unsigned short value, size_t count, LibreCUstream stream);
LIBRECUDA_EXPORT libreCudaStatus_t libreCuMemsetD32(void *dstDevice, unsigned int value, size_t count, LibreCUstream stream);
LIBRECUDA_EXPORT libreCudaStatus_t libreCuMemsetD32Async(void *dstDevice, unsigned int value, size_t count, LibreCUstream stream);

// Make work recorded on `stream` after this call wait, on the GPU, for `event` (recorded on any
// stream of any context).  The event's stream must be commenced before or together with `stream`;
// libreCuStreamCommence(stream) returns NOT_READY if the event was recorded but never submitted.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuStreamWaitEvent(LibreCUstream stream, LibreCUEvent event);
// SUCCESS once the event was reached, NOT_READY before.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuEventQuery(LibreCUEvent event);
// GPU time of a reached event in nanoseconds since the event's context was created.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuEventGetTimestamp(uint64_t *pNanosecondsOut, LibreCUEvent event);

// Peer access between the contexts of one process (NVLink / NVSwitch).
LIBRECUDA_EXPORT libreCudaStatus_t libreCuDeviceCanAccessPeer(int *pCanAccess, LibreCUdevice device, LibreCUdevice peerDevice);
// Lets kernels and copies of the current context reach memory allocated in `peerCtx`.  Idempotent.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuCtxEnablePeerAccess(LibreCUcontext peerCtx, unsigned int flags);
// Copy between device buffers that may live on different GPUs: by the copy kernel on the GPU that owns
// `stream` (stores to, or loads from, the peer over NVLink) or, between two GPUs from 64 MiB up, by the copy
// engines (the faster form there; lcb_tune("peer_copy_engine", MiB) moves the threshold, 0 = never).
LIBRECUDA_EXPORT libreCudaStatus_t libreCuMemcpyPeer(void *dstDevice, const void *srcDevice, size_t byteCount, LibreCUstream stream, bool async = false);

// offsetsOut[0..parts] <- boundaries of `parts` contiguous shards of `totalBytes`, every interior
// boundary a multiple of `alignBytes` (power of two; 0 selects 2 MiB); the last shard takes the tail.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuPartitionPlan(size_t totalBytes, int parts, size_t alignBytes, size_t *offsetsOut);
// Scatter: shard g of `src` (libreCuPartitionPlan boundaries) is copied to dsts[g] on streams[g].
LIBRECUDA_EXPORT libreCudaStatus_t libreCuMemcpyPartitioned(void *const *dsts, const void *src, size_t totalBytes, int parts, size_t alignBytes, const LibreCUstream *streams);
// One rank's half of an all-to-all over peer-mapped buffers: chunk j of `sendBuf` is stored into
// peerRecvBufs[j] + rank * chunkBytes, for every j in [0, nRanks), by one kernel on `stream`.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuAllToAllPush(void *const *peerRecvBufs, const void *sendBuf, size_t chunkBytes, int nRanks, int rank, LibreCUstream stream);
// The same exchange by remote loads: chunk `rank` of peerSendBufs[j] is
// loaded into recvBuf + j * chunkBytes, for every j, by one kernel on `stream`.  Peers' send buffers must be
// complete before this runs and unchanged until every rank has finished.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuAllToAllPull(void *const *peerSendBufs, void *recvBuf, size_t chunkBytes, int nRanks, int rank, LibreCUstream stream);
// The same exchange on the COPY ENGINES for one process per GPU (the fastest form measured on NVLink 5 from
// chunks of 64 MiB up: 734-756 GB/s per GPU against 707 for the push kernel): nRanks - 1 peer copies recorded on
// `stream`, the local chunk by a kernel beside them, the ranks kept in lock-step -- every GPU has exactly one
// sender at a time -- through flag words in each other's memory.  peerFlags[j] points at rank j's flag words
// (nRanks unsigned ints of device memory, zero before the first call, mapped into this process; peerFlags[rank]
// are this rank's own); `epoch` is 1, 2, 3 ... , the same on every rank for the same exchange; a rank that waits
// longer than timeoutMs (1..10000) for a peer goes on unsynchronised and the next libreCuStreamAwait returns
// LIBRECUDA_ERROR_UNKNOWN.  With nRanks <= 2 no flags are needed (peerFlags may be NULL).
LIBRECUDA_EXPORT libreCudaStatus_t libreCuAllToAllEngines(void *const *peerRecvBufs, const void *sendBuf, size_t chunkBytes, int nRanks, int rank, void *const *peerFlags, unsigned int epoch, unsigned int timeoutMs, LibreCUstream stream);
// Single-process collectives over the devices of `streams[0..nDev)` (one stream per device, peer
// access enabled).  useNccl == 1 runs them through NCCL (ncclSend/ncclRecv, ncclBroadcast); useNccl == 0 runs
// the library's own peer-memory kernels; useNccl == 2 runs them on the copy engines: the all-to-all as G-1
// rotated peer copies per GPU (the fastest form measured on NVLink 5 when all GPUs exchange at once), the
// broadcast as a chain root -> next device -> ... pipelined in pieces with one event per piece and hop.
// libreCuBroadcast also takes useNccl == 3: NVLink multicast.  The root writes its buffer once with multimem
// stores to a multicast address, NVSwitch delivers a copy into a staging slab of the library on every GPU, and
// each GPU copies the pieces from its slab into its buffer; nothing is forwarded by a GPU, so the rate does not
// drop with the number of GPUs (measured 527-552 GB/s at 2 and 4 GPUs: multicast writes of one GPU are capped there,
// below the engine chain of form 2 at those counts).  The buffers themselves can be any device memory (any alignment on the
// receivers; a root buffer that is not 16-byte aligned, or GPUs without multicast support, take form 2 -- form 0
// with two GPUs -- instead).  The slabs (512 MiB per GPU by default) are created at the first call for a group
// of devices and released by libreCuCtxDestroy of any of them, or at exit.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuAllToAll(void *const *recvBufs, void *const *sendBufs, size_t chunkBytes, int nDev, const LibreCUstream *streams, int useNccl);
LIBRECUDA_EXPORT libreCudaStatus_t libreCuBroadcast(void *const *bufs, int root, size_t byteCount, int nDev, const LibreCUstream *streams, int useNccl);
// useNccl == 4: a ring of kernels, one launch per GPU, each receiving its buffer from the previous GPU of the chain
// root -> next device -> ... and forwarding it to the next in 128 KiB chunks as they arrive (remote stores, one flag
// word per chunk in the receiver's memory, bounded waits): the forwarding is fused into the copy, so a hop adds
// tens of microseconds where the engine chain of form 2 adds the time of a whole piece (676-679 GB/s at 4 GPUs).  Buffers
// must be 16-byte aligned (else form 2 runs).
// useNccl == 5: the same fused kernels over two complementary binary trees instead of one chain: the first half of the
// buffer goes down a tree over the non-root GPUs, the second half down a tree in which the inner nodes of the first
// are leaves, so the last GPU is 1 + log2(nDev - 1) hops from the root instead of nDev - 1 while every GPU still
// receives each byte once and sends at most one buffer's worth.  Same alignment rule and fall-back as form 4.
// The form the most recent libreCuBroadcast of this process actually ran (0..5; -1 before the first call): a
// request for form 3, 4 or 5 runs as 2 (0 with two GPUs) when its requirements are not met.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuBroadcastLastForm(int *pFormOut);

// Inter-process sharing of a libreCuMemAlloc allocation (one process per GPU).  `handle` points at
// LIBRECUDA_IPC_HANDLE_SIZE bytes that the exporting process sends to its peers by any means.
#define LIBRECUDA_IPC_HANDLE_SIZE 72
LIBRECUDA_EXPORT libreCudaStatus_t libreCuIpcGetMemHandle(void *handle, void *devicePointer);
LIBRECUDA_EXPORT libreCudaStatus_t libreCuIpcOpenMemHandle(void **pDevicePointer, const void *handle);
LIBRECUDA_EXPORT libreCudaStatus_t libreCuIpcCloseMemHandle(void *devicePointer);

// The raw CUDA stream behind a LibreCUstream (a cudaStream_t / CUstream), for interop with other
// CUDA code in the process.  Work launched on it directly is not tracked by Commence / Await.
LIBRECUDA_EXPORT libreCudaStatus_t libreCuStreamGetNativeHandle(void **pNativeStreamOut, LibreCUstream stream);

#endif  // LIBRECUDA_B200_H
