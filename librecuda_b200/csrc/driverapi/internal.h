// Internal records behind the opaque libreCu* handles, and the deferred command list of a stream.
//
// The reference keeps a hand-built GPFIFO push buffer per stream (driverapi/internal/cmdqueue.h:51-57,
// driverapi/src/cmdqueue.cpp:200-218).  Here a stream records small command objects and replays them into
// CUDA streams at libreCuStreamCommence; the GPU front end orders them, so no CPU round trip is needed
// when copies and kernels alternate (the reference waits on the CPU at every switch, cmdqueue.cpp:826-844).
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <map>
#include <memory>
#include <new>
#include <set>
#include <string>
#include <vector>

#include "host_logic.h"
#include "lcb200_kernels.h"
#include "librecuda.h"

// <cuda.h> cannot be included next to librecuda.h (both define the CU_DEVICE_ATTRIBUTE_* enumerators), so
// the handful of driver types used here are declared by hand; they are ABI-compatible with the driver's.
typedef struct CUmod_st *CUmodule;
typedef struct CUfunc_st *CUfunction;
typedef cudaStream_t CUstream;
typedef int CUresult;
typedef int CUfunction_attribute;
constexpr CUresult CUDA_SUCCESS = 0;
constexpr CUresult CUDA_ERROR_OUT_OF_MEMORY = 2;

namespace lcu {

// ---- status helpers -------------------------------------------------------------------------------
libreCudaStatus_t from_cuda(cudaError_t err);
libreCudaStatus_t from_cu(CUresult res);
const char *status_name(libreCudaStatus_t code);

#define LCU_CUDA(expr)                                                   \
    do {                                                                 \
        cudaError_t lcu_err_ = (expr);                                   \
        if (lcu_err_ != cudaSuccess) {                                   \
            LIBRECUDA_DEBUG(__FILE__ ":" LIBRECUDA_STR_(__LINE__) ": " #expr " -> " << cudaGetErrorName(lcu_err_)); \
            (void)cudaGetLastError();                                    \
            return lcu::from_cuda(lcu_err_);                             \
        }                                                                \
    } while (0)

#define LCU_CU(expr)                                                     \
    do {                                                                 \
        CUresult lcu_res_ = (expr);                                      \
        if (lcu_res_ != CUDA_SUCCESS) {                                  \
            LIBRECUDA_DEBUG(__FILE__ ":" LIBRECUDA_STR_(__LINE__) ": " #expr " -> CUresult " << (int)lcu_res_); \
            return lcu::from_cu(lcu_res_);                               \
        }                                                                \
    } while (0)

// status of an lcb_* launcher (0 or a cudaError_t value)
#define LCU_LCB(expr)                                                    \
    do {                                                                 \
        int lcu_rc_ = (expr);                                            \
        if (lcu_rc_ != 0) {                                              \
            LIBRECUDA_DEBUG(__FILE__ ":" LIBRECUDA_STR_(__LINE__) ": " #expr " -> " << lcu_rc_); \
            return lcu::from_cuda((cudaError_t)lcu_rc_);                 \
        }                                                                \
    } while (0)

// ---- driver entry points (modules and raw launches only; everything else is the runtime API) ------
struct DriverTable {
    CUresult (*ModuleLoadData)(CUmodule *, const void *);
    CUresult (*ModuleUnload)(CUmodule);
    CUresult (*ModuleGetFunction)(CUfunction *, CUmodule, const char *);
    CUresult (*ModuleGetFunctionCount)(unsigned int *, CUmodule);
    CUresult (*ModuleEnumerateFunctions)(CUfunction *, unsigned int, CUmodule);
    CUresult (*FuncGetName)(const char **, CUfunction);
    CUresult (*FuncGetParamInfo)(CUfunction, size_t, size_t *, size_t *);
    CUresult (*FuncSetAttribute)(CUfunction, CUfunction_attribute, int);
    CUresult (*FuncGetAttribute)(int *, CUfunction_attribute, CUfunction);
    CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream,
                             void **, void **);
};
// nullptr (and a message on stderr) when the CUDA driver is not usable in this process
const DriverTable *driver();

// ---- global state ------------------------------------------------------------------------------------
struct Allocation {
    void *raw;        // pointer returned by the CUDA allocator (what is freed)
    size_t size;      // usable bytes from the aligned pointer
    int device;       // the GPU whose memory it is (for an IPC mapping: the exporting process's GPU)
    bool mapped;      // host-dereferenceable (managed)
    bool ipc;         // opened from another process's handle
    int opener = -1;  // IPC mappings: the device that was current when the handle was opened (bound again to close it)
};

struct Globals {
    bool initialized = false;
    std::vector<std::unique_ptr<LibreCUdevice_>> devices;
    LibreCUcontext current = nullptr;
    std::map<uintptr_t, Allocation> allocations;  // keyed by the aligned pointer handed to the caller
};
Globals &globals();

enum class PtrClass { Host, Device };
// classification used for the direction dispatch of libreCuMemCpy (reference: isDevicePtr,
// driverapi/src/librecuda.cpp:821-836): library allocations first, then whatever the CUDA driver knows
PtrClass classify(const void *p);
// Device ordinal that owns a device pointer, or -1 when every device can reach it (managed memory) or the
// owner is unknown to both the library and the CUDA driver.
int owner_device(const void *p);

}  // namespace lcu

// ---- handle records -----------------------------------------------------------------------------------
struct LibreCUdevice_ {
    int ordinal = 0;
    std::string name;
    int cc_major = 0, cc_minor = 0;
    int smem_per_block = 0, smem_optin = 0;
    int max_block_x = 1024, max_block_y = 1024, max_block_z = 64, max_threads = 1024;
    int max_grid_x = 2147483647, max_grid_y = 65535, max_grid_z = 65535;
};

struct LibreCUcontext_ {
    LibreCUdevice device = nullptr;
    int flags = 0;
    // Event timestamps count from epochs[0], recorded at creation.  A new epoch is recorded in front of an
    // event when the newest one is older than a couple of seconds, so that the float distance CUDA reports
    // between an event and its epoch keeps sub-microsecond resolution however old the context is.
    struct Epoch {
        cudaEvent_t ev = nullptr;
        uint64_t host_ms = 0;  // host clock when it was recorded
    };
    std::vector<Epoch> epochs;
    std::vector<uint64_t> epoch_base_ns;  // offset of epochs[k] from epochs[0], valid below epochs_resolved
    size_t epochs_resolved = 0;
    std::set<int> peers;          // device ordinals whose memory this context may access
};

struct LibreCUFunction_ {
    LibreCUmodule module = nullptr;
    CUfunction fn = nullptr;
    std::string name;
    std::vector<size_t> param_offset, param_size;
    size_t param_bytes = 0;
    int dyn_smem_attr = 0;  // value given to libreCuFuncSetAttribute
};

struct LibreCUmodule_ {
    LibreCUcontext ctx = nullptr;
    CUmodule mod = nullptr;
    std::vector<std::unique_ptr<LibreCUFunction_>> functions;
};

struct LibreCUEvent_ {
    enum State { Never, Pending, Submitted };
    State state = Never;
    LibreCUstream stream = nullptr;
    LibreCUcontext ctx = nullptr;
    cudaEvent_t ev = nullptr;
    int device = -1;
    size_t epoch_idx = 0;  // the context epoch that was newest when the event was submitted
};

namespace lcu {

struct Command {
    enum Kind { CopyKernel, CopyEngine, Memset, Launch, EventRecord, WaitEvent, AllToAllPush, AllToAllPull, AllToAllEngines };
    Kind kind;
    bool async = false;
    // copies / memset
    void *dst = nullptr;
    const void *src = nullptr;
    size_t bytes = 0;
    cudaMemcpyKind copy_kind = cudaMemcpyDefault;
    unsigned int value = 0;
    int elem = 1;
    // launch
    LibreCUFunction fn = nullptr;
    unsigned grid[3] = {1, 1, 1}, block[3] = {1, 1, 1};
    unsigned smem = 0;
    std::vector<unsigned char> params;  // argument values captured at record time
    // events
    LibreCUEvent event = nullptr;
    // all-to-all (per-rank forms)
    std::vector<void *> peers;
    int rank = 0;
    std::vector<void *> peer_flags;  // lock-step engine form: every rank's flag words, own ones at [rank]
    unsigned int epoch = 0, timeout_ms = 0;
};

constexpr int kSideLanes = 8;
constexpr uint64_t kEpochRollMs = 2000;             // a new timestamp epoch once the newest is this old
constexpr int kStageSlots = 4;                      // pinned bounce slots per stream for pageable host copies
constexpr size_t kStageBytes = (size_t)8 << 20;    // bytes per slot
constexpr size_t kStageMinBytes = (size_t)1 << 20; // smaller pageable copies go straight to the runtime

}  // namespace lcu

struct LibreCUstream_ {
    LibreCUcontext ctx = nullptr;
    cudaStream_t main = nullptr;
    cudaStream_t side[lcu::kSideLanes] = {};
    cudaEvent_t side_done[lcu::kSideLanes] = {};
    bool side_dirty[lcu::kSideLanes] = {};
    cudaEvent_t fork = nullptr;
    int next_side = 0;
    lcu::WriteLog main_writes;  // what library kernels possibly still running on `main` write
    std::vector<lcu::Command> pending;
    void *stage[lcu::kStageSlots] = {};
    cudaEvent_t stage_done[lcu::kStageSlots] = {};
    bool stage_busy[lcu::kStageSlots] = {};
    int stage_next = 0;
};

namespace lcu {
// Make the context's device current for runtime-API and kernel-layer calls of this thread.
libreCudaStatus_t bind(LibreCUcontext ctx);
libreCudaStatus_t record(LibreCUstream stream, Command &&cmd);
libreCudaStatus_t commence(LibreCUstream stream);
// Makes the main lane wait for every side lane that carries async work (the caller has bound the stream's device).
libreCudaStatus_t join_sides(LibreCUstream stream);
// Starts side lane `i` at the main lane's current tail (created on first use) and marks it for the next
// join_sides; work put on `*lane` may overlap what follows on the main lane (device bound by the caller).
libreCudaStatus_t fork_side(LibreCUstream stream, int i, cudaStream_t *lane);
libreCudaStatus_t host_wait_stream(LibreCUcontext ctx, cudaStream_t s);
libreCudaStatus_t host_wait_event(LibreCUcontext ctx, cudaEvent_t e);
bool is_pageable_host(const void *p);
libreCudaStatus_t staged_h2d(LibreCUstream st, cudaStream_t lane, void *dst, const void *src, size_t bytes);
libreCudaStatus_t staged_d2h(LibreCUstream st, cudaStream_t lane, void *dst, const void *src, size_t bytes);
void free_ring(LibreCUstream st);
}  // namespace lcu

// No C++ exception may cross the C ABI (the reference lets one escape, cmdqueue.cpp:353-355): entry points that
// allocate run their body through this guard.
template <typename Fn>
inline libreCudaStatus_t lcu_guarded(Fn &&body) {
    try {
        return body();
    } catch (const std::bad_alloc &) {
        return LIBRECUDA_ERROR_OUT_OF_MEMORY;
    } catch (...) {
        return LIBRECUDA_ERROR_UNKNOWN;
    }
}

#define LCU_ENSURE_INIT() LIBRECUDA_VALIDATE(lcu::globals().initialized, LIBRECUDA_ERROR_NOT_INITIALIZED)
#define LCU_ENSURE_CTX() LIBRECUDA_VALIDATE(lcu::globals().current != nullptr, LIBRECUDA_ERROR_INVALID_CONTEXT)
