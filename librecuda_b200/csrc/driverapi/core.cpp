// Status symbols, initialisation, devices, contexts and memory of the libreCu* API, on top of the CUDA
// runtime in each device's primary context.  Replaces the raw RM/UVM ioctl front end of the reference
// (driverapi/src/librecuda.cpp:80-871) while keeping its observable behaviour.
#include <algorithm>
#include <cstring>

#include "internal.h"
#include "multicast.h"

// ---- status variables (data symbols, reference driverapi/src/librecuda_status.cpp:7-11) -----------------
extern "C" {
libreCudaStatus_t LIBRECUDA_SUCCESS = 0;
libreCudaStatus_t LIBRECUDA_ERROR_INVALID_VALUE = 1;
libreCudaStatus_t LIBRECUDA_ERROR_OUT_OF_MEMORY = 2;
libreCudaStatus_t LIBRECUDA_ERROR_NOT_INITIALIZED = 3;
libreCudaStatus_t LIBRECUDA_ERROR_INVALID_DEVICE = 101;
libreCudaStatus_t LIBRECUDA_ERROR_INVALID_IMAGE = 200;
libreCudaStatus_t LIBRECUDA_ERROR_INVALID_CONTEXT = 201;
libreCudaStatus_t LIBRECUDA_ERROR_NOT_FOUND = 500;
libreCudaStatus_t LIBRECUDA_ERROR_NOT_READY = 600;
libreCudaStatus_t LIBRECUDA_ERROR_LAUNCH_OUT_OF_RESOURCES = 701;
libreCudaStatus_t LIBRECUDA_ERROR_COMPAT_NOT_SUPPORTED_ON_DEVICE = 804;
libreCudaStatus_t LIBRECUDA_ERROR_UNKNOWN = 999;
}

namespace lcu {

const char *status_name(libreCudaStatus_t code) {
    switch (code) {
        case 0: return "LIBRECUDA_SUCCESS";
        case 1: return "LIBRECUDA_ERROR_INVALID_VALUE";
        case 2: return "LIBRECUDA_ERROR_OUT_OF_MEMORY";
        case 3: return "LIBRECUDA_ERROR_NOT_INITIALIZED";
        case 101: return "LIBRECUDA_ERROR_INVALID_DEVICE";
        case 200: return "LIBRECUDA_ERROR_INVALID_IMAGE";
        case 201: return "LIBRECUDA_ERROR_INVALID_CONTEXT";
        case 500: return "LIBRECUDA_ERROR_NOT_FOUND";
        case 600: return "LIBRECUDA_ERROR_NOT_READY";
        case 701: return "LIBRECUDA_ERROR_LAUNCH_OUT_OF_RESOURCES";
        case 804: return "LIBRECUDA_ERROR_COMPAT_NOT_SUPPORTED_ON_DEVICE";
        case 999: return "LIBRECUDA_ERROR_UNKNOWN";
        default: return nullptr;
    }
}

libreCudaStatus_t from_cuda(cudaError_t err) {
    switch (err) {
        case cudaSuccess: return LIBRECUDA_SUCCESS;
        case cudaErrorInvalidValue: return LIBRECUDA_ERROR_INVALID_VALUE;
        case cudaErrorMemoryAllocation: return LIBRECUDA_ERROR_OUT_OF_MEMORY;
        case cudaErrorInitializationError: return LIBRECUDA_ERROR_NOT_INITIALIZED;
        case cudaErrorInvalidDevice: return LIBRECUDA_ERROR_INVALID_DEVICE;
        case cudaErrorInvalidKernelImage:
        case cudaErrorInvalidPtx:
        case cudaErrorNoKernelImageForDevice: return LIBRECUDA_ERROR_INVALID_IMAGE;
        case cudaErrorDeviceUninitialized:
        case cudaErrorContextIsDestroyed: return LIBRECUDA_ERROR_INVALID_CONTEXT;
        case cudaErrorSymbolNotFound: return LIBRECUDA_ERROR_NOT_FOUND;
        case cudaErrorNotReady: return LIBRECUDA_ERROR_NOT_READY;
        case cudaErrorLaunchOutOfResources:
        case cudaErrorInvalidConfiguration: return LIBRECUDA_ERROR_LAUNCH_OUT_OF_RESOURCES;
        case cudaErrorNoDevice:
        case cudaErrorInsufficientDriver:
        case cudaErrorNotSupported: return LIBRECUDA_ERROR_COMPAT_NOT_SUPPORTED_ON_DEVICE;
        default: return LIBRECUDA_ERROR_UNKNOWN;
    }
}

libreCudaStatus_t from_cu(CUresult res) { return from_cuda(static_cast<cudaError_t>(res)); }

const DriverTable *driver() {
    static DriverTable table{};
    static int state = 0;  // 0 untried, 1 ok, -1 unavailable
    if (state == 0) {
        bool ok = true;
        auto get = [&](const char *name, void **out) {
            cudaDriverEntryPointQueryResult qr;
            if (cudaGetDriverEntryPoint(name, out, cudaEnableDefault, &qr) != cudaSuccess ||
                qr != cudaDriverEntryPointSuccess || *out == nullptr) {
                (void)cudaGetLastError();
                LIBRECUDA_DEBUG("CUDA driver entry point unavailable: " << name);
                ok = false;
            }
        };
        get("cuModuleLoadData", reinterpret_cast<void **>(&table.ModuleLoadData));
        get("cuModuleUnload", reinterpret_cast<void **>(&table.ModuleUnload));
        get("cuModuleGetFunction", reinterpret_cast<void **>(&table.ModuleGetFunction));
        get("cuModuleGetFunctionCount", reinterpret_cast<void **>(&table.ModuleGetFunctionCount));
        get("cuModuleEnumerateFunctions", reinterpret_cast<void **>(&table.ModuleEnumerateFunctions));
        get("cuFuncGetName", reinterpret_cast<void **>(&table.FuncGetName));
        get("cuFuncGetParamInfo", reinterpret_cast<void **>(&table.FuncGetParamInfo));
        get("cuFuncSetAttribute", reinterpret_cast<void **>(&table.FuncSetAttribute));
        get("cuFuncGetAttribute", reinterpret_cast<void **>(&table.FuncGetAttribute));
        get("cuLaunchKernel", reinterpret_cast<void **>(&table.LaunchKernel));
        state = ok ? 1 : -1;
    }
    return state == 1 ? &table : nullptr;
}

Globals &globals() {
    static Globals g;
    return g;
}

libreCudaStatus_t bind(LibreCUcontext ctx) {
    LIBRECUDA_VALIDATE(ctx != nullptr, LIBRECUDA_ERROR_INVALID_CONTEXT);
    LCU_CUDA(cudaSetDevice(ctx->device->ordinal));
    LIBRECUDA_SUCCEED();
}

PtrClass classify(const void *p) {
    auto &allocs = globals().allocations;
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    auto it = allocs.upper_bound(a);
    if (it != allocs.begin()) {
        --it;
        if (a < it->first + it->second.size) return PtrClass::Device;
    }
    cudaPointerAttributes attr{};
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return PtrClass::Host;
    }
    return (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) ? PtrClass::Device : PtrClass::Host;
}

int owner_device(const void *p) {
    auto &allocs = globals().allocations;
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    auto it = allocs.upper_bound(a);
    if (it != allocs.begin()) {
        --it;
        if (a < it->first + it->second.size) return it->second.mapped ? -1 : it->second.device;
    }
    cudaPointerAttributes attr{};
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return -1;
    }
    return attr.type == cudaMemoryTypeDevice ? attr.device : -1;
}

}  // namespace lcu

using namespace lcu;

// ---- init / devices ---------------------------------------------------------------------------------------

libreCudaStatus_t libreCuInit(int flags) {
    return lcu_guarded([&]() -> libreCudaStatus_t {
        (void)flags;
        Globals &g = globals();
        if (g.initialized) LIBRECUDA_SUCCEED();
        int count = 0;
        cudaError_t err = cudaGetDeviceCount(&count);
        if (err != cudaSuccess || count <= 0) {
            (void)cudaGetLastError();
            LIBRECUDA_DEBUG("no usable CUDA device: " << (err != cudaSuccess ? cudaGetErrorName(err) : "device count 0"));
            LIBRECUDA_FAIL(LIBRECUDA_ERROR_COMPAT_NOT_SUPPORTED_ON_DEVICE);
        }
        LIBRECUDA_VALIDATE(driver() != nullptr, LIBRECUDA_ERROR_COMPAT_NOT_SUPPORTED_ON_DEVICE);
        for (int i = 0; i < count; ++i) {
            auto d = std::make_unique<LibreCUdevice_>();
            d->ordinal = i;
            cudaDeviceProp prop{};
            LCU_CUDA(cudaGetDeviceProperties(&prop, i));
            d->name = prop.name;
            d->cc_major = prop.major;
            d->cc_minor = prop.minor;
            d->smem_per_block = (int)prop.sharedMemPerBlock;
            d->smem_optin = (int)prop.sharedMemPerBlockOptin;
            d->max_block_x = prop.maxThreadsDim[0];
            d->max_block_y = prop.maxThreadsDim[1];
            d->max_block_z = prop.maxThreadsDim[2];
            d->max_threads = prop.maxThreadsPerBlock;
            d->max_grid_x = prop.maxGridSize[0];
            d->max_grid_y = prop.maxGridSize[1];
            d->max_grid_z = prop.maxGridSize[2];
            g.devices.push_back(std::move(d));
        }
        g.initialized = true;
        LIBRECUDA_SUCCEED();
    });
}

libreCudaStatus_t libreCuDeviceGetCount(int *pDeviceCount) {
    LIBRECUDA_VALIDATE(pDeviceCount != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LCU_ENSURE_INIT();
    *pDeviceCount = (int)globals().devices.size();
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t libreCuDeviceGet(LibreCUdevice *device, int deviceOrdinal) {
    LIBRECUDA_VALIDATE(device != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LCU_ENSURE_INIT();
    LIBRECUDA_VALIDATE(deviceOrdinal >= 0 && deviceOrdinal < (int)globals().devices.size(), LIBRECUDA_ERROR_INVALID_DEVICE);
    *device = globals().devices[deviceOrdinal].get();
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t libreCuGetErrorString(libreCudaStatus_t status, const char **pStatusName) {
    LIBRECUDA_VALIDATE(pStatusName != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    *pStatusName = status_name(status);
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t libreCuDeviceGetName(char *pDeviceName, int length, LibreCUdevice device) {
    LIBRECUDA_VALIDATE(pDeviceName != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(device != nullptr, LIBRECUDA_ERROR_INVALID_DEVICE);
    LIBRECUDA_VALIDATE(length > 0, LIBRECUDA_ERROR_INVALID_VALUE);
    LCU_ENSURE_CTX();
    std::strncpy(pDeviceName, device->name.c_str(), (size_t)length);
    pDeviceName[length - 1] = '\0';
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t libreCuDeviceGetAttribute(int *pValOut, LibreCuDeviceAttribute attribute, LibreCUdevice device) {
    LIBRECUDA_VALIDATE(pValOut != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(device != nullptr, LIBRECUDA_ERROR_INVALID_DEVICE);
    switch (attribute) {
        case CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR: *pValOut = device->cc_major; break;
        case CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR: *pValOut = device->cc_minor; break;
        case CU_DEVICE_ATTRIBUTE_MAX_SHARED_MEMORY_PER_BLOCK: *pValOut = device->smem_per_block; break;
        case CU_DEVICE_ATTRIBUTE_MAX_SHARED_MEMORY_PER_BLOCK_OPTIN: *pValOut = device->smem_optin; break;
        default: LIBRECUDA_FAIL(LIBRECUDA_ERROR_INVALID_VALUE);
    }
    LIBRECUDA_SUCCEED();
}

// ---- contexts ----------------------------------------------------------------------------------------------

libreCudaStatus_t libreCuCtxCreate_v2(LibreCUcontext *pCtx, int flags, LibreCUdevice device) {
    return lcu_guarded([&]() -> libreCudaStatus_t {
        LIBRECUDA_VALIDATE(pCtx != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        LIBRECUDA_VALIDATE(device != nullptr, LIBRECUDA_ERROR_INVALID_DEVICE);
        LCU_ENSURE_INIT();
        auto ctx = std::make_unique<LibreCUcontext_>();
        ctx->device = device;
        ctx->flags = flags;
        ctx->peers.insert(device->ordinal);
        LCU_CUDA(cudaSetDevice(device->ordinal));
        LCU_CUDA(cudaFree(nullptr));  // forces creation of the primary context
        LibreCUcontext_::Epoch first;
        LCU_CUDA(cudaEventCreate(&first.ev));
        LCU_CUDA(cudaEventRecord(first.ev, nullptr));
        first.host_ms = steady_ms();
        ctx->epochs.push_back(first);
        ctx->epoch_base_ns.push_back(0);
        LCU_LCB(lcb_preload());  // the reference loads its copy kernels here as well (librecuda.cpp:622)
        globals().current = ctx.get();  // reference: librecuda.cpp:619
        *pCtx = ctx.release();
        LIBRECUDA_SUCCEED();
    });
}

libreCudaStatus_t libreCuCtxDestroy(LibreCUcontext ctx) {
    LIBRECUDA_VALIDATE(ctx != nullptr, LIBRECUDA_ERROR_INVALID_CONTEXT);
    if (globals().current == ctx) globals().current = nullptr;
    mc_release_all();  // multicast slabs bound on this GPU go before its context does (re-created on demand)
    if (cudaSetDevice(ctx->device->ordinal) == cudaSuccess) {
        (void)cudaDeviceSynchronize();
        for (auto &ep : ctx->epochs)
            if (ep.ev) (void)cudaEventDestroy(ep.ev);
    }
    (void)cudaGetLastError();
    delete ctx;
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t libreCuCtxSetCurrent(LibreCUcontext ctx) {
    LIBRECUDA_VALIDATE(ctx != nullptr, LIBRECUDA_ERROR_INVALID_CONTEXT);
    LIBRECUDA_ERR_PROPAGATE(bind(ctx));
    globals().current = ctx;
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t libreCuCtxGetCurrent(LibreCUcontext *pCtxOut) {
    LIBRECUDA_VALIDATE(pCtxOut != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    *pCtxOut = globals().current;
    LIBRECUDA_SUCCEED();
}

// ---- memory ---------------------------------------------------------------------------------------------------

libreCudaStatus_t libreCuMemAlloc(void **pDevicePointer, size_t bytesize, bool mapToCpu) {
    return lcu_guarded([&]() -> libreCudaStatus_t {
        LIBRECUDA_VALIDATE(pDevicePointer != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        LIBRECUDA_VALIDATE(bytesize != 0, LIBRECUDA_ERROR_INVALID_VALUE);
        LCU_ENSURE_CTX();
        Globals &g = globals();
        LIBRECUDA_ERR_PROPAGATE(bind(g.current));
        // the reference rounds to 4 KiB pages (2 MiB above 16 MiB) and returns page-aligned addresses
        // (librecuda.cpp:694-695,743); keep the 4 KiB alignment guarantee
        constexpr size_t kPage = 4096;
        const size_t rounded = (bytesize + kPage - 1) / kPage * kPage;
        void *raw = nullptr;
        auto alloc = [&](size_t n) -> cudaError_t {
            return mapToCpu ? cudaMallocManaged(&raw, n, cudaMemAttachGlobal) : cudaMalloc(&raw, n);
        };
        LCU_CUDA(alloc(rounded));
        void *aligned = raw;
        if (reinterpret_cast<uintptr_t>(raw) % kPage) {
            LCU_CUDA(cudaFree(raw));
            LCU_CUDA(alloc(rounded + kPage));
            aligned = reinterpret_cast<void *>((reinterpret_cast<uintptr_t>(raw) + kPage - 1) / kPage * kPage);
        }
        g.allocations[reinterpret_cast<uintptr_t>(aligned)] = Allocation{raw, rounded, g.current->device->ordinal, mapToCpu, false};
        *pDevicePointer = aligned;
        LIBRECUDA_SUCCEED();
    });
}

libreCudaStatus_t libreCuMemFree(void *devicePointer) {
    LIBRECUDA_VALIDATE(devicePointer != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LCU_ENSURE_CTX();
    Globals &g = globals();
    auto it = g.allocations.find(reinterpret_cast<uintptr_t>(devicePointer));
    LIBRECUDA_VALIDATE(it != g.allocations.end(), LIBRECUDA_ERROR_INVALID_VALUE);  // must be an allocation base
    LIBRECUDA_VALIDATE(!it->second.ipc, LIBRECUDA_ERROR_INVALID_VALUE);           // use libreCuIpcCloseMemHandle
    LCU_CUDA(cudaSetDevice(it->second.device));
    void *raw = it->second.raw;
    g.allocations.erase(it);
    LCU_CUDA(cudaFree(raw));
    LIBRECUDA_ERR_PROPAGATE(bind(g.current));
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t libreCuMemAllocHost(void **pHostPointer, size_t bytesize) {
    LIBRECUDA_VALIDATE(pHostPointer != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(bytesize != 0, LIBRECUDA_ERROR_INVALID_VALUE);
    LCU_ENSURE_CTX();
    LIBRECUDA_ERR_PROPAGATE(bind(globals().current));
    LCU_CUDA(cudaHostAlloc(pHostPointer, bytesize, cudaHostAllocPortable));
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t libreCuMemFreeHost(void *hostPointer) {
    LIBRECUDA_VALIDATE(hostPointer != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LCU_ENSURE_CTX();
    LCU_CUDA(cudaFreeHost(hostPointer));
    LIBRECUDA_SUCCEED();
}
