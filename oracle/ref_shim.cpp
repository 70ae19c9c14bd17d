// Host harness that runs the reference's own DtoD copy path on the CPU.
// TEST INFRASTRUCTURE ONLY -- never linked into the shipped library.
//
// It is linked with the reference's unmodified driverapi/src/memcopy.cpp, driverapi/src/librecuda_status.cpp
// and driverapi/kernels/memcpy/memcpy.cu (the latter compiled as host C++ through ref_host_cuda_shim.h),
// all compiled where they lie in the reference checkout by oracle/build_ref.sh.  This file supplies the few
// libreCu* entry points memcopy.cpp calls: module loading is faked, and libreCuLaunchKernel records the
// launch (kernel, grid, arguments) and, if asked, executes it by looping over every block and thread.
#include <cstring>
#include <string>

#include <librecuda.h>
#include <librecuda_internal.h>
#include <memcopy.h>

#include "ref_host_cuda_shim.h"

orc_dim3 blockIdx, threadIdx, gridDim, blockDim;

extern "C" void memcpyKernelHighBW(uint32_t *dst, const uint32_t *src);
extern "C" void memcpyKernelLowLatency(uint32_t *dst, const uint32_t *src, size_t n);
extern "C" void memcpyKernelTrailing(uint8_t *dst, const uint8_t *src, size_t n);

LibreCUcontext current_ctx = nullptr;

namespace {
LibreCUdevice_ g_device{};
LibreCUcontext_ g_ctx{};
LibreCUmodule_ g_module{};
LibreCUFunction_ g_funcs[3];

struct RefLaunch {
    int kernel;  // 1 HighBW, 2 LowLatency, 3 Trailing
    uint64_t grid_x, grid_y, offset, n;
    int async;
};
RefLaunch g_log[8];
int g_nlog = 0;
bool g_execute = false;
uint8_t *g_dst_base = nullptr;
uint64_t g_exec_limit = 0;  // blocks of the HighBW kernel beyond this many bytes are not executed
}  // namespace

libreCudaStatus_t libreCuDeviceGetAttribute(int *pValOut, LibreCuDeviceAttribute attribute, LibreCUdevice) {
    // pretend to be an sm_89 part so the dispatcher finds an embedded image
    *pValOut = attribute == CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR ? 8 : 9;
    return LIBRECUDA_SUCCESS;
}

libreCudaStatus_t libreCuModuleLoadData(LibreCUmodule *pModuleOut, const void *image, size_t imageSize) {
    if (image == nullptr || imageSize == 0) return LIBRECUDA_ERROR_INVALID_IMAGE;
    *pModuleOut = &g_module;
    return LIBRECUDA_SUCCESS;
}

libreCudaStatus_t libreCuModuleGetFunction(LibreCUFunction *pFunc, LibreCUmodule, const char *name) {
    static const char *names[3] = {"memcpyKernelHighBW", "memcpyKernelLowLatency", "memcpyKernelTrailing"};
    for (int i = 0; i < 3; ++i) {
        if (std::strcmp(name, names[i]) == 0) {
            g_funcs[i].name = names[i];
            *pFunc = &g_funcs[i];
            return LIBRECUDA_SUCCESS;
        }
    }
    return LIBRECUDA_ERROR_NOT_FOUND;
}

libreCudaStatus_t libreCuLaunchKernel(LibreCUFunction function, uint32_t gridDimX, uint32_t gridDimY, uint32_t gridDimZ,
                                      uint32_t blockDimX, uint32_t blockDimY, uint32_t blockDimZ, uint32_t, LibreCUstream,
                                      void **kernelParams, size_t numParams, void **, bool async) {
    const int k = (int)(function - g_funcs) + 1;
    if (k < 1 || k > 3 || g_nlog >= 8) return LIBRECUDA_ERROR_INVALID_VALUE;
    if (numParams != (k == 1 ? 2u : 3u)) return LIBRECUDA_ERROR_INVALID_VALUE;
    uint8_t *d = *static_cast<uint8_t **>(kernelParams[0]);
    const uint8_t *s = *static_cast<const uint8_t **>(kernelParams[1]);
    const size_t n = k == 1 ? 0 : *static_cast<size_t *>(kernelParams[2]);
    g_log[g_nlog++] = RefLaunch{k, gridDimX, gridDimY, (uint64_t)(d - g_dst_base), n, async ? 1 : 0};
    if (!g_execute) return LIBRECUDA_SUCCESS;
    gridDim = {gridDimX, gridDimY, gridDimZ};
    blockDim = {blockDimX, blockDimY, blockDimZ};
    for (uint32_t by = 0; by < gridDimY; ++by)
        for (uint32_t bx = 0; bx < gridDimX; ++bx) {
            blockIdx = {bx, by, 0};
            if (k == 1 && ((uint64_t)by * gridDimX + bx + 1) * 4096ull > g_exec_limit) continue;  // out of bounds
            for (uint32_t t = 0; t < blockDimX; ++t) {
                threadIdx = {t, 0, 0};
                if (k == 1) memcpyKernelHighBW(reinterpret_cast<uint32_t *>(d), reinterpret_cast<const uint32_t *>(s));
                else if (k == 2) memcpyKernelLowLatency(reinterpret_cast<uint32_t *>(d), reinterpret_cast<const uint32_t *>(s), n);
                else memcpyKernelTrailing(d, s, n);
            }
        }
    return LIBRECUDA_SUCCESS;
}

// ---- entry points used by the tests (ctypes) ----------------------------------------------------

// Runs the reference's memcpyD2D(dst, src, size).  execute = 0 only records the launch plan.
// log_out receives 6 uint64 per launch: kernel, grid_x, grid_y, offset, n, async.  Returns the number of
// launches, or a negative status.
extern "C" int ref_memcpy_d2d(void *dst, void *src, uint64_t size, int execute, int async, uint64_t *log_out) {
    g_device.ordinal = 0;
    g_ctx.device = &g_device;
    current_ctx = &g_ctx;
    libreCudaStatus_t st = loadMemcpyKernelsIfNeeded(&g_device);
    if (st != LIBRECUDA_SUCCESS) return -st;
    g_nlog = 0;
    g_execute = execute != 0;
    g_dst_base = static_cast<uint8_t *>(dst);
    g_exec_limit = size;
    LibreCUstream_ stream{};
    st = memcpyD2D(dst, src, size, &stream, async != 0);
    if (st != LIBRECUDA_SUCCESS) return -st;
    for (int i = 0; i < g_nlog; ++i) {
        log_out[6 * i + 0] = (uint64_t)g_log[i].kernel;
        log_out[6 * i + 1] = g_log[i].grid_x;
        log_out[6 * i + 2] = g_log[i].grid_y;
        log_out[6 * i + 3] = g_log[i].offset;
        log_out[6 * i + 4] = g_log[i].n;
        log_out[6 * i + 5] = (uint64_t)g_log[i].async;
    }
    return g_nlog;
}

// The reference's status table (driverapi/src/librecuda_status.cpp): name of a code, or NULL.
void internalLibreCuInitStatusNames();
const char *internalLibreCuGetStatusName(int code);
extern "C" const char *ref_status_name(int code) {
    static bool init = false;
    if (!init) {
        internalLibreCuInitStatusNames();
        init = true;
    }
    return internalLibreCuGetStatusName(code);
}
