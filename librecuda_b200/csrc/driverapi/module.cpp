// Modules, functions and kernel launches of the libreCu* API.
//
// The reference parses the cubin ELF itself and builds a QMD launch descriptor per launch
// (driverapi/src/librecuda.cpp:888-1460, driverapi/src/cmdqueue.cpp:459-729).  Here the CUDA driver loads
// the image and launches; this file keeps the reference's caller-visible rules: the image is copied, the
// function list can be enumerated, numParams must match the kernel's parameter list, argument values are
// captured when libreCuLaunchKernel returns, and launches are recorded into the stream.
#include <cstring>

#include "internal.h"

using namespace lcu;

static libreCudaStatus_t describe(LibreCUFunction f) {
    const DriverTable *drv = driver();
    const char *name = nullptr;
    LCU_CU(drv->FuncGetName(&name, f->fn));
    f->name = name ? name : "";
    f->param_offset.clear();
    f->param_size.clear();
    f->param_bytes = 0;
    for (size_t i = 0;; ++i) {
        size_t off = 0, size = 0;
        if (drv->FuncGetParamInfo(f->fn, i, &off, &size) != CUDA_SUCCESS) break;  // past the last parameter
        f->param_offset.push_back(off);
        f->param_size.push_back(size);
        if (off + size > f->param_bytes) f->param_bytes = off + size;
    }
    // With lazy module loading the code of a function is brought onto the device at its first launch (about
    // 10 us); asking for an attribute loads it now, so that the cost is paid in libreCuModuleLoadData -- where
    // the reference uploads its image too (librecuda.cpp:1376) -- and not inside the first Commence.
    int regs = 0;
    LCU_CU(drv->FuncGetAttribute(&regs, /*CU_FUNC_ATTRIBUTE_NUM_REGS*/ 4, f->fn));
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t libreCuModuleLoadData(LibreCUmodule *pModuleOut, const void *image, size_t imageSize) {
    return lcu_guarded([&]() -> libreCudaStatus_t {
        LIBRECUDA_VALIDATE(pModuleOut != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        LIBRECUDA_VALIDATE(image != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        LIBRECUDA_VALIDATE(imageSize >= 4, LIBRECUDA_ERROR_INVALID_IMAGE);
        LCU_ENSURE_CTX();
        const DriverTable *drv = driver();
        LIBRECUDA_VALIDATE(drv != nullptr, LIBRECUDA_ERROR_NOT_INITIALIZED);
        LibreCUcontext ctx = globals().current;
        LIBRECUDA_ERR_PROPAGATE(bind(ctx));
        auto mod = std::make_unique<LibreCUmodule_>();
        mod->ctx = ctx;
        CUresult res = drv->ModuleLoadData(&mod->mod, image);
        if (res != CUDA_SUCCESS) {
            LIBRECUDA_DEBUG("cuModuleLoadData failed: CUresult " << (int)res);
            LIBRECUDA_FAIL(res == CUDA_ERROR_OUT_OF_MEMORY ? LIBRECUDA_ERROR_OUT_OF_MEMORY : LIBRECUDA_ERROR_INVALID_IMAGE);
        }
        unsigned int count = 0;
        LCU_CU(drv->ModuleGetFunctionCount(&count, mod->mod));
        std::vector<CUfunction> fns(count);
        if (count) LCU_CU(drv->ModuleEnumerateFunctions(fns.data(), count, mod->mod));
        for (CUfunction fn : fns) {
            auto f = std::make_unique<LibreCUFunction_>();
            f->module = mod.get();
            f->fn = fn;
            LIBRECUDA_ERR_PROPAGATE(describe(f.get()));
            mod->functions.push_back(std::move(f));
        }
        *pModuleOut = mod.release();
        LIBRECUDA_SUCCEED();
    });
}

libreCudaStatus_t libreCuModuleUnload(LibreCUmodule module) {
    LIBRECUDA_VALIDATE(module != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    const DriverTable *drv = driver();
    LIBRECUDA_VALIDATE(drv != nullptr, LIBRECUDA_ERROR_NOT_INITIALIZED);
    LIBRECUDA_ERR_PROPAGATE(bind(module->ctx));
    LCU_CU(drv->ModuleUnload(module->mod));
    delete module;
    LibreCUcontext cur = globals().current;
    if (cur != nullptr) LIBRECUDA_ERR_PROPAGATE(bind(cur));
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t libreCuModuleGetFunctionCount(uint32_t *count, LibreCUmodule mod) {
    LIBRECUDA_VALIDATE(count != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(mod != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    *count = (uint32_t)mod->functions.size();
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t libreCuModuleEnumerateFunctions(LibreCUFunction *functionsOut, uint32_t numFunctions, LibreCUmodule mod) {
    LIBRECUDA_VALIDATE(functionsOut != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(mod != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(numFunctions >= mod->functions.size(), LIBRECUDA_ERROR_INVALID_VALUE);
    for (size_t i = 0; i < mod->functions.size(); ++i) functionsOut[i] = mod->functions[i].get();
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t libreCuFuncGetName(const char **pNameOut, LibreCUFunction func) {
    LIBRECUDA_VALIDATE(pNameOut != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(func != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    *pNameOut = func->name.c_str();
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t libreCuModuleGetFunction(LibreCUFunction *pFunc, LibreCUmodule module, const char *name) {
    LIBRECUDA_VALIDATE(pFunc != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(module != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(name != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    for (auto &f : module->functions) {
        if (f->name == name) {
            *pFunc = f.get();
            LIBRECUDA_SUCCEED();
        }
    }
    LIBRECUDA_FAIL(LIBRECUDA_ERROR_NOT_FOUND);
}

libreCudaStatus_t libreCuFuncSetAttribute(LibreCUFunction function, LibreCuFunctionAttribute attribute, int value) {
    LIBRECUDA_VALIDATE(function != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
    LIBRECUDA_VALIDATE(attribute == CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, LIBRECUDA_ERROR_INVALID_VALUE);
    LibreCUcontext ctx = function->module->ctx;
    LIBRECUDA_VALIDATE(value >= 0 && value <= ctx->device->smem_optin, LIBRECUDA_ERROR_INVALID_VALUE);  // reference librecuda.cpp:1596-1601
    LIBRECUDA_ERR_PROPAGATE(bind(ctx));
    LCU_CU(driver()->FuncSetAttribute(function->fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, value));
    function->dyn_smem_attr = value;
    LibreCUcontext cur = globals().current;
    if (cur != nullptr && cur != ctx) LIBRECUDA_ERR_PROPAGATE(bind(cur));
    LIBRECUDA_SUCCEED();
}

libreCudaStatus_t libreCuLaunchKernel(LibreCUFunction function, uint32_t gridDimX, uint32_t gridDimY, uint32_t gridDimZ,
                                      uint32_t blockDimX, uint32_t blockDimY, uint32_t blockDimZ, uint32_t sharedMemBytes,
                                      LibreCUstream stream, void **kernelParams, size_t numParams, void **extra, bool async) {
    return lcu_guarded([&]() -> libreCudaStatus_t {
        (void)extra;
        LIBRECUDA_VALIDATE(function != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        LIBRECUDA_VALIDATE(stream != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        LCU_ENSURE_CTX();
        LIBRECUDA_VALIDATE(numParams == function->param_size.size(), LIBRECUDA_ERROR_INVALID_VALUE);  // reference cmdqueue.cpp:467
        LIBRECUDA_VALIDATE(numParams == 0 || kernelParams != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
        const LibreCUdevice dev = stream->ctx->device;
        // launch limits of the device (the reference hard-codes them, cmdqueue.cpp:592-598)
        LIBRECUDA_VALIDATE(blockDimX >= 1 && blockDimX <= (uint32_t)dev->max_block_x, LIBRECUDA_ERROR_LAUNCH_OUT_OF_RESOURCES);
        LIBRECUDA_VALIDATE(blockDimY >= 1 && blockDimY <= (uint32_t)dev->max_block_y, LIBRECUDA_ERROR_LAUNCH_OUT_OF_RESOURCES);
        LIBRECUDA_VALIDATE(blockDimZ >= 1 && blockDimZ <= (uint32_t)dev->max_block_z, LIBRECUDA_ERROR_LAUNCH_OUT_OF_RESOURCES);
        LIBRECUDA_VALIDATE((uint64_t)blockDimX * blockDimY * blockDimZ <= (uint64_t)dev->max_threads, LIBRECUDA_ERROR_LAUNCH_OUT_OF_RESOURCES);
        LIBRECUDA_VALIDATE(gridDimX >= 1 && gridDimX <= (uint32_t)dev->max_grid_x, LIBRECUDA_ERROR_LAUNCH_OUT_OF_RESOURCES);
        LIBRECUDA_VALIDATE(gridDimY >= 1 && gridDimY <= (uint32_t)dev->max_grid_y, LIBRECUDA_ERROR_LAUNCH_OUT_OF_RESOURCES);
        LIBRECUDA_VALIDATE(gridDimZ >= 1 && gridDimZ <= (uint32_t)dev->max_grid_z, LIBRECUDA_ERROR_LAUNCH_OUT_OF_RESOURCES);
        Command c;
        c.kind = Command::Launch;
        c.async = async;
        c.fn = function;
        c.grid[0] = gridDimX; c.grid[1] = gridDimY; c.grid[2] = gridDimZ;
        c.block[0] = blockDimX; c.block[1] = blockDimY; c.block[2] = blockDimZ;
        // shared memory = max(value set through libreCuFuncSetAttribute, sharedMemBytes), reference cmdqueue.cpp:585
        c.smem = sharedMemBytes > (uint32_t)function->dyn_smem_attr ? sharedMemBytes : (uint32_t)function->dyn_smem_attr;
        LIBRECUDA_VALIDATE(c.smem <= (uint32_t)dev->smem_optin, LIBRECUDA_ERROR_LAUNCH_OUT_OF_RESOURCES);
        c.params.assign(function->param_bytes, 0);
        for (size_t i = 0; i < numParams; ++i) {
            LIBRECUDA_VALIDATE(kernelParams[i] != nullptr, LIBRECUDA_ERROR_INVALID_VALUE);
            std::memcpy(c.params.data() + function->param_offset[i], kernelParams[i], function->param_size[i]);
        }
        return record(stream, std::move(c));
    });
}
