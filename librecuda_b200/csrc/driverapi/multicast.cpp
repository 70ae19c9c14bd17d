// NVLink multicast windows on the CUDA virtual-memory API (cuMulticastCreate / cuMulticastBindMem): see
// multicast.h.  Driver entry points are resolved at first use through the runtime, so the library still
// loads on a machine without a driver.  No counterpart in the reference (single-GPU, librecuda.cpp:61).
#include "multicast.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

namespace lcu {
namespace {

struct McDriver {
    CUresult (*DeviceGet)(CUdevice *, int);
    CUresult (*DeviceGetAttribute)(int *, CUdevice_attribute, CUdevice);
    CUresult (*MemGetAllocationGranularity)(size_t *, const CUmemAllocationProp *, CUmemAllocationGranularity_flags);
    CUresult (*MemCreate)(CUmemGenericAllocationHandle *, size_t, const CUmemAllocationProp *, unsigned long long);
    CUresult (*MemRelease)(CUmemGenericAllocationHandle);
    CUresult (*MemAddressReserve)(CUdeviceptr *, size_t, size_t, CUdeviceptr, unsigned long long);
    CUresult (*MemAddressFree)(CUdeviceptr, size_t);
    CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
    CUresult (*MemUnmap)(CUdeviceptr, size_t);
    CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc *, size_t);
    CUresult (*MulticastCreate)(CUmemGenericAllocationHandle *, const CUmulticastObjectProp *);
    CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
    CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t,
                                 unsigned long long);
    CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
    CUresult (*MulticastGetGranularity)(size_t *, const CUmulticastObjectProp *, CUmulticastGranularity_flags);
};

const McDriver *mc_driver() {
    static McDriver t{};
    static int state = 0;
    if (state == 0) {
        bool ok = true;
        auto get = [&](const char *name, void **out) {
            cudaDriverEntryPointQueryResult qr;
            if (cudaGetDriverEntryPoint(name, out, cudaEnableDefault, &qr) != cudaSuccess || qr != cudaDriverEntryPointSuccess ||
                *out == nullptr) {
                (void)cudaGetLastError();
                ok = false;
            }
        };
        get("cuDeviceGet", reinterpret_cast<void **>(&t.DeviceGet));
        get("cuDeviceGetAttribute", reinterpret_cast<void **>(&t.DeviceGetAttribute));
        get("cuMemGetAllocationGranularity", reinterpret_cast<void **>(&t.MemGetAllocationGranularity));
        get("cuMemCreate", reinterpret_cast<void **>(&t.MemCreate));
        get("cuMemRelease", reinterpret_cast<void **>(&t.MemRelease));
        get("cuMemAddressReserve", reinterpret_cast<void **>(&t.MemAddressReserve));
        get("cuMemAddressFree", reinterpret_cast<void **>(&t.MemAddressFree));
        get("cuMemMap", reinterpret_cast<void **>(&t.MemMap));
        get("cuMemUnmap", reinterpret_cast<void **>(&t.MemUnmap));
        get("cuMemSetAccess", reinterpret_cast<void **>(&t.MemSetAccess));
        get("cuMulticastCreate", reinterpret_cast<void **>(&t.MulticastCreate));
        get("cuMulticastAddDevice", reinterpret_cast<void **>(&t.MulticastAddDevice));
        get("cuMulticastBindMem", reinterpret_cast<void **>(&t.MulticastBindMem));
        get("cuMulticastUnbind", reinterpret_cast<void **>(&t.MulticastUnbind));
        get("cuMulticastGetGranularity", reinterpret_cast<void **>(&t.MulticastGetGranularity));
        state = ok ? 1 : -1;
    }
    return state == 1 ? &t : nullptr;
}

// Everything a window owns, in the order it was acquired; released in reverse.
struct Owned {
    McWindow pub;
    size_t size = 0;  // mapped bytes (pub.bytes rounded up to the granularity)
    CUdevice cu_dev[16] = {};
    CUmemGenericAllocationHandle mc_handle = 0;
    bool have_mc = false;
    CUmemGenericAllocationHandle mem[16] = {};
    bool have_mem[16] = {};
    bool bound[16] = {};
    CUdeviceptr va[16] = {};
    bool reserved[16] = {}, mapped[16] = {};
    CUdeviceptr mc_va = 0;
    bool mc_reserved = false, mc_mapped = false;
};

std::vector<Owned *> &windows() {
    static std::vector<Owned *> w;
    return w;
}

void destroy(Owned *o) {
    const McDriver *d = mc_driver();
    if (d == nullptr) return;
    // nothing may still be running on the slabs: wait for every member
    int cur = -1;
    (void)cudaGetDevice(&cur);
    for (int k = 0; k < o->pub.n; ++k) {
        if (cudaSetDevice(o->pub.devs[k]) == cudaSuccess) (void)cudaDeviceSynchronize();
    }
    if (cur >= 0) (void)cudaSetDevice(cur);
    (void)cudaGetLastError();
    if (o->mc_mapped) (void)d->MemUnmap(o->mc_va, o->size);
    if (o->mc_reserved) (void)d->MemAddressFree(o->mc_va, o->size);
    for (int k = o->pub.n - 1; k >= 0; --k) {
        if (o->bound[k]) (void)d->MulticastUnbind(o->mc_handle, o->cu_dev[k], 0, o->size);
        if (o->mapped[k]) (void)d->MemUnmap(o->va[k], o->size);
        if (o->reserved[k]) (void)d->MemAddressFree(o->va[k], o->size);
        if (o->have_mem[k]) (void)d->MemRelease(o->mem[k]);
    }
    if (o->have_mc) (void)d->MemRelease(o->mc_handle);
    delete o;
}

#define MC_TRY(expr)                                                                        \
    do {                                                                                    \
        CUresult mc_r_ = (expr);                                                            \
        if (mc_r_ != CUDA_SUCCESS) {                                                        \
            std::fprintf(stderr, "[LibreCuda Debug]: multicast: %s -> CUresult %d\n", #expr, (int)mc_r_); \
            destroy(o);                                                                     \
            return (int)mc_r_;                                                              \
        }                                                                                   \
    } while (0)

int create(const int *devs, int n, size_t min_bytes, Owned **out) {
    const McDriver *d = mc_driver();
    if (d == nullptr) return -1;
    Owned *o = new Owned();
    o->pub.n = n;
    for (int k = 0; k < n; ++k) {
        o->pub.devs[k] = devs[k];
        MC_TRY(d->DeviceGet(&o->cu_dev[k], devs[k]));
        int supported = 0;
        MC_TRY(d->DeviceGetAttribute(&supported, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, o->cu_dev[k]));
        if (!supported) {
            destroy(o);
            return -1;
        }
    }
    CUmulticastObjectProp mp{};
    mp.numDevices = (unsigned)n;
    mp.size = min_bytes;
    mp.handleTypes = 0;  // not exported to other processes
    mp.flags = 0;
    size_t gran = 0;
    MC_TRY(d->MulticastGetGranularity(&gran, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED));
    for (int k = 0; k < n; ++k) {  // physical allocations have their own granularity; both are powers of two
        CUmemAllocationProp ap{};
        ap.type = CU_MEM_ALLOCATION_TYPE_PINNED;
        ap.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        ap.location.id = devs[k];
        size_t g2 = 0;
        MC_TRY(d->MemGetAllocationGranularity(&g2, &ap, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
        if (g2 > gran) gran = g2;
    }
    if (gran == 0) gran = (size_t)2 << 20;
    o->size = (min_bytes + gran - 1) / gran * gran;
    o->pub.bytes = o->size;
    mp.size = o->size;
    MC_TRY(d->MulticastCreate(&o->mc_handle, &mp));
    o->have_mc = true;
    for (int k = 0; k < n; ++k) MC_TRY(d->MulticastAddDevice(o->mc_handle, o->cu_dev[k]));  // all members before any bind
    for (int k = 0; k < n; ++k) {
        CUmemAllocationProp ap{};
        ap.type = CU_MEM_ALLOCATION_TYPE_PINNED;
        ap.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        ap.location.id = devs[k];
        MC_TRY(d->MemCreate(&o->mem[k], o->size, &ap, 0));
        o->have_mem[k] = true;
        MC_TRY(d->MulticastBindMem(o->mc_handle, 0, o->mem[k], 0, o->size, 0));
        o->bound[k] = true;
        MC_TRY(d->MemAddressReserve(&o->va[k], o->size, gran, 0, 0));
        o->reserved[k] = true;
        MC_TRY(d->MemMap(o->va[k], o->size, 0, o->mem[k], 0));
        o->mapped[k] = true;
        CUmemAccessDesc ad{};
        ad.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        ad.location.id = devs[k];
        ad.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
        MC_TRY(d->MemSetAccess(o->va[k], o->size, &ad, 1));
        o->pub.local[k] = reinterpret_cast<void *>(o->va[k]);
    }
    MC_TRY(d->MemAddressReserve(&o->mc_va, o->size, gran, 0, 0));
    o->mc_reserved = true;
    MC_TRY(d->MemMap(o->mc_va, o->size, 0, o->mc_handle, 0));
    o->mc_mapped = true;
    std::vector<CUmemAccessDesc> all((size_t)n);
    for (int k = 0; k < n; ++k) {
        all[(size_t)k].location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        all[(size_t)k].location.id = devs[k];
        all[(size_t)k].flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    }
    MC_TRY(d->MemSetAccess(o->mc_va, o->size, all.data(), (size_t)n));
    o->pub.mc = reinterpret_cast<void *>(o->mc_va);
    *out = o;
    return 0;
}

}  // namespace

int mc_window_acquire(const int *devs, int n, size_t min_bytes, const McWindow **out) {
    if (devs == nullptr || out == nullptr || n < 2 || n > 16 || min_bytes == 0) return 1;
    static bool exit_hook = false;
    auto &ws = windows();
    for (size_t i = 0; i < ws.size(); ++i) {
        Owned *o = ws[i];
        if (o->pub.n != n || std::memcmp(o->pub.devs, devs, sizeof(int) * (size_t)n) != 0) continue;
        if (o->pub.bytes >= min_bytes) {
            *out = &o->pub;
            return 0;
        }
        ws.erase(ws.begin() + (long)i);  // too small: replace it
        destroy(o);
        break;
    }
    Owned *o = nullptr;
    const int rc = create(devs, n, min_bytes, &o);
    if (rc != 0) return rc;
    if (!exit_hook) {  // registered after the CUDA runtime's own exit handlers, so it runs before them
        exit_hook = true;
        std::atexit(mc_release_all);
    }
    ws.push_back(o);
    *out = &o->pub;
    return 0;
}

void mc_release_all() {
    auto &ws = windows();
    while (!ws.empty()) {
        Owned *o = ws.back();
        ws.pop_back();
        destroy(o);
    }
}

}  // namespace lcu
