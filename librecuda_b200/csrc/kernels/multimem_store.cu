// Store kernel for NVLink multicast (NVSwitch replication): reads a span of this GPU's memory once and
// writes it with multimem.st to a multicast address, so that every byte leaves the GPU's port once and the
// switch delivers a copy into the memory of every GPU bound to the multicast object.  This is what the
// library's multicast broadcast is built from; the reference is single-GPU (driverapi/src/librecuda.cpp:61)
// and has no counterpart.  Only multimem stores are issued on the multicast address -- no loads, no bulk
// (TMA) copies.
#include "common.cuh"
#include "lcb200_kernels.h"

namespace lcb {

// Weak 16-byte stores: relaxed.sys stores, 1 ... 8 vectors per thread, 128 ... 512 threads per CTA and 16 ... 1184
// CTAs all measured the same 543-552 GB/s, the fabric's rate for multicast writes issued by one GPU.
__device__ __forceinline__ void multimem_store(uint4 *mc, uint4 v) {
    asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1,%2,%3,%4};"
                 :: "l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// mc_dst: 16-byte aligned multicast address; src: 16-byte aligned ordinary (unicast) address; nvec 16-byte vectors.
template <int U>
__global__ void __launch_bounds__(512) multicast_store_kernel(uint4 *__restrict__ mc_dst, const uint4 *__restrict__ src,
                                                              size_t nvec) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t tile = (size_t)U * blockDim.x;
    const size_t ntiles = (nvec + tile - 1) / tile;
    for (size_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
        const size_t base = t * tile + threadIdx.x;
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const size_t j = base + (size_t)u * blockDim.x;
            v[u] = j < nvec ? ld_stream<2>(src + j) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const size_t j = base + (size_t)u * blockDim.x;
            if (j < nvec) multimem_store(mc_dst + j, v[u]);
        }
    }
    // the stores are weak; the kernel boundary makes them visible to work ordered after this kernel on any GPU
    __threadfence_system();
}

}  // namespace lcb

extern "C" int lcb_multicast_store(void *mc_dst, const void *src, size_t bytes, int ctas, lcbStream stream) {
    using namespace lcb;
    if (bytes == 0) return 0;
    if (mc_dst == nullptr || src == nullptr || ctas < 0) return 1;
    if ((reinterpret_cast<uintptr_t>(mc_dst) | reinterpret_cast<uintptr_t>(src) | bytes) & 15) return 1;
    const size_t nvec = bytes / 16;
    const int threads = 512;
    constexpr int U = 4;
    size_t need = (nvec + (size_t)U * threads - 1) / ((size_t)U * threads);
    const size_t cap = ctas > 0 ? (size_t)ctas : ((size_t)1 << 30);
    const int grid = (int)(need < cap ? need : cap);
    return launch_kernel(multicast_store_kernel<U>, grid, threads, 0, static_cast<cudaStream_t>(stream),
                         static_cast<uint4 *>(mc_dst), static_cast<const uint4 *>(src), nvec);
}
