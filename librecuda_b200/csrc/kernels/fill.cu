// Write-only kernels for sm_100a: memset (D8/D16/D32), index fill, and the y = a*x + b fixture kernel.
//
// The reference has no memset (driverapi/include/librecuda.h:37-114); its fill kernels are the test
// fixtures tests/indexing/write_float.cu:1-4 (one scalar store per thread over a 1-D grid) and
// tests/write_float/write_float.cu:1-7.  Here:
//  * memset_vec_kernel   16-byte streaming stores, U per lane per tile; one short CTA per tile by default.
//  * memset_bulk_kernel  fills ONE shared-memory tile with the pattern, then one thread per warp replays it
//                        with bulk stores (cp.async.bulk shared->global); the SM issues one instruction
//                        per `chunk` bytes written.
//  * index_fill_kernel   out[i] = float(i), four consecutive elements per 16-byte store.
//  * axpb_kernel         y = a*x + b with separate multiply and add roundings.
#include "common.cuh"
#include "lcb200_kernels.h"

namespace lcb {

struct FillEdges {
    uint8_t *dst;
    int head;          // bytes before the 16-byte aligned body
    int tail;          // bytes after it
    size_t tail_off;
    uint32_t pattern;  // 32-bit replicated pattern, valid at any offset that is a multiple of elem size
    int elem;          // element bytes: 1, 2 or 4
};

// byte k of the destination gets byte (k mod elem) of the pattern; head offsets are multiples of elem
__device__ __forceinline__ void fill_edges(const FillEdges &e, int t) {
    if (t < e.head) e.dst[t] = (uint8_t)(e.pattern >> (8 * (t & (e.elem - 1))));
    int u = t - 32;
    if (u >= 0 && u < e.tail) e.dst[e.tail_off + u] = (uint8_t)(e.pattern >> (8 * (u & (e.elem - 1))));
}

template <int U>
__global__ void __launch_bounds__(512) memset_vec_kernel(uint4 *__restrict__ dstv, size_t nvec, FillEdges e) {
    pdl_launch_dependents();
    pdl_wait();
    if (blockIdx.x == 0) fill_edges(e, threadIdx.x);
    const uint4 p = make_uint4(e.pattern, e.pattern, e.pattern, e.pattern);
    const size_t tile = (size_t)U * blockDim.x;
    const size_t ntiles = (nvec + tile - 1) / tile;
    for (size_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
        const size_t base = t * tile + threadIdx.x;
        if ((t + 1) * tile <= nvec) {
#pragma unroll
            for (int u = 0; u < U; ++u) st_stream<0>(dstv + base + (size_t)u * blockDim.x, p);
        } else {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const size_t j = base + (size_t)u * blockDim.x;
                if (j < nvec) st_stream<0>(dstv + j, p);
            }
        }
    }
}

// blockDim = 32 * issuers.  All threads fill the tile; lane 0 of every warp then issues bulk stores of the
// same tile for its share of the chunks (several issuers per SM keep the store queue full).  The tile is
// never rewritten, so no store has to be waited for until the end.
template <bool HINT>
__global__ void __launch_bounds__(256) memset_bulk_kernel(uint8_t *__restrict__ body_dst, size_t body, uint32_t chunk,
                                                          FillEdges e) {
    extern __shared__ __align__(128) uint8_t smem[];
    pdl_launch_dependents();
    const size_t nchunks = (body + chunk - 1) / chunk;
    const size_t issuers = blockDim.x >> 5;
    const bool has_chunks = (size_t)blockIdx.x * issuers < nchunks;
    if (has_chunks) {  // the tile is built while the previous kernel on the stream is still draining
        const uint4 p = make_uint4(e.pattern, e.pattern, e.pattern, e.pattern);
        uint4 *tile = reinterpret_cast<uint4 *>(smem);
        for (uint32_t i = threadIdx.x; i < chunk / 16; i += blockDim.x) tile[i] = p;
        fence_generic_to_async_smem();
    }
    __syncthreads();
    pdl_wait();
    if (blockIdx.x == 0) fill_edges(e, threadIdx.x);
    if (!has_chunks) return;
    if ((threadIdx.x & 31) != 0) return;
    uint64_t pol = 0;
    if (HINT) pol = policy_evict_first();
    const uint32_t tile_addr = smem_addr(smem);
    const size_t stride = (size_t)gridDim.x * issuers;
    for (size_t c = (size_t)blockIdx.x * issuers + (threadIdx.x >> 5); c < nchunks; c += stride) {
        const size_t off = c * (size_t)chunk;
        const size_t rem = body - off;
        bulk_s2g<HINT>(body_dst + off, tile_addr, (uint32_t)(rem < chunk ? rem : chunk), pol);
        bulk_commit();
    }
    bulk_wait_all();
}

// dst4 is the 16-byte aligned body; element index of dst4[0].x is first.
__global__ void __launch_bounds__(512) index_fill_kernel(float *__restrict__ dst, size_t count, int head,
                                                         size_t nvec) {
    // head elements (until dst+head is 16-byte aligned) and tail elements go out as scalars
    float4 *dst4 = reinterpret_cast<float4 *>(dst + head);
    pdl_launch_dependents();
    pdl_wait();
    if (blockIdx.x == 0) {
        const int t = threadIdx.x;
        if (t < head) dst[t] = (float)t;
        const size_t tail_first = (size_t)head + nvec * 4;
        const int u = t - 32;
        if (u >= 0 && tail_first + u < count) dst[tail_first + u] = __ull2float_rn(tail_first + u);
    }
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x; j < nvec; j += stride) {
        const unsigned long long i0 = (unsigned long long)head + j * 4ull;
        float4 v;
        v.x = __ull2float_rn(i0);
        v.y = __ull2float_rn(i0 + 1);
        v.z = __ull2float_rn(i0 + 2);
        v.w = __ull2float_rn(i0 + 3);
        uint4 bits = make_uint4(__float_as_uint(v.x), __float_as_uint(v.y), __float_as_uint(v.z), __float_as_uint(v.w));
        st_stream<0>(reinterpret_cast<uint4 *>(dst4 + j), bits);
    }
}

// VEC: both pointers 16-byte aligned.  Tile = U vectors per thread; all loads of a tile are issued before its
// stores, and the launcher sizes the grid to one short CTA per tile (see the copy kernels).
template <bool VEC, int U>
__global__ void __launch_bounds__(512) axpb_kernel(float *__restrict__ y, const float *__restrict__ x, float a, float b,
                                                   size_t count) {
    pdl_launch_dependents();
    pdl_wait();
    if (VEC) {
        const size_t nvec = count / 4;
        const uint4 *x4 = reinterpret_cast<const uint4 *>(x);
        uint4 *y4 = reinterpret_cast<uint4 *>(y);
        const size_t tile = (size_t)U * blockDim.x;
        const size_t ntiles = (nvec + tile - 1) / tile;
        for (size_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
            const size_t base = t * tile + threadIdx.x;
            uint4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const size_t j = base + (size_t)u * blockDim.x;
                v[u] = (j < nvec) ? ld_stream<2>(x4 + j) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const size_t j = base + (size_t)u * blockDim.x;
                uint4 w = v[u];
                w.x = __float_as_uint(__fadd_rn(__fmul_rn(a, __uint_as_float(w.x)), b));
                w.y = __float_as_uint(__fadd_rn(__fmul_rn(a, __uint_as_float(w.y)), b));
                w.z = __float_as_uint(__fadd_rn(__fmul_rn(a, __uint_as_float(w.z)), b));
                w.w = __float_as_uint(__fadd_rn(__fmul_rn(a, __uint_as_float(w.w)), b));
                if (j < nvec) st_stream<2>(y4 + j, w);
            }
        }
        if (blockIdx.x == 0) {  // up to three trailing elements
            const size_t i = nvec * 4 + threadIdx.x;
            if (i < count) y[i] = __fadd_rn(__fmul_rn(a, x[i]), b);
        }
    } else {
        const size_t stride = (size_t)gridDim.x * blockDim.x;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride)
            y[i] = __fadd_rn(__fmul_rn(a, x[i]), b);
    }
}

// Seeded byte stream: word i = mix64(seed + (i + 1) * golden).  Two words per 16-byte store.
__global__ void __launch_bounds__(512) splitmix_fill_kernel(uint64_t *__restrict__ dst, size_t nwords, uint64_t seed,
                                                            uint8_t *tail_dst, int tail_bytes) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool al16 = (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
    if (al16) {
        const size_t npair = nwords / 2;
        for (size_t j = tid; j < npair; j += stride) {
            const uint64_t w0 = mix64(seed + (2 * j + 1) * kGolden);
            const uint64_t w1 = mix64(seed + (2 * j + 2) * kGolden);
            st_stream<0>(reinterpret_cast<uint4 *>(dst) + j,
                         make_uint4((uint32_t)w0, (uint32_t)(w0 >> 32), (uint32_t)w1, (uint32_t)(w1 >> 32)));
        }
        if (tid == 0 && (nwords & 1)) dst[nwords - 1] = mix64(seed + nwords * kGolden);
    } else {
        for (size_t i = tid; i < nwords; i += stride) dst[i] = mix64(seed + (i + 1) * kGolden);
    }
    if (tid == 0 && tail_bytes) {
        const uint64_t w = mix64(seed + (nwords + 1) * kGolden);
        for (int b = 0; b < tail_bytes; ++b) tail_dst[b] = (uint8_t)(w >> (8 * b));
    }
}

namespace {

int grid_for(size_t items, int threads, int ctas_sm) {
    size_t need = (items + threads - 1) / threads;
    if (need == 0) need = 1;
    const size_t cap = (size_t)sm_count() * ctas_sm;
    return (int)(need < cap ? need : cap);
}

int memset_any(void *dst, uint32_t pattern, int elem, size_t count, int path, int ctas, cudaStream_t st) {
    if (count == 0) return 0;
    if (dst == nullptr || ctas < 0) return 1;
    const uintptr_t a = reinterpret_cast<uintptr_t>(dst);
    if (a & (uintptr_t)(elem - 1)) return 1;
    const size_t bytes = count * (size_t)elem;
    FillEdges e;
    e.dst = static_cast<uint8_t *>(dst);
    size_t head = (16 - (a & 15)) & 15;
    if (head > bytes) head = bytes;
    const size_t nvec = (bytes - head) / 16;
    e.head = (int)head;
    e.tail = (int)(bytes - head - nvec * 16);
    e.tail_off = head + nvec * 16;
    e.pattern = pattern;
    e.elem = elem;
    uint8_t *body = e.dst + head;
    const Tuning &tu = tuning();
    if (path == 0) path = tu.memset_path;
    if (path == 0) path = 1;  // vector stores measured faster than the bulk replay at every size
    if (path == 2) {
        const uint32_t chunk = (uint32_t)tu.memset_chunk;
        if (chunk < 1024 || chunk > 65536 || (chunk & 127)) return 1;
        int issuers = tu.memset_issuers;
        if (issuers < 2) issuers = 2;  // two warps are needed for the edge bytes
        if (issuers > 8) issuers = 8;
        const int bthreads = 32 * issuers;
        const size_t nchunks = (nvec * 16 + chunk - 1) / chunk;
        const size_t need = (nchunks + issuers - 1) / issuers;
        size_t cap = ctas > 0 ? (size_t)ctas : (size_t)sm_count() * tu.memset_bulk_ctas_sm;
        const int grid = (int)(need < cap ? (need ? need : 1) : cap);
        if (tu.memset_cache_hint) return launch_kernel(memset_bulk_kernel<true>, grid, bthreads, chunk, st, body, nvec * 16, chunk, e);
        return launch_kernel(memset_bulk_kernel<false>, grid, bthreads, chunk, st, body, nvec * 16, chunk, e);
    }
    if (path != 1) return 1;
    int threads = tu.memset_threads;
    int unroll = tu.memset_unroll;
    const size_t want = (size_t)sm_count() * 2;
    while (unroll > 1 && (nvec / ((size_t)unroll * threads)) < want) unroll >>= 1;
    while (threads > 64 && (nvec / ((size_t)unroll * threads)) < want) threads >>= 1;
    const size_t per_cta = (size_t)unroll * threads;
    size_t need = (nvec + per_cta - 1) / per_cta;
    if (need == 0) need = 1;
    size_t cap = ctas > 0 ? (size_t)ctas : (size_t)sm_count() * tu.memset_ctas_sm * (512 / threads);
    const int grid = (int)(need < cap ? need : cap);
    uint4 *dv = reinterpret_cast<uint4 *>(body);
    const size_t pad = (size_t)tu.memset_smem_pad;
    switch (unroll) {
        case 1: return launch_kernel(memset_vec_kernel<1>, grid, threads, pad, st, dv, nvec, e);
        case 2: return launch_kernel(memset_vec_kernel<2>, grid, threads, pad, st, dv, nvec, e);
        case 4: return launch_kernel(memset_vec_kernel<4>, grid, threads, pad, st, dv, nvec, e);
        default: return launch_kernel(memset_vec_kernel<8>, grid, threads, pad, st, dv, nvec, e);
    }
}

}  // namespace
}  // namespace lcb

namespace lcb {
int preload_fill_kernels() {
    cudaFuncAttributes a;
    cudaError_t e = cudaFuncGetAttributes(&a, memset_vec_kernel<8>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, memset_vec_kernel<1>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, index_fill_kernel);
    return (int)e;
}
}  // namespace lcb

extern "C" int lcb_memset_ex(void *dst, unsigned int value, int elem_bytes, size_t count, int path, int ctas,
                             lcbStream stream) {
    uint32_t pattern;
    switch (elem_bytes) {
        case 1: pattern = (value & 0xffu) * 0x01010101u; break;
        case 2: pattern = (value & 0xffffu) * 0x00010001u; break;
        case 4: pattern = value; break;
        default: return 1;
    }
    if (path < 0 || path > 2) return 1;
    return lcb::memset_any(dst, pattern, elem_bytes, count, path, ctas, static_cast<cudaStream_t>(stream));
}

extern "C" int lcb_memset_d8(void *dst, unsigned char value, size_t count, lcbStream stream) {
    return lcb_memset_ex(dst, value, 1, count, 0, 0, stream);
}
extern "C" int lcb_memset_d16(void *dst, unsigned short value, size_t count, lcbStream stream) {
    return lcb_memset_ex(dst, value, 2, count, 0, 0, stream);
}
extern "C" int lcb_memset_d32(void *dst, unsigned int value, size_t count, lcbStream stream) {
    return lcb_memset_ex(dst, value, 4, count, 0, 0, stream);
}

extern "C" int lcb_index_fill_f32(float *dst, size_t count, lcbStream stream) {
    using namespace lcb;
    if (count == 0) return 0;
    if (dst == nullptr || (reinterpret_cast<uintptr_t>(dst) & 3)) return 1;
    size_t head = ((16 - (reinterpret_cast<uintptr_t>(dst) & 15)) & 15) / 4;
    if (head > count) head = count;
    const size_t nvec = (count - head) / 4;
    const int threads = 512;
    const int grid = grid_for(nvec, threads, tuning().fill_ctas_sm);
    return launch_kernel(index_fill_kernel, grid, threads, 0, static_cast<cudaStream_t>(stream), dst, count, (int)head, nvec);
}

extern "C" int lcb_axpb_f32(float *y, const float *x, float a, float b, size_t count, lcbStream stream) {
    using namespace lcb;
    if (count == 0) return 0;
    if (y == nullptr || x == nullptr) return 1;
    if ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(x)) & 3) return 1;
    const bool vec = ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(x)) & 15) == 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (vec) {
        // one short CTA per tile of 128 threads x 2 vectors (4 KiB), like the copy kernel it resembles
        const int threads = 128;
        const size_t tiles = (count / 4 + 2 * threads - 1) / (2 * threads);
        const size_t cap = (size_t)sm_count() * tuning().axpb_ctas_sm;
        const int grid = (int)(tiles == 0 ? 1 : (tiles < cap ? tiles : cap));
        return launch_kernel(axpb_kernel<true, 2>, grid, threads, 0, st, y, x, a, b, count);
    }
    return launch_kernel(axpb_kernel<false, 1>, grid_for(count, 512, 64), 512, 0, st, y, x, a, b, count);
}

extern "C" int lcb_fill_splitmix64(void *dst, size_t bytes, uint64_t seed, lcbStream stream) {
    using namespace lcb;
    if (bytes == 0) return 0;
    if (dst == nullptr || (reinterpret_cast<uintptr_t>(dst) & 7)) return 1;
    const size_t nwords = bytes / 8;
    const int tail = (int)(bytes - nwords * 8);
    const int threads = 512;
    splitmix_fill_kernel<<<grid_for(nwords / 2 + 1, threads, 4), threads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint64_t *>(dst), nwords, seed, static_cast<uint8_t *>(dst) + nwords * 8, tail);
    return check_launch();
}

extern "C" int lcb_fill_splitmix64_at(void *dst, size_t bytes, uint64_t seed, uint64_t first_word, lcbStream stream) {
    // word first_word + i of the stream is mix64(seed + (first_word + i + 1) * golden): the same stream started
    // from a shifted seed
    return lcb_fill_splitmix64(dst, bytes, seed + first_word * lcb::kGolden, stream);
}
