// Device-to-device copy kernels for sm_100a and their C-ABI launchers.
//
// Replaces the reference's three-kernel split (memcpyD2D, driverapi/src/memcopy.cpp:77-158, launching
// memcpyKernelHighBW / LowLatency / Trailing, driverapi/kernels/memcpy/memcpy.cu:5-27) with ONE launch
// per copy that handles any size and any alignment:
//
//   dst:  [ head < 16 B ][ body: nvec 16-byte vectors, dst 16-byte aligned ][ tail < 16 B ]
//
//  * copy_vec_kernel    each lane keeps U 16-byte loads in flight before storing; launched as one short CTA
//                       per tile (the hardware deals tiles to SMs in address order as they free up).
//                       If src is not congruent to dst mod 16 the lanes load ALIGNED source vectors and
//                       rebuild each output vector from their own vector and their right neighbour's,
//                       fetched with one warp shuffle per word (lane 0 supplies the first vector of the
//                       next row), then a funnel shift for the sub-word part.  No misaligned access is
//                       ever issued; DRAM traffic stays at the algorithmic 2 bytes per byte copied.
//  * copy_tma_kernel    for mutually aligned spans: one thread per CTA moves its chunks through shared
//                       memory with bulk copies (cp.async.bulk global->shared with mbarrier complete_tx,
//                       then shared->global in bulk groups); by default one 32 KiB chunk per CTA, or a
//                       persistent multi-stage ring.  Non-multicast forms only, so the same kernel is
//                       usable with a peer GPU's memory on either side.
//  * alltoall_kernel     one launch that moves every chunk of an all-to-all between this GPU and all its
//                       peers (the copy fused with the exchange), by remote loads (pull) or stores (push).
#include <cstdio>

#include "common.cuh"
#include "lcb200_kernels.h"

namespace lcb {

// Sticky per-device error word, read and cleared by lcb_device_error_word().
__device__ unsigned int g_error_word = 0;
// Host-mapped mirror of that word (set up per device by setup_error_mirror): a kernel that gives up a wait
// also raises the bit there, so the host can look at it after any stream wait without a device round trip.
__device__ unsigned int *g_error_mirror = nullptr;

__device__ __forceinline__ void raise_error(unsigned int bits) {
    atomicOr(&g_error_word, bits);
    unsigned int *m = g_error_mirror;
    if (m != nullptr) {
        atomicOr_system(m, bits);
        __threadfence_system();
    }
}

// ---------------------------------------------------------------------------------------------
// vector path
// ---------------------------------------------------------------------------------------------

// Output vector from two consecutive aligned source vectors when the source stream starts
// s = 4*SW + sb bytes into `a` (sb8 = 8*sb).
template <int SW>
__device__ __forceinline__ uint4 realign(const uint4 &a, const uint4 &b, int sb8) {
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    uint4 o;
    o.x = __funnelshift_r(w[SW + 0], w[SW + 1], sb8);
    o.y = __funnelshift_r(w[SW + 1], w[SW + 2], sb8);
    o.z = __funnelshift_r(w[SW + 2], w[SW + 3], sb8);
    o.w = __funnelshift_r(w[SW + 3], w[SW + 4], sb8);
    return o;
}

struct Edges {            // the < 16-byte pieces either side of the vector body
    uint8_t *dst;         // original dst
    const uint8_t *src;   // original src
    int head;             // bytes before the body
    int tail;             // bytes after the body
    size_t tail_off;      // offset of the tail from dst / src
};

__device__ __forceinline__ void copy_edges(const Edges &e, int t) {
    // two different warps so head and tail go out together
    if (t < e.head) e.dst[t] = e.src[t];
    int u = t - 32;
    if (u >= 0 && u < e.tail) e.dst[e.tail_off + u] = e.src[e.tail_off + u];
}

// SW < 0: src and dst congruent mod 16 (srcv is the source body itself).
// SW in 0..3: srcv is the source body rounded DOWN to 16 bytes; output vector j is bytes
// [16 j + s, 16 j + s + 16) of the srcv stream with s = 4 SW + sb8 / 8, 1 <= s <= 15.
// early != 0: the caller vouches that nothing still running on the stream writes the source, so the first
// tile's loads are issued BEFORE the wait for the previous kernel (they fly while that kernel drains); every
// store still comes after the wait.
template <int SW, int U, int MODE>
__global__ void __launch_bounds__(512) copy_vec_kernel(uint4 *__restrict__ dstv, const uint4 *__restrict__ srcv,
                                                       size_t nvec, int sb8, Edges e, int early) {
    const int lane = threadIdx.x & 31;
    const size_t warps_total = (size_t)gridDim.x * (blockDim.x >> 5);
    const size_t gwarp = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    constexpr size_t TILE = (size_t)U * 32;  // vectors per warp per iteration
    const size_t ntiles = (nvec + TILE - 1) / TILE;
    uint64_t pol = 0;
    if (MODE >= 3) pol = policy_evict_first();

    pdl_launch_dependents();
    bool waited = false;
    if (!early) {
        pdl_wait();
        waited = true;
        if (blockIdx.x == 0) copy_edges(e, threadIdx.x);
    }

    for (size_t t = gwarp; t < ntiles; t += warps_total) {
        const size_t base = t * TILE;
        uint4 v[U];
        if (base + TILE <= nvec) {  // full tile: no guards
#pragma unroll
            for (int u = 0; u < U; ++u) v[u] = ld_stream<MODE>(srcv + base + u * 32 + lane, pol);
            uint4 extra = make_uint4(0, 0, 0, 0);
            if (SW >= 0 && lane == 0) extra = ld_stream<MODE>(srcv + base + TILE, pol);
            if (!waited) {
                pdl_wait();
                waited = true;
            }
            if (SW < 0) {
#pragma unroll
                for (int u = 0; u < U; ++u) st_stream<MODE>(dstv + base + u * 32 + lane, v[u], pol);
            } else {
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    // every lane needs the vector one to its right; lane 31's neighbour is lane 0's next row
                    uint4 give = v[u];
                    if (lane == 0) give = (u + 1 < U) ? v[(u + 1 < U) ? u + 1 : u] : extra;
                    uint4 nxt;
                    const int from = (lane + 1) & 31;
                    nxt.x = __shfl_sync(0xffffffffu, give.x, from);
                    nxt.y = __shfl_sync(0xffffffffu, give.y, from);
                    nxt.z = __shfl_sync(0xffffffffu, give.z, from);
                    nxt.w = __shfl_sync(0xffffffffu, give.w, from);
                    st_stream<MODE>(dstv + base + u * 32 + lane, realign<(SW < 0 ? 0 : SW)>(v[u], nxt, sb8), pol);
                }
            }
        } else {  // last, partial tile
            // realign mode also needs source vector index nvec (it holds the last bytes of the body)
            const size_t src_limit = (SW < 0) ? nvec : nvec + 1;
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const size_t j = base + u * 32 + lane;
                v[u] = (j < src_limit) ? ld_stream<MODE>(srcv + j, pol) : make_uint4(0, 0, 0, 0);
            }
            uint4 extra = make_uint4(0, 0, 0, 0);
            if (SW >= 0 && lane == 0 && base + TILE < src_limit) extra = ld_stream<MODE>(srcv + base + TILE, pol);
            if (!waited) {
                pdl_wait();
                waited = true;
            }
            if (SW < 0) {
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const size_t j = base + u * 32 + lane;
                    if (j < nvec) st_stream<MODE>(dstv + j, v[u], pol);
                }
            } else {
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    uint4 give = v[u];
                    if (lane == 0) give = (u + 1 < U) ? v[(u + 1 < U) ? u + 1 : u] : extra;
                    uint4 nxt;
                    const int from = (lane + 1) & 31;
                    nxt.x = __shfl_sync(0xffffffffu, give.x, from);
                    nxt.y = __shfl_sync(0xffffffffu, give.y, from);
                    nxt.z = __shfl_sync(0xffffffffu, give.z, from);
                    nxt.w = __shfl_sync(0xffffffffu, give.w, from);
                    const size_t j = base + u * 32 + lane;
                    if (j < nvec) st_stream<MODE>(dstv + j, realign<(SW < 0 ? 0 : SW)>(v[u], nxt, sb8), pol);
                }
            }
        }
    }
    if (early) {  // every thread passes the wait before it exits, so completion of this kernel implies completion
                  // of the one before it (the next kernel's wait relies on that); the edge bytes are stores
        if (!waited) pdl_wait();
        if (blockIdx.x == 0) copy_edges(e, threadIdx.x);
    }
}


// ---------------------------------------------------------------------------------------------
// 32-byte vector path (sm_100 256-bit global accesses with an L2 evict_first priority)
// ---------------------------------------------------------------------------------------------
struct V8 {
    uint32_t r[8];
};

__device__ __forceinline__ V8 ld_v8(const void *p) {
    V8 v;
    asm volatile("ld.global.L1::no_allocate.L2::evict_first.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v.r[0]), "=r"(v.r[1]), "=r"(v.r[2]), "=r"(v.r[3]), "=r"(v.r[4]), "=r"(v.r[5]), "=r"(v.r[6]),
                   "=r"(v.r[7])
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void st_v8(void *p, const V8 &v) {
    asm volatile("st.global.L1::no_allocate.L2::evict_first.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 :: "l"(p), "r"(v.r[0]), "r"(v.r[1]), "r"(v.r[2]), "r"(v.r[3]), "r"(v.r[4]), "r"(v.r[5]), "r"(v.r[6]),
                    "r"(v.r[7])
                 : "memory");
}

// Both bodies 32-byte aligned; n32 32-byte vectors; edges (< 32 bytes each side) by the first two warps of CTA 0.
template <int U>
__global__ void __launch_bounds__(512) copy_vec32_kernel(uint8_t *__restrict__ dst, const uint8_t *__restrict__ src,
                                                         size_t n32, Edges e) {
    pdl_launch_dependents();
    pdl_wait();
    if (blockIdx.x == 0) copy_edges(e, threadIdx.x);
    const int lane = threadIdx.x & 31;
    const size_t warps_total = (size_t)gridDim.x * (blockDim.x >> 5);
    const size_t gwarp = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    constexpr size_t TILE = (size_t)U * 32;
    const size_t ntiles = (n32 + TILE - 1) / TILE;
    for (size_t t = gwarp; t < ntiles; t += warps_total) {
        const size_t base = t * TILE;
        V8 v[U];
        if (base + TILE <= n32) {
#pragma unroll
            for (int u = 0; u < U; ++u) v[u] = ld_v8(src + (base + u * 32 + lane) * 32);
#pragma unroll
            for (int u = 0; u < U; ++u) st_v8(dst + (base + u * 32 + lane) * 32, v[u]);
        } else {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const size_t j = base + u * 32 + lane;
                if (j < n32) st_v8(dst + j * 32, ld_v8(src + j * 32));
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// bulk-copy ring
// ---------------------------------------------------------------------------------------------

// One CTA = one warp; lane 0 runs the ring, the other lanes of CTA 0 copy the edge bytes.
// Chunk c of the body (chunk bytes each, the last one shorter) belongs to CTA c % gridDim.x.
// S stages, L loads in flight ahead of the store front.  Stage reuse: before loading chunk k+L into
// its stage, the bulk store that last read that stage (chunk k+L-S) must have finished reading
// shared memory, i.e. at most S-L younger store groups may still be pending.
template <int S, int L, bool HINT>
__global__ void __launch_bounds__(32) copy_tma_kernel(uint8_t *__restrict__ dst, const uint8_t *__restrict__ src,
                                                      size_t body, uint32_t chunk, Edges e, int early) {
    extern __shared__ __align__(128) uint8_t smem[];
    static_assert(L >= 1 && L < S, "need at least one stage of slack between loads and stores");
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t)S * chunk);

    pdl_launch_dependents();
    if (threadIdx.x == 0) {  // barrier set-up overlaps the previous kernel's tail
        for (int s = 0; s < S; ++s) mbar_init(smem_addr(bars) + 8 * s, 1);
        mbar_init_fence();
    }
    // early != 0 (nothing still running on the stream writes the source): the first loads are issued before
    // the wait for the previous kernel; stores, edge bytes included, always come after it
    if (!early) pdl_wait();
    if (blockIdx.x == 0 && threadIdx.x != 0) {
        if (early) pdl_wait();
        // lanes 1..15 -> head bytes, lanes 16..31 -> tail bytes
        const int t = threadIdx.x;
        if (t < 16) {
            if (t - 1 < e.head) e.dst[t - 1] = e.src[t - 1];
        } else if (t - 16 < e.tail) {
            e.dst[e.tail_off + (t - 16)] = e.src[e.tail_off + (t - 16)];
        }
        // (head and tail are < 16 by construction, 15 lanes each are enough)
    }
    if (threadIdx.x != 0) return;

    // Chunk c of the body belongs to CTA c % gridDim.x; this CTA's k-th chunk starts at (blockIdx.x + k * grid) * chunk.
    // The issuing thread is the only one running, so everything in its loop is kept incremental: no division,
    // no 64-bit multiply, stage and parity carried along.
    const size_t nchunks = (body + chunk - 1) / chunk;
    if ((size_t)blockIdx.x >= nchunks) {
        if (early) pdl_wait();
        return;
    }
    const uint32_t n_my = (uint32_t)((nchunks - blockIdx.x + gridDim.x - 1) / gridDim.x);
    const size_t stride = (size_t)gridDim.x * chunk;
    const uint32_t smem_base = smem_addr(smem);
    const uint32_t bar_base = smem_addr(bars);

    uint64_t pol = 0;
    if (HINT) pol = policy_evict_first();

    // load cursor
    size_t ld_off = (size_t)blockIdx.x * chunk;
    uint32_t ld_stage = 0, issued = 0;
    auto issue_load = [&]() {
        const size_t left = body - ld_off;
        const uint32_t len = left < chunk ? (uint32_t)left : chunk;
        const uint32_t bar = bar_base + 8 * ld_stage;
        mbar_expect_tx(bar, len);
        bulk_g2s<HINT>(smem_base + ld_stage * chunk, src + ld_off, len, bar, pol);
        ld_off += stride;
        ld_stage = (ld_stage + 1 == S) ? 0 : ld_stage + 1;
        ++issued;
    };
    while (issued < (uint32_t)L && issued < n_my) issue_load();
    if (early) pdl_wait();

    // store cursor
    size_t st_off = (size_t)blockIdx.x * chunk;
    uint32_t st_stage = 0, parity = 0, k = 0;
    bool ok = true;
    for (; k < n_my; ++k) {
        if (!mbar_wait_bounded(bar_base + 8 * st_stage, parity)) { ok = false; break; }
        const size_t left = body - st_off;
        bulk_s2g<HINT>(dst + st_off, smem_base + st_stage * chunk, left < chunk ? (uint32_t)left : chunk, pol);
        bulk_commit();
        st_off += stride;
        if (++st_stage == S) {
            st_stage = 0;
            parity ^= 1;
        }
        if (issued < n_my) {
            // the stage about to be reloaded was last read by the store S-L groups back
            if (issued >= (uint32_t)S) bulk_wait_read<S - L>();
            issue_load();
        }
    }
    if (!ok) {
        raise_error(kErrMbarrierTimeout);
        // loads already issued still target our shared memory: give each one more bounded wait
        for (uint32_t j = k; j < issued; ++j) mbar_wait_bounded(bar_base + 8 * (j % S), (j / S) & 1);
    }
    bulk_wait_all();
}


// Two-issuer variant of the bulk ring: lane 0 of warp 0 only issues loads, lane 0 of warp 1 only issues
// stores.  full[s] (complete_tx) tells the storer a stage is loaded; empty[s] (one arrival) tells the loader
// that the store which last used the stage has finished reading it -- the storer learns that from
// cp.async.bulk.wait_group.read D, D store groups behind its newest one.  Neither thread ever waits for the
// other's kind of work, so twice as many bulk instructions can be in issue per SM.
template <int S, int D, bool HINT>
__global__ void __launch_bounds__(64) copy_tma2_kernel(uint8_t *__restrict__ dst, const uint8_t *__restrict__ src,
                                                       size_t body, uint32_t chunk, Edges e) {
    extern __shared__ __align__(128) uint8_t smem[];
    static_assert(D >= 1 && D < S, "the storer must release stages before the loader runs out of them");
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t)S * chunk);
    const uint32_t full_base = smem_addr(bars), empty_base = full_base + 8 * S;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < 2 * S; ++s) mbar_init(full_base + 8 * s, 1);
        mbar_init_fence();
    }
    __syncthreads();
    pdl_wait();
    if (blockIdx.x == 0) {  // lanes 1..15 of warp 0 -> head bytes, lanes 1..15 of warp 1 -> tail bytes
        const int t = threadIdx.x;
        if (t >= 1 && t < 16 && t - 1 < e.head) e.dst[t - 1] = e.src[t - 1];
        if (t >= 33 && t < 48 && t - 33 < e.tail) e.dst[e.tail_off + (t - 33)] = e.src[e.tail_off + (t - 33)];
    }
    if ((threadIdx.x & 31) != 0) return;

    const size_t nchunks = (body + chunk - 1) / chunk;
    if ((size_t)blockIdx.x >= nchunks) return;
    const uint32_t n_my = (uint32_t)((nchunks - blockIdx.x + gridDim.x - 1) / gridDim.x);
    const size_t stride = (size_t)gridDim.x * chunk;
    const uint32_t smem_base = smem_addr(smem);
    uint64_t pol = 0;
    if (HINT) pol = policy_evict_first();
    size_t off = (size_t)blockIdx.x * chunk;
    uint32_t stage = 0, parity = 0;
    bool ok = true;

    if (threadIdx.x == 0) {  // ---- loader
        for (uint32_t j = 0; j < n_my; ++j) {
            // second and later trips round the ring wait for the stage to be released (phase j/S - 1)
            if (j >= (uint32_t)S && !mbar_wait_bounded(empty_base + 8 * stage, parity ^ 1)) { ok = false; break; }
            const size_t left = body - off;
            const uint32_t len = left < chunk ? (uint32_t)left : chunk;
            mbar_expect_tx(full_base + 8 * stage, len);
            bulk_g2s<HINT>(smem_base + stage * chunk, src + off, len, full_base + 8 * stage, pol);
            off += stride;
            if (++stage == S) {
                stage = 0;
                parity ^= 1;
            }
        }
        if (!ok) raise_error(kErrMbarrierTimeout);
        return;
    }
    // ---- storer
    uint32_t rel_stage = 0;  // stage of the chunk released next
    for (uint32_t k = 0; k < n_my; ++k) {
        if (!mbar_wait_bounded(full_base + 8 * stage, parity)) { ok = false; break; }
        const size_t left = body - off;
        bulk_s2g<HINT>(dst + off, smem_base + stage * chunk, left < chunk ? (uint32_t)left : chunk, pol);
        bulk_commit();
        off += stride;
        if (++stage == S) {
            stage = 0;
            parity ^= 1;
        }
        if (k >= (uint32_t)D) {
            bulk_wait_read<D>();  // store k-D no longer reads shared memory
            mbar_arrive(empty_base + 8 * rel_stage);
            rel_stage = (rel_stage + 1 == S) ? 0 : rel_stage + 1;
        }
    }
    if (!ok) raise_error(kErrMbarrierTimeout);
    bulk_wait_all();
}

// ---------------------------------------------------------------------------------------------
// phase-grouped bulk copy (experiment: does separating reads from writes in time help the DRAM?)
// ---------------------------------------------------------------------------------------------
// One CTA per SM, S stages of `chunk` bytes of shared memory each.  All CTAs of the GPU load while
// (globaltimer / phase_ns) is even and store while it is odd, so that -- as far as the SMs can arrange it -- the
// memory system sees T nanoseconds of reads followed by T nanoseconds of writes instead of a 50/50 mix.  Within a
// stage index the CTAs touch one compact window of the buffers.  Waiting for a phase is bounded by the clock
// itself (at most two phase lengths).  Measured: see the launcher.
__device__ __forceinline__ void wait_for_phase(unsigned long long phase_ns, unsigned int want) {
    if (phase_ns == 0) return;
    unsigned long long t0, t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    t = t0;
    while (((t / phase_ns) & 1ull) != want && t - t0 < 2 * phase_ns) {
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    }
}

template <int S>
__global__ void __launch_bounds__(32) copy_phase_kernel(uint8_t *__restrict__ dst, const uint8_t *__restrict__ src, size_t body,
                                                        uint32_t chunk, unsigned long long phase_ns, Edges e) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t)S * chunk);
    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) mbar_init(smem_addr(bars) + 8 * s, 1);
        mbar_init_fence();
    }
    pdl_wait();
    if (blockIdx.x == 0 && threadIdx.x != 0) {
        const int t = threadIdx.x;
        if (t < 16) {
            if (t - 1 < e.head) e.dst[t - 1] = e.src[t - 1];
        } else if (t - 16 < e.tail) {
            e.dst[e.tail_off + (t - 16)] = e.src[e.tail_off + (t - 16)];
        }
    }
    if (threadIdx.x != 0) return;
    const size_t nchunks = (body + chunk - 1) / chunk;
    const size_t per_round = (size_t)gridDim.x * S;
    const uint32_t smem_base = smem_addr(smem), bar_base = smem_addr(bars);
    uint32_t parity = 0;
    bool ok = true;
    for (size_t first = 0; first < nchunks && ok; first += per_round) {
        int loaded = 0;
        wait_for_phase(phase_ns, 0);
        for (int s = 0; s < S; ++s) {
            const size_t c = first + (size_t)s * gridDim.x + blockIdx.x;
            if (c >= nchunks) break;
            const size_t off = c * chunk;
            const uint32_t len = body - off < chunk ? (uint32_t)(body - off) : chunk;
            mbar_expect_tx(bar_base + 8 * s, len);
            bulk_g2s<false>(smem_base + s * chunk, src + off, len, bar_base + 8 * s, 0);
            ++loaded;
        }
        for (int s = 0; s < loaded; ++s) {
            if (!mbar_wait_bounded(bar_base + 8 * s, parity)) {
                ok = false;
                break;
            }
        }
        if (!ok) break;
        wait_for_phase(phase_ns, 1);
        for (int s = 0; s < loaded; ++s) {
            const size_t off = (first + (size_t)s * gridDim.x + blockIdx.x) * chunk;
            const uint32_t len = body - off < chunk ? (uint32_t)(body - off) : chunk;
            bulk_s2g<false>(dst + off, smem_base + s * chunk, len, 0);
        }
        bulk_commit();
        bulk_wait_read<0>();
        parity ^= 1;  // every barrier that was used completed one phase; unused ones are never waited on again
        if (loaded < S) break;  // the last, partial round
    }
    if (!ok) raise_error(kErrMbarrierTimeout);
    bulk_wait_all();
}

// ---------------------------------------------------------------------------------------------
// all-to-all (push and pull)
// ---------------------------------------------------------------------------------------------
struct PeerPtrs {
    uint4 *buf[16];
};

// The exchange fused into one copy kernel.  CTA b serves peer (rank + 1 + b % n) % n, so consecutive CTAs
// talk to different GPUs and every NVLink port is busy from the first wave on; within a peer the CTAs stride
// over warp tiles.
//   PULL = false: `mine` is this rank's send buffer, peers.buf[j] the receive buffers: chunk j of `mine` is
//                 STORED to peers.buf[j] + rank * chunk.
//   PULL = true:  `mine` is this rank's receive buffer, peers.buf[j] the send buffers: chunk `rank` of
//                 peers.buf[j] is LOADED into mine + j * chunk.
// Measured on NVLink 5 (GB/s per GPU): one direction of a link busy -- loads 786, stores 716; both directions
// busy, as in a real all-to-all -- stores 704, loads 665 (load requests compete with the peer's data).
template <int U, int MODE, bool PULL>
__global__ void __launch_bounds__(512) alltoall_kernel(PeerPtrs peers, uint4 *__restrict__ mine,
                                                       size_t chunk_vec, int n, int rank) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int slot = blockIdx.x % n;
    const int peer = (rank + 1 + slot) % n;
    const size_t ctas_per_peer = gridDim.x / n;  // grid is a multiple of n
    const size_t cta_in_peer = blockIdx.x / n;
    const size_t warps_total = ctas_per_peer * (blockDim.x >> 5);
    const size_t gwarp = cta_in_peer * (blockDim.x >> 5) + (threadIdx.x >> 5);
    constexpr size_t TILE = (size_t)U * 32;
    const size_t ntiles = (chunk_vec + TILE - 1) / TILE;
    const uint4 *s = PULL ? peers.buf[peer] + (size_t)rank * chunk_vec : mine + (size_t)peer * chunk_vec;
    uint4 *d = PULL ? mine + (size_t)peer * chunk_vec : peers.buf[peer] + (size_t)rank * chunk_vec;
    for (size_t t = gwarp; t < ntiles; t += warps_total) {
        const size_t base = t * TILE;
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const size_t j = base + u * 32 + lane;
            v[u] = (j < chunk_vec) ? ld_stream<MODE>(s + j) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const size_t j = base + u * 32 + lane;
            if (j < chunk_vec) st_stream<1>(d + j, v[u]);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// flags between GPUs (one thread each): how ranks that live in different processes keep a schedule of
// copy-engine transfers in lock-step without the host
// ---------------------------------------------------------------------------------------------
__global__ void flag_post_kernel(unsigned int *flag, unsigned int value) {
    // everything earlier on the stream (the engine copy this announces) has completed before this kernel starts
    asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(flag), "r"(value) : "memory");
}

// Returns when *flag has reached `value` (counters only grow; the comparison survives wrap-around), or after
// `timeout_ns` of GPU time: then it raises kErrFlagTimeout in the sticky error word and returns all the same,
// so a peer that died or never posts costs a bounded wait and an error status, not a hung GPU.
__device__ __forceinline__ void flag_wait(const unsigned int *flag, unsigned int value, unsigned long long timeout_ns);

__global__ void flag_wait_kernel(const unsigned int *flag, unsigned int value, unsigned long long timeout_ns) {
    flag_wait(flag, value, timeout_ns);
}

// Post one flag, then wait for another, in one launch: between two engine copies of the lock-step exchange this
// saves a kernel launch and an engine-kernel switch.
__global__ void flag_post_wait_kernel(unsigned int *post, unsigned int post_value, const unsigned int *flag, unsigned int value,
                                      unsigned long long timeout_ns) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(post), "r"(post_value) : "memory");
    flag_wait(flag, value, timeout_ns);
}

__device__ __forceinline__ void flag_wait(const unsigned int *flag, unsigned int value, unsigned long long timeout_ns) {
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (unsigned int polls = 0; polls < (1u << 26); ++polls) {
        unsigned int v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if ((int)(v - value) >= 0) return;
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (now - t0 > timeout_ns) break;
        __nanosleep(100);
    }
    raise_error(kErrFlagTimeout);
}

// ---------------------------------------------------------------------------------------------
// ring broadcast: the copy fused with the forwarding
// ---------------------------------------------------------------------------------------------
// One kernel per GPU of a chain root -> d1 -> d2 -> ...  Every GPU but the last copies its own buffer, chunk by
// chunk, into the NEXT GPU's buffer with remote stores; every GPU but the root first waits, per chunk, until the
// previous GPU has delivered that chunk.  "Delivered" is a flag word per chunk in the receiving GPU's memory: the
// sender stores the data, fences at system scope and stores the call's epoch into the flag with release
// semantics; the receiver polls it with acquire loads (one thread per CTA, the others behind a barrier) and
// reads the chunk with volatile loads.  Chunks are small (128 KiB by default), so a byte is forwarded some tens
// of microseconds after it arrived -- all CTAs' chunks in flight, about 37 MiB, divided by the link rate -- where
// the copy-engine chain forwards whole pieces of tens of MiB.  CTA b handles chunks b, b + grid, ...; all CTAs of a GPU work on one
// compact window.  Waits are bounded: a CTA whose wait runs out raises kErrFlagTimeout, sets the GPU's abort
// word so that the other CTAs stop at their next chunk, and returns.
__device__ unsigned int g_ring_abort = 0;

__device__ __forceinline__ uint4 ld_volatile_v4(const uint4 *p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

template <bool ROOT>
__global__ void __launch_bounds__(512) ring_bcast_kernel(const uint4 *__restrict__ local, uint4 *__restrict__ next,
                                                         const unsigned int *flags_in, unsigned int *flags_next, size_t nvec,
                                                         size_t chunk_vec, unsigned int epoch, unsigned long long timeout_ns) {
    __shared__ int proceed;
    const size_t nchunks = (nvec + chunk_vec - 1) / chunk_vec;
    for (size_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
        if (!ROOT) {
            if (threadIdx.x == 0) {
                int ok = 0;
                unsigned long long t0, now;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
                for (unsigned int polls = 0; polls < (1u << 26); ++polls) {
                    unsigned int v;
                    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags_in + c) : "memory");
                    if ((int)(v - epoch) >= 0) {
                        ok = 1;
                        break;
                    }
                    if (*(volatile unsigned int *)&g_ring_abort == epoch) break;  // another CTA of this GPU gave up
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                    if (now - t0 > timeout_ns) {
                        raise_error(kErrFlagTimeout);
                        *(volatile unsigned int *)&g_ring_abort = epoch;
                        break;
                    }
                }
                proceed = ok;
            }
            __syncthreads();
            if (!proceed) return;
        }
        if (next != nullptr) {
            const size_t first = c * chunk_vec;
            const size_t end = first + chunk_vec < nvec ? first + chunk_vec : nvec;
            constexpr int U = 4;
            for (size_t base = first + threadIdx.x; base < end; base += (size_t)U * blockDim.x) {
                uint4 v[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const size_t j = base + (size_t)u * blockDim.x;
                    if (j < end) v[u] = ROOT ? ld_stream<2>(local + j) : ld_volatile_v4(local + j);
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const size_t j = base + (size_t)u * blockDim.x;
                    if (j < end) st_stream<1>(next + j, v[u]);
                }
            }
            __syncthreads();  // every thread's stores are ordered before thread 0's fence by the barrier ...
            if (threadIdx.x == 0) {
                __threadfence_system();  // ... the fence makes them visible system-wide (it is cumulative) ...
                asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(flags_next + c), "r"(epoch) : "memory");  // ... before the flag
            }
        }
        if (!ROOT) __syncthreads();  // `proceed` is rewritten in the next round
    }
}

// Chunks handed out by ticket instead of by a fixed stride: a warp that is done takes the oldest chunk nobody has
// taken yet, so a slow warp (an SM that carries more CTAs, a late flag) delays one chunk and not every W-th.  The
// ticket counters are per GPU; the last warp to leave a kernel sets them back to zero for the next launch (the
// kernels that use them are launched without programmatic overlap and one broadcast at a time per GPU).
__device__ unsigned int g_bcast_ticket[2] = {0, 0};
__device__ unsigned int g_bcast_exit = 0;

__device__ __forceinline__ unsigned int take_ticket(int role, unsigned lane) {
    unsigned int t = 0;
    if (lane == 0) t = atomicAdd(&g_bcast_ticket[role], 1u);
    return __shfl_sync(0xffffffffu, t, 0);
}
__device__ __forceinline__ void leave_tickets(unsigned lane, unsigned int total_warps) {
    __syncwarp();
    if (lane == 0) {
        __threadfence();
        if (atomicAdd(&g_bcast_exit, 1u) == total_warps - 1) {
            g_bcast_ticket[0] = 0;
            g_bcast_ticket[1] = 0;
            __threadfence();
            g_bcast_exit = 0;
        }
    }
}

// The same protocol with one chunk per WARP (8 KiB by default, one flag word each): a warp polls, loads, stores, posts
// and moves on by itself, so nothing in the CTA idles while one warp's release waits for its remote stores to be
// acknowledged, and a byte can be forwarded a few microseconds after it arrived instead of after the time all
// CTAs' chunks take to drain.  Every lane polls the flag (one request per warp: same address) and so holds its
// own acquire; the release is lane 0's, after a warp barrier, and is cumulative over what the barrier ordered
// before it.  Chunks go to the warps by ticket (DYN) or by a fixed stride: warp w handles chunks w, w + W, ...
template <bool ROOT, bool DYN>
__global__ void __launch_bounds__(512) ring_bcast_warp_kernel(const uint4 *__restrict__ local, uint4 *__restrict__ next,
                                                              const unsigned int *flags_in, unsigned int *flags_next, size_t nvec,
                                                              size_t chunk_vec, unsigned int epoch, unsigned long long timeout_ns) {
    const unsigned lane = threadIdx.x & 31u;
    const size_t warps = (size_t)gridDim.x * (blockDim.x >> 5);
    const size_t nchunks = (nvec + chunk_vec - 1) / chunk_vec;
    for (size_t c = DYN ? take_ticket(0, lane) : (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); c < nchunks;
         c = DYN ? take_ticket(0, lane) : c + warps) {
        if (!ROOT) {
            bool ok = false;
            unsigned long long t0, now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
            for (unsigned int polls = 0; polls < (1u << 26); ++polls) {  // uniform over the warp: same address, same clock
                unsigned int v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags_in + c) : "memory");
                if ((int)(v - epoch) >= 0) {
                    ok = true;
                    break;
                }
                if (*(volatile unsigned int *)&g_ring_abort == epoch) break;  // another warp of this GPU gave up
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (now - t0 > timeout_ns) {
                    if (lane == 0) {
                        raise_error(kErrFlagTimeout);
                        *(volatile unsigned int *)&g_ring_abort = epoch;
                    }
                    break;
                }
            }
            if (!__all_sync(0xffffffffu, ok)) break;
        }
        if (next != nullptr) {
            const size_t first = c * chunk_vec;
            const size_t end = first + chunk_vec < nvec ? first + chunk_vec : nvec;
            constexpr int U = 8;
            for (size_t base = first + lane; base < end; base += (size_t)U * 32) {
                uint4 v[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const size_t j = base + (size_t)u * 32;
                    if (j < end) v[u] = ROOT ? ld_stream<2>(local + j) : ld_volatile_v4(local + j);
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const size_t j = base + (size_t)u * 32;
                    if (j < end) st_stream<1>(next + j, v[u]);
                }
            }
            __syncwarp();
            if (lane == 0) asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(flags_next + c), "r"(epoch) : "memory");
        }
    }
    if (DYN) leave_tickets(lane, (unsigned int)warps);
}

// ---------------------------------------------------------------------------------------------
// tree broadcast: two complementary binary trees, one per half of the buffer
// ---------------------------------------------------------------------------------------------
// A chain of G GPUs pays G - 1 hops before the last one is done, each hop worth the chunks of all resident warps.
// Here the first half of the chunks travels down one binary tree over the non-root GPUs and the second half down
// another in which the inner nodes of the first are leaves: every GPU still receives each byte once and sends at
// most one buffer's worth (an inner node stores its half to two children), but the depth is 1 + log2(G - 1).  One
// kernel per GPU serves both halves: the warps are divided between the two roles, a role with children
// forwards (the chunk-per-warp protocol of ring_bcast_warp_kernel, each vector stored once per child, one
// release and one flag store per child), a role without children only waits for its chunks.
struct TreeRole {
    size_t c_lo, c_hi;             // this half: chunks [c_lo, c_hi) of the buffer
    uint4 *child[2];               // the children's buffers (whole buffers, indexed like `local`); null = no child
    unsigned int *child_flags[2];  // the children's flag arrays
};
struct TreeArgs {
    TreeRole role[2];
    unsigned int warps0;  // warps of the grid that work for role[0]; the others work for role[1]
};

template <bool ROOT, bool DYN>
__global__ void __launch_bounds__(512) tree_bcast_kernel(const uint4 *__restrict__ local, const unsigned int *flags_in,
                                                         const TreeArgs a, size_t nvec, size_t chunk_vec, unsigned int epoch,
                                                         unsigned long long timeout_ns) {
    const unsigned lane = threadIdx.x & 31u;
    const size_t gw = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const size_t total = (size_t)gridDim.x * (blockDim.x >> 5);
    const bool second = gw >= a.warps0;
    const size_t w = second ? gw - a.warps0 : gw;
    const size_t W = second ? total - a.warps0 : a.warps0;
    const size_t c_lo = second ? a.role[1].c_lo : a.role[0].c_lo, c_hi = second ? a.role[1].c_hi : a.role[0].c_hi;
    uint4 *const kid0 = second ? a.role[1].child[0] : a.role[0].child[0];
    uint4 *const kid1 = second ? a.role[1].child[1] : a.role[0].child[1];
    unsigned int *const kf0 = second ? a.role[1].child_flags[0] : a.role[0].child_flags[0];
    unsigned int *const kf1 = second ? a.role[1].child_flags[1] : a.role[0].child_flags[1];
    for (size_t c = c_lo + (DYN ? take_ticket(second ? 1 : 0, lane) : w); c < c_hi;
         c = DYN ? c_lo + take_ticket(second ? 1 : 0, lane) : c + W) {
        if (!ROOT) {
            bool ok = false;
            unsigned long long t0, now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
            for (unsigned int polls = 0; polls < (1u << 26); ++polls) {  // uniform over the warp
                unsigned int v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags_in + c) : "memory");
                if ((int)(v - epoch) >= 0) {
                    ok = true;
                    break;
                }
                if (*(volatile unsigned int *)&g_ring_abort == epoch) break;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (now - t0 > timeout_ns) {
                    if (lane == 0) {
                        raise_error(kErrFlagTimeout);
                        *(volatile unsigned int *)&g_ring_abort = epoch;
                    }
                    break;
                }
            }
            if (!__all_sync(0xffffffffu, ok)) break;
        }
        if (kid0 != nullptr) {
            const size_t first = c * chunk_vec;
            const size_t end = first + chunk_vec < nvec ? first + chunk_vec : nvec;
            constexpr int U = 8;
            for (size_t base = first + lane; base < end; base += (size_t)U * 32) {
                uint4 v[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const size_t j = base + (size_t)u * 32;
                    if (j < end) v[u] = ROOT ? ld_stream<2>(local + j) : ld_volatile_v4(local + j);
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const size_t j = base + (size_t)u * 32;
                    if (j < end) st_stream<1>(kid0 + j, v[u]);
                }
                if (kid1 != nullptr) {
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const size_t j = base + (size_t)u * 32;
                        if (j < end) st_stream<1>(kid1 + j, v[u]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) {  // one release for both children, then the flags
                asm volatile("fence.acq_rel.sys;" ::: "memory");
                asm volatile("st.relaxed.sys.global.u32 [%0], %1;" :: "l"(kf0 + c), "r"(epoch) : "memory");
                if (kid1 != nullptr) asm volatile("st.relaxed.sys.global.u32 [%0], %1;" :: "l"(kf1 + c), "r"(epoch) : "memory");
            }
        }
    }
    if (DYN) leave_tickets(lane, (unsigned int)total);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
namespace {

// What a launcher decided; filled instead of launching when the caller only asks for the plan.
struct Plan {
    char text[160];
};

struct Split {
    Edges e;
    uint4 *dstv;
    const uint8_t *src_body;
    size_t nvec;
};

Split split_copy(void *dst, const void *src, size_t bytes) {
    Split sp;
    uint8_t *d = static_cast<uint8_t *>(dst);
    const uint8_t *s = static_cast<const uint8_t *>(src);
    size_t head = (16 - (reinterpret_cast<uintptr_t>(d) & 15)) & 15;
    if (head > bytes) head = bytes;
    const size_t nvec = (bytes - head) / 16;
    const size_t tail = bytes - head - nvec * 16;
    sp.e.dst = d;
    sp.e.src = s;
    sp.e.head = (int)head;
    sp.e.tail = (int)tail;
    sp.e.tail_off = head + nvec * 16;
    sp.dstv = reinterpret_cast<uint4 *>(d + head);
    sp.src_body = s + head;
    sp.nvec = nvec;
    return sp;
}

template <int SW, int U>
int launch_vec_mode(int mode, int grid, int threads, cudaStream_t st, uint4 *dstv, const uint4 *srcv, size_t nvec,
                    int sb8, const Edges &e, int early) {
    const size_t pad = (size_t)tuning().copy_vec_smem_pad;
    if constexpr (SW < 0) {  // the L2-policy modes exist for congruent pointers only
        if (mode == 3) return launch_kernel(copy_vec_kernel<SW, U, 3>, grid, threads, pad, st, dstv, srcv, nvec, sb8, e, early);
        if (mode == 4) return launch_kernel(copy_vec_kernel<SW, U, 4>, grid, threads, pad, st, dstv, srcv, nvec, sb8, e, early);
    }
    switch (mode) {
        case 0: return launch_kernel(copy_vec_kernel<SW, U, 0>, grid, threads, pad, st, dstv, srcv, nvec, sb8, e, early);
        case 1: return launch_kernel(copy_vec_kernel<SW, U, 1>, grid, threads, pad, st, dstv, srcv, nvec, sb8, e, early);
        default: return launch_kernel(copy_vec_kernel<SW, U, 2>, grid, threads, pad, st, dstv, srcv, nvec, sb8, e, early);
    }
}

template <int SW>
int launch_vec_unroll(int unroll, int mode, int grid, int threads, cudaStream_t st, uint4 *dstv, const uint4 *srcv,
                      size_t nvec, int sb8, const Edges &e, int early) {
    switch (unroll) {
        case 1: return launch_vec_mode<SW, 1>(mode, grid, threads, st, dstv, srcv, nvec, sb8, e, early);
        case 2: return launch_vec_mode<SW, 2>(mode, grid, threads, st, dstv, srcv, nvec, sb8, e, early);
        case 8: return launch_vec_mode<SW, 8>(mode, grid, threads, st, dstv, srcv, nvec, sb8, e, early);
        default: return launch_vec_mode<SW, 4>(mode, grid, threads, st, dstv, srcv, nvec, sb8, e, early);
    }
}

int launch_vec(const Split &sp, int ctas, bool small, cudaStream_t st, int early, Plan *plan) {
    const Tuning &tu = tuning();
    // Launch shape.  Measured on B200: one SHORT CTA per tile -- a grid as large as the tile count, scheduled by
    // the hardware as SMs free up -- beats a persistent grid at every size above L2 (7.0 vs 6.65 TB/s at
    // 1 GiB).  Tile: 512 threads x 4 vectors (32 KiB); 128 x 2 measured 0.5-1.5 % less from 96 MiB to 1 GiB once
    // the loads may run ahead of the stream wait.  (Congruent pointers go to the bulk-copy kernel from 96 MiB
    // on, see copy_dispatch.)
    int threads, unroll;
    if (small) {
        threads = 128;
        unroll = 1;
    } else if (tu.copy_vec_threads > 0 && tu.copy_vec_unroll > 0) {
        threads = tu.copy_vec_threads;
        unroll = tu.copy_vec_unroll;
    } else {
        threads = 512;
        unroll = 4;
    }
    if (!small) {
        // mid sizes: shrink the tile until every SM gets work
        const size_t want = (size_t)sm_count() * 2;
        while (unroll > 1 && (sp.nvec / ((size_t)unroll * threads)) < want) unroll >>= 1;
        while (threads > 128 && (sp.nvec / ((size_t)unroll * threads)) < want) threads >>= 1;
    }
    const size_t per_cta = (size_t)unroll * threads;
    size_t need = (sp.nvec + per_cta - 1) / per_cta;
    if (need == 0) need = 1;
    // copy_vec_ctas_sm > 0 (or an explicit `ctas`) caps the grid and makes the CTAs loop (persistent form)
    size_t cap = ctas > 0 ? (size_t)ctas
                 : tu.copy_vec_ctas_sm > 0 ? (size_t)sm_count() * tu.copy_vec_ctas_sm * (512 / threads)
                                           : ((size_t)1 << 30);
    const int grid = (int)(need < cap ? need : cap);

    const uintptr_t sa = reinterpret_cast<uintptr_t>(sp.src_body);
    const int s = (int)(sa & 15);
    const uint4 *srcv = reinterpret_cast<const uint4 *>(sa - s);
    const int sb8 = (s & 3) * 8;
    int mode = tu.copy_cache_mode;
    if (s != 0 && mode > 2) mode = 2;
    if (unroll != 1 && unroll != 2 && unroll != 8) unroll = 4;
    if (plan != nullptr) {
        snprintf(plan->text, sizeof(plan->text), "copy_vec_kernel<%d,%d,%d>, %d CTAs x %d threads, %zu bytes per CTA%s%s",
                 s == 0 ? -1 : (s >> 2), unroll, mode, grid, threads, per_cta * 16, (size_t)grid < need ? ", looping" : "",
                 early ? ", loads before the stream wait" : "");
        return 0;
    }
    if (s == 0) return launch_vec_unroll<-1>(unroll, mode, grid, threads, st, sp.dstv, srcv, sp.nvec, 0, sp.e, early);
    switch (s >> 2) {
        case 0: return launch_vec_unroll<0>(unroll, mode, grid, threads, st, sp.dstv, srcv, sp.nvec, sb8, sp.e, early);
        case 1: return launch_vec_unroll<1>(unroll, mode, grid, threads, st, sp.dstv, srcv, sp.nvec, sb8, sp.e, early);
        case 2: return launch_vec_unroll<2>(unroll, mode, grid, threads, st, sp.dstv, srcv, sp.nvec, sb8, sp.e, early);
        default: return launch_vec_unroll<3>(unroll, mode, grid, threads, st, sp.dstv, srcv, sp.nvec, sb8, sp.e, early);
    }
}


int launch_vec32(void *dst, const void *src, size_t bytes, int ctas, cudaStream_t st) {
    const Tuning &tu = tuning();
    uint8_t *d = static_cast<uint8_t *>(dst);
    const uint8_t *s = static_cast<const uint8_t *>(src);
    size_t head = (32 - (reinterpret_cast<uintptr_t>(d) & 31)) & 31;
    if (head > bytes) head = bytes;
    const size_t n32 = (bytes - head) / 32;
    Edges e;
    e.dst = d;
    e.src = s;
    e.head = (int)head;
    e.tail = (int)(bytes - head - n32 * 32);
    e.tail_off = head + n32 * 32;
    const int threads = tu.copy_vec_threads > 0 ? tu.copy_vec_threads : 512;
    const int unroll = tu.copy_vec_unroll == 2 ? 2 : 4;
    const size_t per_cta = (size_t)unroll * threads;
    size_t need = (n32 + per_cta - 1) / per_cta;
    if (need == 0) need = 1;
    size_t cap = ctas > 0 ? (size_t)ctas : (size_t)sm_count() * (tu.copy_vec_ctas_sm > 0 ? tu.copy_vec_ctas_sm : 1) * (512 / threads);
    const int grid = (int)(need < cap ? need : cap);
    if (unroll == 4) return launch_kernel(copy_vec32_kernel<4>, grid, threads, 0, st, d + head, s + head, n32, e);
    return launch_kernel(copy_vec32_kernel<2>, grid, threads, 0, st, d + head, s + head, n32, e);
}

template <int S, int L>
int launch_tma_cfg(bool hint, int grid, size_t smem, cudaStream_t st, uint8_t *d, const uint8_t *s, size_t body,
                   uint32_t chunk, const Edges &e, int early) {
    const size_t total = smem + (size_t)tuning().tma_smem_pad;
    if (hint) return launch_kernel(copy_tma_kernel<S, L, true>, grid, 32, total, st, d, s, body, chunk, e, early);
    return launch_kernel(copy_tma_kernel<S, L, false>, grid, 32, total, st, d, s, body, chunk, e, early);
}

int launch_tma(const Split &sp, int ctas, cudaStream_t st, int early, Plan *plan) {
    const Tuning &tu = tuning();
    const size_t body = sp.nvec * 16;
    uint32_t chunk = (uint32_t)tu.tma_chunk;
    int S = tu.tma_stages, L = tu.tma_lookahead;
    if (chunk == 0) {
        // One shape for every size (every CTA moves ONE chunk; measured on B200 with the loads issued ahead of the
        // stream wait): a 12 KiB chunk with three stages' worth of shared memory reserved, which caps residency at
        // 6 CTAs per SM.  It is first or second of 50 (chunk, reservation) pairs at 128 MiB, 256 MiB, 512 MiB and
        // 1 GiB (6880 / 6995 / 6987 / 6997 GB/s; 8 KiB x 3: 6862 / 6967 / 6944 / 6967; 32 KiB x 2: 6882 / 6977 /
        // 6961 / 6977; the vector kernel 6766-6820 / 6858-6885 / 6913-6921 / 6949-6951).
        chunk = 12288;
        S = 3;
        L = 2;
    }
    if (chunk < 1024 || chunk > 65536 || (chunk & 127)) return 1;
    const size_t smem = (size_t)S * chunk + 8 * S;
    if (smem > 227 * 1024) return 1;
    const size_t nchunks = (body + chunk - 1) / chunk;
    // tma_ctas_sm == 0: one chunk per CTA (short CTAs, 7.0 TB/s); > 0: persistent ring of that many CTAs per SM
    size_t cap = ctas > 0 ? (size_t)ctas : tu.tma_ctas_sm > 0 ? (size_t)sm_count() * tu.tma_ctas_sm : ((size_t)1 << 30);
    int grid = (int)(nchunks < cap ? (nchunks ? nchunks : 1) : cap);
    uint8_t *d = reinterpret_cast<uint8_t *>(sp.dstv);
    const bool hint = tu.tma_cache_hint != 0;
    if (plan != nullptr) {
        snprintf(plan->text, sizeof(plan->text), "copy_tma_kernel<%d,%d,%d>, %d CTAs x 32 threads, %u-byte bulk copies%s%s", S, L,
                 hint ? 1 : 0, grid, chunk, (size_t)grid < nchunks ? ", persistent ring" : ", one per CTA",
                 early ? ", loads before the stream wait" : "");
        return 0;
    }
#define LCB_TMA_CFG(S_, L_) \
    if (S == S_ && L == L_) return launch_tma_cfg<S_, L_>(hint, grid, smem, st, d, sp.src_body, body, chunk, sp.e, early)
    LCB_TMA_CFG(2, 1);
    LCB_TMA_CFG(3, 2);
    LCB_TMA_CFG(4, 2);
    LCB_TMA_CFG(4, 3);
    LCB_TMA_CFG(6, 3);
    LCB_TMA_CFG(6, 4);
    LCB_TMA_CFG(8, 4);
    LCB_TMA_CFG(8, 6);
    LCB_TMA_CFG(12, 8);
    LCB_TMA_CFG(16, 8);
    LCB_TMA_CFG(16, 12);
#undef LCB_TMA_CFG
    return 1;
}


template <int S, int D>
int launch_tma2_cfg(bool hint, int grid, size_t smem, cudaStream_t st, uint8_t *d, const uint8_t *s, size_t body,
                    uint32_t chunk, const Edges &e) {
    if (hint) return launch_kernel(copy_tma2_kernel<S, D, true>, grid, 64, smem, st, d, s, body, chunk, e);
    return launch_kernel(copy_tma2_kernel<S, D, false>, grid, 64, smem, st, d, s, body, chunk, e);
}

// Phase-grouped copy (LCB_COPY_PHASED).  Not reachable from LCB_COPY_AUTO: see the measurements in the design notes.
int launch_phased(const Split &sp, int ctas, cudaStream_t st) {
    const Tuning &tu = tuning();
    const uint32_t chunk = (uint32_t)tu.phase_chunk;
    const int S = tu.phase_stages;
    if (chunk < 1024 || chunk > 65536 || (chunk & 127)) return 1;
    const size_t smem = (size_t)S * chunk + 8 * (size_t)S;
    if (smem > 227 * 1024) return 1;
    const size_t body = sp.nvec * 16;
    const size_t nchunks = (body + chunk - 1) / chunk;
    const size_t cap = ctas > 0 ? (size_t)ctas : (size_t)sm_count();
    const int grid = (int)(nchunks < cap ? (nchunks ? nchunks : 1) : cap);
    uint8_t *d = reinterpret_cast<uint8_t *>(sp.dstv);
    const unsigned long long phase_ns = (unsigned long long)tu.phase_ns;
    switch (S) {
        case 2: return launch_kernel(copy_phase_kernel<2>, grid, 32, smem, st, d, sp.src_body, body, chunk, phase_ns, sp.e);
        case 3: return launch_kernel(copy_phase_kernel<3>, grid, 32, smem, st, d, sp.src_body, body, chunk, phase_ns, sp.e);
        case 4: return launch_kernel(copy_phase_kernel<4>, grid, 32, smem, st, d, sp.src_body, body, chunk, phase_ns, sp.e);
        case 6: return launch_kernel(copy_phase_kernel<6>, grid, 32, smem, st, d, sp.src_body, body, chunk, phase_ns, sp.e);
        case 12: return launch_kernel(copy_phase_kernel<12>, grid, 32, smem, st, d, sp.src_body, body, chunk, phase_ns, sp.e);
        case 24: return launch_kernel(copy_phase_kernel<24>, grid, 32, smem, st, d, sp.src_body, body, chunk, phase_ns, sp.e);
        default: return 1;
    }
}

int launch_tma2(const Split &sp, int ctas, cudaStream_t st) {
    const Tuning &tu = tuning();
    const uint32_t chunk = (uint32_t)tu.tma2_chunk;
    if (chunk < 1024 || chunk > 65536 || (chunk & 127)) return 1;
    const int S = tu.tma2_stages, D = tu.tma2_depth;
    const size_t smem = (size_t)S * chunk + 16 * S + (size_t)tu.tma_smem_pad;
    if (smem > 227 * 1024) return 1;
    const size_t body = sp.nvec * 16;
    const size_t nchunks = (body + chunk - 1) / chunk;
    const size_t cap = ctas > 0 ? (size_t)ctas : (size_t)sm_count() * (tu.tma_ctas_sm > 0 ? tu.tma_ctas_sm : 1);
    const int grid = (int)(nchunks < cap ? (nchunks ? nchunks : 1) : cap);
    uint8_t *d = reinterpret_cast<uint8_t *>(sp.dstv);
    const bool hint = tu.tma_cache_hint != 0;
#define LCB_TMA2_CFG(S_, D_) \
    if (S == S_ && D == D_) return launch_tma2_cfg<S_, D_>(hint, grid, smem, st, d, sp.src_body, body, chunk, sp.e)
    LCB_TMA2_CFG(4, 1);
    LCB_TMA2_CFG(4, 2);
    LCB_TMA2_CFG(8, 1);
    LCB_TMA2_CFG(8, 2);
    LCB_TMA2_CFG(8, 4);
    LCB_TMA2_CFG(12, 2);
    LCB_TMA2_CFG(12, 4);
    LCB_TMA2_CFG(16, 2);
    LCB_TMA2_CFG(16, 4);
    LCB_TMA2_CFG(16, 8);
    LCB_TMA2_CFG(24, 4);
    LCB_TMA2_CFG(24, 8);
#undef LCB_TMA2_CFG
    return 1;
}

}  // namespace
}  // namespace lcb

namespace lcb {
// Self-test of the give-up path of the bounded wait: waits on a barrier that nothing ever completes, with a
// small try limit, then does exactly what the bulk ring does when a wait runs out (sticky error bit, return).
// Nothing faults and nothing hangs; the context stays usable.
__global__ void wait_timeout_selftest_kernel(uint32_t max_tries) {
    __shared__ uint64_t bar;
    if (threadIdx.x != 0) return;
    mbar_init(smem_addr(&bar), 1);
    mbar_init_fence();
    if (!mbar_wait_bounded(smem_addr(&bar), 0, max_tries)) raise_error(kErrMbarrierTimeout);
}
}  // namespace lcb

extern "C" int lcb_selftest_wait_timeout(unsigned int max_tries, lcbStream stream) {
    if (max_tries == 0 || max_tries > 100000u) return 1;  // keeps the self-test in the millisecond range
    lcb::wait_timeout_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(max_tries);
    return lcb::check_launch();
}

namespace lcb {
// With lazy module loading a kernel is loaded at its first launch; touching the default instantiations here
// moves that cost out of the first copy (the reference loads its copy kernels when a context is created,
// driverapi/src/librecuda.cpp:622).
int preload_copy_kernels() {
    cudaFuncAttributes a;
    cudaError_t e = cudaFuncGetAttributes(&a, copy_vec_kernel<-1, 4, 2>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, copy_vec_kernel<-1, 2, 2>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, copy_vec_kernel<-1, 1, 2>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, copy_vec_kernel<0, 4, 2>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, copy_vec_kernel<1, 4, 2>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, copy_vec_kernel<2, 4, 2>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, copy_vec_kernel<3, 4, 2>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, copy_tma_kernel<2, 1, false>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, copy_tma_kernel<3, 2, false>);
    // kernels that wait for another GPU's kernel must not meet a module load at their first launch
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, ring_bcast_kernel<true>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, ring_bcast_kernel<false>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, ring_bcast_warp_kernel<true, false>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, ring_bcast_warp_kernel<false, false>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, ring_bcast_warp_kernel<true, true>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, ring_bcast_warp_kernel<false, true>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, tree_bcast_kernel<true, false>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, tree_bcast_kernel<false, false>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, tree_bcast_kernel<true, true>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, tree_bcast_kernel<false, true>);
    return (int)e;
}
}  // namespace lcb

namespace lcb {
namespace {
// Shared by the launcher and the plan query, so the description cannot drift from what is launched.
int copy_dispatch(void *dst, const void *src, size_t bytes, int path_and_flags, int ctas, cudaStream_t st, Plan *plan) {
    if (dst == nullptr || src == nullptr || ctas < 0) return 1;
    const int early = (path_and_flags & LCB_COPY_SRC_STABLE) ? 1 : 0;
    int path = path_and_flags & 0xff;
    if ((path_and_flags & ~(0xff | LCB_COPY_SRC_STABLE | LCB_COPY_NO_PDL)) != 0) return 1;
    NoPdlScope no_pdl((path_and_flags & LCB_COPY_NO_PDL) != 0);
    const Split sp = split_copy(dst, src, bytes);
    const bool mutual = ((reinterpret_cast<uintptr_t>(dst) ^ reinterpret_cast<uintptr_t>(src)) & 15) == 0;
    if (path == LCB_COPY_AUTO) {
        const Tuning &tu = tuning();
        if (bytes < 64 * 1024) path = LCB_COPY_SMALL;
        else if (mutual && tu.auto_tma_min_mib >= 0 && bytes >= ((size_t)tu.auto_tma_min_mib << 20)) path = LCB_COPY_TMA;
        else path = LCB_COPY_VEC;
    }
    switch (path) {
        case LCB_COPY_VEC: return launch_vec(sp, ctas, false, st, early, plan);
        case LCB_COPY_SMALL: return launch_vec(sp, ctas, true, st, early, plan);
        case LCB_COPY_TMA:
            if (!mutual) return 1;
            return launch_tma(sp, ctas, st, early, plan);
        case LCB_COPY_TMA2:
            if (!mutual || plan != nullptr) return 1;
            return launch_tma2(sp, ctas, st);
        case LCB_COPY_PHASED:
            if (!mutual || plan != nullptr) return 1;
            return launch_phased(sp, ctas, st);
        case LCB_COPY_VEC32:
            if (((reinterpret_cast<uintptr_t>(dst) ^ reinterpret_cast<uintptr_t>(src)) & 31) != 0 || plan != nullptr) return 1;
            return launch_vec32(dst, src, bytes, ctas, st);
        default: return 1;
    }
}
}  // namespace
}  // namespace lcb

extern "C" int lcb_copy_d2d_ex(void *dst, const void *src, size_t bytes, int path, int ctas, lcbStream stream) {
    if (bytes == 0) return 0;
    return lcb::copy_dispatch(dst, src, bytes, path, ctas, static_cast<cudaStream_t>(stream), nullptr);
}

extern "C" int lcb_copy_d2d(void *dst, const void *src, size_t bytes, lcbStream stream) {
    return lcb_copy_d2d_ex(dst, src, bytes, LCB_COPY_AUTO, 0, stream);
}

extern "C" int lcb_copy_d2d_describe(const void *dst, const void *src, size_t bytes, int path, int ctas, char *text,
                                     size_t text_bytes) {
    if (text == nullptr || text_bytes == 0 || bytes == 0) return 1;
    lcb::Plan plan{};
    const int rc = lcb::copy_dispatch(const_cast<void *>(dst), src, bytes, path, ctas, nullptr, &plan);
    if (rc != 0) return rc;
    snprintf(text, text_bytes, "%s", plan.text);
    return 0;
}

namespace lcb {
namespace {
int launch_alltoall(bool pull, void *const *peer_bufs, void *mine, size_t chunk_bytes, int n_ranks, int rank,
                    lcbStream stream) {
    if (n_ranks < 1 || n_ranks > 16 || rank < 0 || rank >= n_ranks || peer_bufs == nullptr || mine == nullptr) return 1;
    if (chunk_bytes == 0) return 0;
    if ((chunk_bytes & 15) || (reinterpret_cast<uintptr_t>(mine) & 15)) return 1;
    PeerPtrs pp{};
    for (int j = 0; j < n_ranks; ++j) {
        if (peer_bufs[j] == nullptr || (reinterpret_cast<uintptr_t>(peer_bufs[j]) & 15)) return 1;
        pp.buf[j] = static_cast<uint4 *>(peer_bufs[j]);
    }
    const Tuning &tu = tuning();
    const int threads = 512;
    const size_t chunk_vec = chunk_bytes / 16;
    const size_t per_cta = (size_t)4 * threads;
    size_t per_peer = (chunk_vec + per_cta - 1) / per_cta;
    // CTAs per peer: at least half an SM count's worth, whatever the number of peers (measured: 74 per peer is
    // best at 2 GPUs and at 8 -- 694 vs 648 GB/s per GPU with 18 per peer)
    size_t cap = ((size_t)sm_count() * tu.a2a_ctas_sm + n_ranks - 1) / n_ranks;
    if (cap < (size_t)sm_count() / 2) cap = (size_t)sm_count() / 2;
    if (per_peer > cap) per_peer = cap;
    if (per_peer == 0) per_peer = 1;
    const int grid = (int)(per_peer * n_ranks);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint4 *m = static_cast<uint4 *>(mine);
    if (pull) return launch_kernel(alltoall_kernel<4, 2, true>, grid, threads, 0, st, pp, m, chunk_vec, n_ranks, rank);
    return launch_kernel(alltoall_kernel<4, 2, false>, grid, threads, 0, st, pp, m, chunk_vec, n_ranks, rank);
}
}  // namespace
}  // namespace lcb

extern "C" int lcb_alltoall_push(void *const *peer_recv, const void *send, size_t chunk_bytes, int n_ranks, int rank,
                                 lcbStream stream) {
    return lcb::launch_alltoall(false, peer_recv, const_cast<void *>(send), chunk_bytes, n_ranks, rank, stream);
}

extern "C" int lcb_alltoall_pull(void *const *peer_send, void *recv, size_t chunk_bytes, int n_ranks, int rank,
                                 lcbStream stream) {
    return lcb::launch_alltoall(true, peer_send, recv, chunk_bytes, n_ranks, rank, stream);
}

extern "C" int lcb_bcast_ring_hop(const void *local, void *next, const void *flags_in, void *flags_next, size_t bytes,
                                  size_t chunk_bytes, unsigned int epoch, unsigned int timeout_ms, int ctas, lcbStream stream) {
    using namespace lcb;
    if (bytes == 0) return 0;
    if (local == nullptr || epoch == 0 || ctas < 0) return 1;
    if (timeout_ms == 0 || timeout_ms > 10000u) return 1;
    if (chunk_bytes < 4096 || (chunk_bytes & 15) || (bytes & 15)) return 1;
    if ((reinterpret_cast<uintptr_t>(local) | reinterpret_cast<uintptr_t>(next)) & 15) return 1;
    if ((reinterpret_cast<uintptr_t>(flags_in) | reinterpret_cast<uintptr_t>(flags_next)) & 3) return 1;
    if (next != nullptr && flags_next == nullptr) return 1;
    if (next == nullptr && flags_in == nullptr) return 0;  // neither receives nor forwards: nothing to do
    const size_t nvec = bytes / 16, chunk_vec = chunk_bytes / 16;
    const size_t nchunks = (nvec + chunk_vec - 1) / chunk_vec;
    size_t grid = ctas > 0 ? (size_t)ctas : (size_t)sm_count() * (tuning().bcast_ring_warp ? 1 : 2);
    if (grid > nchunks) grid = nchunks;
    NoPdlScope plain(true);  // a kernel that polls must not sit on the SMs before its predecessor on the stream is done
    const unsigned long long timeout_ns = (unsigned long long)timeout_ms * 1000000ull;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint4 *l = static_cast<const uint4 *>(local);
    uint4 *n = static_cast<uint4 *>(next);
    const unsigned int *fi = static_cast<const unsigned int *>(flags_in);
    unsigned int *fn = static_cast<unsigned int *>(flags_next);
    if (tuning().bcast_ring_warp) {  // one chunk per warp: 16 warps per CTA share the chunks
        if (grid * 16 > nchunks) grid = (nchunks + 15) / 16;
        const bool dyn = tuning().bcast_ring_tickets != 0;
        auto kernel = flags_in == nullptr ? (dyn ? ring_bcast_warp_kernel<true, true> : ring_bcast_warp_kernel<true, false>)
                                          : (dyn ? ring_bcast_warp_kernel<false, true> : ring_bcast_warp_kernel<false, false>);
        return launch_kernel(kernel, (unsigned)grid, 512, 0, st, l, n, fi, fn, nvec, chunk_vec, epoch, timeout_ns);
    }
    if (flags_in == nullptr) return launch_kernel(ring_bcast_kernel<true>, (unsigned)grid, 512, 0, st, l, n, fi, fn, nvec, chunk_vec, epoch, timeout_ns);
    return launch_kernel(ring_bcast_kernel<false>, (unsigned)grid, 512, 0, st, l, n, fi, fn, nvec, chunk_vec, epoch, timeout_ns);
}

extern "C" int lcb_bcast_tree_plan(int n_ranks, int root, int rank, int *parents, int *children) {
    if (n_ranks < 2 || n_ranks > 64 || root < 0 || root >= n_ranks || rank < 0 || rank >= n_ranks) return 1;
    if (parents == nullptr || children == nullptr) return 1;
    const int m = n_ranks - 1;  // the non-root members: p(i) = root + 1 + i in heap order for the first tree,
    auto p = [&](int i) { return (root + 1 + i) % n_ranks; };  // q(i) = p(m - 1 - i) for the second
    for (int k = 0; k < 4; ++k) children[k] = -1;
    if (rank == root) {
        parents[0] = parents[1] = -1;
        children[0] = p(0);
        children[2] = p(m - 1);
        return 0;
    }
    const int i = (rank - root - 1 + n_ranks) % n_ranks, j = m - 1 - i;
    parents[0] = i == 0 ? root : p((i - 1) / 2);
    if (2 * i + 1 < m) children[0] = p(2 * i + 1);
    if (2 * i + 2 < m) children[1] = p(2 * i + 2);
    parents[1] = j == 0 ? root : p(m - 1 - (j - 1) / 2);
    if (2 * j + 1 < m) children[2] = p(m - 1 - (2 * j + 1));
    if (2 * j + 2 < m) children[3] = p(m - 1 - (2 * j + 2));
    return 0;
}

extern "C" int lcb_bcast_tree_node(const void *local, const void *flags_in, void *const *children, void *const *children_flags,
                                   size_t bytes, size_t chunk_bytes, size_t split_chunk, unsigned int epoch,
                                   unsigned int timeout_ms, int ctas, lcbStream stream) {
    using namespace lcb;
    if (bytes == 0) return 0;
    if (local == nullptr || children == nullptr || children_flags == nullptr || epoch == 0 || ctas < 0) return 1;
    if (timeout_ms == 0 || timeout_ms > 10000u) return 1;
    if (chunk_bytes < 4096 || (chunk_bytes & 15) || (bytes & 15)) return 1;
    if ((reinterpret_cast<uintptr_t>(local) & 15) || (reinterpret_cast<uintptr_t>(flags_in) & 3)) return 1;
    const size_t nvec = bytes / 16, chunk_vec = chunk_bytes / 16;
    const size_t nchunks = (nvec + chunk_vec - 1) / chunk_vec;
    if (split_chunk > nchunks) return 1;
    TreeArgs a{};
    bool forwards[2] = {false, false};
    for (int r = 0; r < 2; ++r) {
        a.role[r].c_lo = r == 0 ? 0 : split_chunk;
        a.role[r].c_hi = r == 0 ? split_chunk : nchunks;
        int filled = 0;
        for (int k = 0; k < 2; ++k) {  // children are packed to the front: the kernel tests child[0] first
            void *c = children[2 * r + k], *f = children_flags[2 * r + k];
            if (c == nullptr) continue;
            if (f == nullptr || (reinterpret_cast<uintptr_t>(c) & 15) || (reinterpret_cast<uintptr_t>(f) & 3)) return 1;
            a.role[r].child[filled] = static_cast<uint4 *>(c);
            a.role[r].child_flags[filled] = static_cast<unsigned int *>(f);
            ++filled;
        }
        forwards[r] = filled > 0;
    }
    if (flags_in == nullptr && !forwards[0] && !forwards[1]) return 0;  // a root without children
    size_t grid = ctas > 0 ? (size_t)ctas : (size_t)sm_count();
    if (grid * 16 > nchunks + 16) grid = (nchunks + 16) / 16;
    if (grid < 2) grid = 2;  // at least a CTA's worth of warps per role
    const size_t total = grid * 16;
    // a role that only waits needs few warps (a poll costs about a microsecond, a chunk arrives every 50 ns)
    size_t waiters = total / 4 < 128 ? total / 4 : 128;
    if (waiters < 16) waiters = 16;
    size_t warps0 = total / 2;
    if (forwards[0] && !forwards[1]) warps0 = total - waiters;
    if (!forwards[0] && forwards[1]) warps0 = waiters;
    a.warps0 = (unsigned int)warps0;
    NoPdlScope plain(true);  // a kernel that polls must not sit on the SMs before its predecessor on the stream is done
    const unsigned long long timeout_ns = (unsigned long long)timeout_ms * 1000000ull;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint4 *l = static_cast<const uint4 *>(local);
    const unsigned int *fi = static_cast<const unsigned int *>(flags_in);
    const bool dyn = tuning().bcast_ring_tickets != 0;
    auto kernel = flags_in == nullptr ? (dyn ? tree_bcast_kernel<true, true> : tree_bcast_kernel<true, false>)
                                      : (dyn ? tree_bcast_kernel<false, true> : tree_bcast_kernel<false, false>);
    return launch_kernel(kernel, (unsigned)grid, 512, 0, st, l, fi, a, nvec, chunk_vec, epoch, timeout_ns);
}

extern "C" int lcb_flag_post(void *flag, unsigned int value, lcbStream stream) {
    if (flag == nullptr || (reinterpret_cast<uintptr_t>(flag) & 3)) return 1;
    lcb::NoPdlScope plain(true);  // must not start before the work it announces has finished
    return lcb::launch_kernel(lcb::flag_post_kernel, 1, 1, 0, static_cast<cudaStream_t>(stream), static_cast<unsigned int *>(flag), value);
}

extern "C" int lcb_flag_wait(const void *flag, unsigned int value, unsigned int timeout_ms, lcbStream stream) {
    if (flag == nullptr || (reinterpret_cast<uintptr_t>(flag) & 3)) return 1;
    if (timeout_ms == 0 || timeout_ms > 10000u) return 1;  // a wait is always bounded, and by seconds at most
    lcb::NoPdlScope plain(true);
    return lcb::launch_kernel(lcb::flag_wait_kernel, 1, 1, 0, static_cast<cudaStream_t>(stream), static_cast<const unsigned int *>(flag),
                              value, (unsigned long long)timeout_ms * 1000000ull);
}

extern "C" int lcb_alltoall_engines_step(int n_ranks, int rank, int step, int *dest, int *wait_slot, int *wait_previous_call,
                                         int *post_rank, int *post_slot) {
    if (n_ranks < 1 || n_ranks > 16 || rank < 0 || rank >= n_ranks || step < 1 || step >= n_ranks) return 1;
    if (dest == nullptr || wait_slot == nullptr || wait_previous_call == nullptr || post_rank == nullptr || post_slot == nullptr) return 1;
    const int n = n_ranks;
    *dest = (rank + step) % n;
    *wait_slot = -1;
    *wait_previous_call = 0;
    *post_rank = -1;
    *post_slot = -1;
    if (n <= 2) return 0;  // one peer: nothing to keep in step
    // GPU `dest` must be free of its previous sender: rank+1 at the step before, or -- for the first step -- rank+2
    // at the last step of the call before this one
    if (step > 1) {
        *wait_slot = step - 1;
    } else {
        *wait_slot = n - 1;
        *wait_previous_call = 1;
    }
    // who waits for THIS copy: rank-1 (at its next step) or, after the last step, rank-2 (at the next call's first)
    const int back = step + 1 < n ? 1 : 2;
    *post_rank = (rank - back + 2 * n) % n;
    *post_slot = step;
    return 0;
}

extern "C" int lcb_alltoall_engines(void *const *peer_recv, const void *send, size_t chunk_bytes, int n_ranks, int rank,
                                    void *flags, void *const *peer_flags, unsigned int epoch, unsigned int timeout_ms,
                                    lcbStream stream, lcbStream local_stream) {
    if (n_ranks < 1 || n_ranks > 16 || rank < 0 || rank >= n_ranks || peer_recv == nullptr || send == nullptr) return 1;
    if (n_ranks > 2 && (flags == nullptr || peer_flags == nullptr || epoch == 0)) return 1;
    if (chunk_bytes == 0) return 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint8_t *s = static_cast<const uint8_t *>(send);
    unsigned int *mine = static_cast<unsigned int *>(flags);
    const int n = n_ranks;
    // the chunk that stays on this GPU: the copy kernel, on the second stream if one was given
    int rc = lcb_copy_d2d(static_cast<uint8_t *>(peer_recv[rank]) + (size_t)rank * chunk_bytes, s + (size_t)rank * chunk_bytes,
                          chunk_bytes, local_stream != nullptr ? local_stream : stream);
    if (rc != 0) return rc;
    if (timeout_ms == 0 || timeout_ms > 10000u) return 1;
    unsigned int *owed = nullptr;  // the post that announces the copy just issued; goes out with the next wait
    for (int step = 1; step < n; ++step) {
        int j, wait_slot, wait_prev, post_rank, post_slot;
        rc = lcb_alltoall_engines_step(n, rank, step, &j, &wait_slot, &wait_prev, &post_rank, &post_slot);
        if (rc != 0) return rc;
        const bool wait = wait_slot >= 0 && !(wait_prev && epoch == 1);  // the very first call has no call before it
        const unsigned int awaited = wait_prev ? epoch - 1 : epoch;
        if (owed != nullptr && wait) {
            lcb::NoPdlScope plain(true);
            rc = lcb::launch_kernel(lcb::flag_post_wait_kernel, 1, 1, 0, st, owed, epoch, static_cast<const unsigned int *>(mine + wait_slot),
                                    awaited, (unsigned long long)timeout_ms * 1000000ull);
        } else {
            if (owed != nullptr) rc = lcb_flag_post(owed, epoch, stream);
            if (rc == 0 && wait) rc = lcb_flag_wait(mine + wait_slot, awaited, timeout_ms, stream);
        }
        if (rc != 0) return rc;
        owed = nullptr;
        cudaError_t err = cudaMemcpyAsync(static_cast<uint8_t *>(peer_recv[j]) + (size_t)rank * chunk_bytes, s + (size_t)j * chunk_bytes,
                                          chunk_bytes, cudaMemcpyDefault, st);
        if (err != cudaSuccess) return (int)err;
        if (post_rank >= 0) {
            unsigned int *theirs = static_cast<unsigned int *>(peer_flags[post_rank]);
            if (theirs == nullptr) return 1;
            owed = theirs + post_slot;
        }
    }
    if (owed != nullptr) rc = lcb_flag_post(owed, epoch, stream);
    return rc;
}

namespace lcb {
namespace {
unsigned int *g_mirror_host[64] = {};  // per device ordinal: the host side of the mirror word
}

// Gives the current device its host-mapped mirror word (once per device).  Called from lcb_preload.
int setup_error_mirror() {
    int dev = -1;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return (int)err;
    if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    if (g_mirror_host[dev] != nullptr) return 0;
    unsigned int *h = nullptr, *d = nullptr;
    err = cudaHostAlloc(reinterpret_cast<void **>(&h), sizeof(unsigned int), cudaHostAllocMapped | cudaHostAllocPortable);
    if (err != cudaSuccess) return (int)err;
    *h = 0;
    err = cudaHostGetDevicePointer(reinterpret_cast<void **>(&d), h, 0);
    if (err == cudaSuccess) err = cudaMemcpyToSymbol(g_error_mirror, &d, sizeof(d));
    if (err != cudaSuccess) {
        (void)cudaFreeHost(h);
        return (int)err;
    }
    g_mirror_host[dev] = h;
    return 0;
}
}  // namespace lcb

extern "C" int lcb_device_error_peek(unsigned int *out) {
    if (out == nullptr) return 1;
    int dev = -1;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return (int)err;
    if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    const volatile unsigned int *h = lcb::g_mirror_host[dev];
    *out = h ? *h : 0u;
    return 0;
}

extern "C" int lcb_device_error_word(unsigned int *out) {
    if (out == nullptr) return 1;
    cudaError_t err = cudaDeviceSynchronize();
    if (err != cudaSuccess) return (int)err;
    unsigned int w = 0;
    err = cudaMemcpyFromSymbol(&w, lcb::g_error_word, sizeof(w));
    if (err != cudaSuccess) return (int)err;
    if (w) {
        unsigned int zero = 0;
        err = cudaMemcpyToSymbol(lcb::g_error_word, &zero, sizeof(zero));
        if (err != cudaSuccess) return (int)err;
    }
    int dev = -1;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64 && lcb::g_mirror_host[dev] != nullptr)
        *lcb::g_mirror_host[dev] = 0;
    *out = w;
    return 0;
}

