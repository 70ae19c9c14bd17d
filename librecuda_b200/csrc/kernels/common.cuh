// Shared device helpers for the sm_100a data-movement kernels: streaming vector accesses, the
// non-multicast bulk-copy (TMA) primitives with bounded mbarrier waits, and launch plumbing.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace lcb {

// Bit 0 of the sticky per-device error word (defined beside the bulk-copy ring that sets it):
// an mbarrier wait gave up.
constexpr unsigned int kErrMbarrierTimeout = 1u;
// Bit 1: a wait for a flag that another GPU posts gave up.
constexpr unsigned int kErrFlagTimeout = 2u;

// Tunables reachable through lcb_tune() (for sweeps; the defaults are the shipped configuration).
struct Tuning {
    int copy_vec_threads;   // threads per CTA of the vector copy kernel (0 with unroll 0: chosen by size)
    int copy_vec_unroll;    // 16-byte vectors in flight per thread
    int copy_vec_ctas_sm;   // 0: one short CTA per tile; > 0: persistent grid of this many CTAs per SM
    int copy_cache_mode;    // 0: ld.cs/st.cs   1: default caching   2: L1::no_allocate
    int tma_chunk;          // bytes per bulk copy; 0: chunk, stages and lookahead chosen by the copy's size
    int tma_stages;         // ring depth
    int tma_lookahead;      // loads in flight ahead of the store
    int tma_ctas_sm;        // 0: one chunk per CTA; > 0: persistent ring, this many CTAs per SM
    int tma_cache_hint;     // 0: none  1: evict_first policy on loads and stores
    int auto_tma_min_mib;   // LCB_COPY_AUTO uses the bulk ring from this many MiB on (congruent pointers only; -1 never)
    int memset_path;        // 0 auto, 1 vector, 2 bulk
    int memset_unroll;
    int memset_threads;
    int memset_ctas_sm;
    int memset_chunk;        // bytes per bulk store of the bulk memset
    int memset_issuers;      // warps per CTA issuing bulk stores
    int memset_bulk_ctas_sm; // CTAs per SM of the bulk memset
    int memset_cache_hint;   // evict_first policy on the bulk stores
    int pdl;                 // 1: launch with programmatic stream serialization (kernel prologues overlap the
                             //    tail of the previous kernel on the stream)
    int copy_vec_smem_pad;   // extra dynamic shared memory per CTA of the vector copy (caps CTAs per SM)
    int tma_smem_pad;        // same for the bulk ring
    int memset_smem_pad;     // same for the vector memset
    int fill_ctas_sm;        // CTAs per SM worth of grid for the index fill (write-only: one short CTA per tile is best)
    int axpb_ctas_sm;        // same for the vector form of y = a*x + b
    int a2a_ctas_sm;         // grid cap of the all-to-all kernel in CTAs per SM, all peers together (large: one short CTA per tile, 709 vs 692 GB/s)
    int tma2_depth;          // two-issuer ring: store groups that may still be reading shared memory
    int tma2_stages;         // two-issuer ring: stages
    int tma2_chunk;          // two-issuer ring: bytes per bulk copy
    int peer_copy_engine;    // libreCuMemCpy / libreCuMemcpyPeer between two GPUs use the copy engines from this many MiB up; 0 = never
    int bcast_piece_mib;     // own broadcast: MiB per pipelined piece
    int bcast_pull_ctas;     // own broadcast: CTAs of the kernel that pulls from the root (it must not fill the GPU)
    int bcast_engine_piece_mib;  // copy-engine chain broadcast: MiB per piece, 0 = chosen from the size and the number of GPUs
    int phase_chunk;             // phase-grouped copy: bytes per bulk copy
    int phase_stages;            // phase-grouped copy: bulk copies per CTA and phase (2, 3, 4, 6, 12 or 24)
    int phase_ns;                // phase-grouped copy: length of a load / store time slice in ns (0: no slicing)
    int bcast_ring_chunk_kib;    // ring-of-kernels broadcast: KiB per chunk (one flag word each); 0: 8 per warp, 128 per CTA
    int bcast_ring_ctas;         // ring-of-kernels broadcast: CTAs per GPU (0: one per SM with a chunk per warp, two with a chunk per CTA)
    int bcast_mc_piece_mib;      // multicast broadcast: MiB per piece
    int bcast_mc_slots;          // multicast broadcast: pieces in the staging ring of every GPU
    int bcast_mc_ctas;           // multicast broadcast: looping CTAs of the root's store kernel (0: one short CTA per tile)
    int bcast_ring_warp;         // ring-of-kernels broadcast: 1 = one chunk (and flag) per warp, 0 = per CTA
    int bcast_ring_tickets;      // ring / tree broadcast, chunk per warp: 1 = chunks handed out by ticket, 0 = by a fixed stride
};
Tuning &tuning();

int preload_copy_kernels();  // force-load the default copy / fill kernels on the current device
int preload_fill_kernels();
int setup_error_mirror();    // host-mapped mirror of the sticky error word for the current device
int sm_count();            // SMs of the current device (cached per device)
int check_launch();        // cudaGetLastError() as int

// ---------------------------------------------------------------------------------------------
// launch helper and programmatic dependent launch
// ---------------------------------------------------------------------------------------------
// Kernels call pdl_launch_dependents() first thing and pdl_wait() before their first global access.  When
// launched with the programmatic-serialization attribute, the CTAs of the NEXT kernel on the stream become
// resident while this one is still running and start the moment it has completed and flushed; without the
// attribute both instructions do nothing.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Launches made by this thread while a NoPdlScope lives go without the programmatic-serialization attribute
// (LCB_COPY_NO_PDL): for callers that run two lanes on one GPU and do not want parked CTAs of a dependent
// kernel to hold SM slots.  Thread-local, so another thread's launches are unaffected.
inline int &no_pdl_depth() {
    static thread_local int depth = 0;
    return depth;
}
struct NoPdlScope {
    bool on;
    explicit NoPdlScope(bool enable) : on(enable) {
        if (on) ++no_pdl_depth();
    }
    ~NoPdlScope() {
        if (on) --no_pdl_depth();
    }
};

template <typename... KArgs, typename... Args>
inline int launch_kernel(void (*kernel)(KArgs...), unsigned grid, unsigned block, size_t smem, cudaStream_t st,
                         Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(block, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    if (tuning().pdl && no_pdl_depth() == 0) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---------------------------------------------------------------------------------------------
// streaming 16-byte accesses
// ---------------------------------------------------------------------------------------------
// MODE 0: .cs both ways   1: default caching   2: L1::no_allocate both ways
//      3: loads as 2, stores with an L2 evict_first policy   4: loads and stores with that policy
// (`pol` is only read by modes 3 and 4: the value of policy_evict_first(), created once per thread)
template <int MODE>
__device__ __forceinline__ uint4 ld_stream(const uint4 *p, uint64_t pol = 0) {
    uint4 v;
    if (MODE == 0) {
        asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    } else if (MODE == 1) {
        asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    } else if (MODE == 4) {
        asm volatile("ld.global.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p), "l"(pol));
    } else {
        asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    }
    return v;
}

template <int MODE>
__device__ __forceinline__ void st_stream(uint4 *p, uint4 v, uint64_t pol = 0) {
    if (MODE == 0) {
        asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};"
                     :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
    } else if (MODE == 1) {
        asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};"
                     :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
    } else if (MODE >= 3) {
        asm volatile("st.global.L1::no_allocate.L2::cache_hint.v4.u32 [%0], {%1,%2,%3,%4}, %5;"
                     :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "l"(pol) : "memory");
    } else {
        asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};"
                     :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// bulk-copy (TMA, untiled) primitives.  Only the non-multicast forms are used anywhere in this library.
// Both addresses of a bulk copy are 16-byte aligned and the size is a multiple of 16.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}

// Bounded wait for the phase with parity `parity`.  Returns false when it gives up.
constexpr uint32_t kMbarMaxTries = 1u << 22;  // each try may itself suspend for a hardware-chosen time
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint32_t max_tries = kMbarMaxTries) {
    for (uint32_t i = 0; i < max_tries; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if (i > 4096) __nanosleep(64);
    }
    return false;
}

template <bool HINT>
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void *src, uint32_t bytes, uint32_t bar,
                                         uint64_t policy) {
    if (HINT) {
        asm volatile(
            "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
            :: "r"(dst_smem), "l"(src), "r"(bytes), "r"(bar), "l"(policy) : "memory");
    } else {
        asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     :: "r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
    }
}

template <bool HINT>
__device__ __forceinline__ void bulk_s2g(void *dst, uint32_t src_smem, uint32_t bytes, uint64_t policy) {
    if (HINT) {
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group.L2::cache_hint [%0], [%1], %2, %3;"
                     :: "l"(dst), "r"(src_smem), "r"(bytes), "l"(policy) : "memory");
    } else {
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                     :: "l"(dst), "r"(src_smem), "r"(bytes) : "memory");
    }
}

__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

template <int N>
__device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" :: "n"(N) : "memory");
}

__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

__device__ __forceinline__ void fence_generic_to_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// splitmix64 finaliser; shared by the seeded generator and the checksum.
__host__ __device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
constexpr uint64_t kGolden = 0x9E3779B97F4A7C15ull;

}  // namespace lcb
