/* lcb200_kernels.h -- thin C-ABI layer over the hand-written sm_100a data-movement kernels.
 *
 * This is the boundary a binding (cgo / JNI / ctypes / the C++ host layer of this library) talks to:
 * `extern "C"`, plain pointers and sizes, a CUDA stream passed as an opaque pointer.  Every launcher
 * enqueues on `stream` (NULL = the legacy default stream) of the device that is current in the
 * calling thread and returns without waiting.  Return value: 0 on success, otherwise a positive
 * `cudaError_t` value (1 = invalid value for rejected arguments).
 *
 * "ref" lines name the reference code (project-relative path:line) each entry point replaces.
 */
#ifndef LCB200_KERNELS_H
#define LCB200_KERNELS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *lcbStream; /* cudaStream_t / CUstream */

/* Copy-path selector for lcb_copy_d2d_ex (lcb_copy_d2d always uses LCB_COPY_AUTO). */
enum lcbCopyPath {
    LCB_COPY_AUTO = 0,  /* pick by size and alignment                                             */
    LCB_COPY_VEC = 1,   /* 16-byte vector loads+stores; src realigned by warp shuffle if needed   */
    LCB_COPY_TMA = 2,   /* cp.async.bulk global->smem->global; needs (src-dst) % 16 == 0            */
    LCB_COPY_SMALL = 3, /* single small CTA wave, latency path                                     */
    LCB_COPY_VEC32 = 4, /* 32-byte vector loads+stores; needs (src-dst) % 32 == 0                   */
    LCB_COPY_TMA2 = 5,  /* bulk ring with separate load- and store-issuing threads; (src-dst) % 16 == 0 */
    LCB_COPY_PHASED = 6 /* bulk copies with all SMs loading and storing in alternating time slices; (src-dst) % 16 == 0 */
};
/* Flag that may be OR'ed into the `path` argument of lcb_copy_d2d_ex (LCB_COPY_AUTO, _VEC, _SMALL, _TMA):
 * the caller vouches that no work submitted earlier to `stream` and possibly still running writes the
 * SOURCE range.  The kernel then issues its first loads while the previous kernel on the stream is still
 * draining and only holds its stores back until that kernel has finished.  Without the flag loads wait too.
 * The libreCu* layer sets it by itself from the command list of a stream. */
#define LCB_COPY_SRC_STABLE 0x100
/* Flag for the same argument: launch this copy without programmatic dependent launch, i.e. its CTAs are not
 * made resident while the previous kernel on the stream still runs.  For callers that drive two streams on
 * one GPU whose kernels would otherwise take SM slots from each other while they wait. */
#define LCB_COPY_NO_PDL 0x200

/* Device-to-device copy of `bytes` bytes, any alignment, any size (64-bit offsets).  Buffers must not
 * overlap.  One launch does head, body and tail.
 * ref: memcpyD2D, driverapi/src/memcopy.cpp:77-158 (dispatcher) and memcpyKernelHighBW /
 * memcpyKernelLowLatency / memcpyKernelTrailing, driverapi/kernels/memcpy/memcpy.cu:5-27. */
int lcb_copy_d2d(void *dst, const void *src, size_t bytes, lcbStream stream);

/* Same copy with an explicit path and grid (ctas = 0: the default grid, one short CTA per tile; ctas > 0:
 * exactly that many CTAs, looping over the tiles).  An
 * infeasible request (LCB_COPY_TMA with mutually misaligned pointers) returns 1. */
int lcb_copy_d2d_ex(void *dst, const void *src, size_t bytes, int path, int ctas, lcbStream stream);

/* Writes into `text` (NUL-terminated, at most text_bytes) which kernel, template arguments, grid and CTA
 * size lcb_copy_d2d_ex would launch for exactly these arguments on the current device, without launching
 * anything.  Returns 0, or 1 where lcb_copy_d2d_ex would refuse the request.
 * ref: the size classes of the reference's dispatcher, driverapi/src/memcopy.cpp:82-107. */
int lcb_copy_d2d_describe(const void *dst, const void *src, size_t bytes, int path, int ctas, char *text,
                          size_t text_bytes);

/* Fill `count` elements of 1, 2 or 4 bytes with `value` (low bytes used).  dst must be aligned to the
 * element size.  ref: none -- the reference has no memset (driverapi/include/librecuda.h:37-114);
 * semantics are those of cuMemsetD8/D16/D32Async. */
int lcb_memset_d8(void *dst, unsigned char value, size_t count, lcbStream stream);
int lcb_memset_d16(void *dst, unsigned short value, size_t count, lcbStream stream);
int lcb_memset_d32(void *dst, unsigned int value, size_t count, lcbStream stream);
/* path: 0 auto, 1 vector stores, 2 bulk (TMA) stores replayed from one shared-memory tile. */
int lcb_memset_ex(void *dst, unsigned int value, int elem_bytes, size_t count, int path, int ctas, lcbStream stream);

/* dst[i] = (float)i for i in [0, count), round-to-nearest-even.
 * ref: grid-indexed fill fixture tests/indexing/write_float.cu:1-4 (+ host check
 * tests/indexing/main.cpp:82-114), generalised from the constant 1.0f to the element index. */
int lcb_index_fill_f32(float *dst, size_t count, lcbStream stream);

/* y[i] = a * x[i] + b (single rounding of a*x followed by the add is NOT fused: computed as
 * __fadd_rn(__fmul_rn(a, x), b) so a host loop compiled without FMA contraction matches bit for bit).
 * ref: the kernel stage between HtoD and DtoH in the reference's stream tests
 * (tests/async_kernels/write_float.cu:1-9 is the reference's stand-in compute kernel). */
int lcb_axpb_f32(float *y, const float *x, float a, float b, size_t count, lcbStream stream);

/* One rank's half of an all-to-all over peer-mapped buffers, fused into one kernel: for every j in
 * [0, n_ranks) chunk j of `send` (chunk_bytes each) is stored to peer_recv[j] + rank * chunk_bytes.
 * All pointers 16-byte aligned, chunk_bytes a multiple of 16.  peer_recv is a HOST array of n_ranks
 * device pointers (n_ranks <= 16).  ref: none (the reference is single-GPU, librecuda.cpp:61). */
int lcb_alltoall_push(void *const *peer_recv, const void *send, size_t chunk_bytes, int n_ranks, int rank,
                      lcbStream stream);
/* The same exchange by remote LOADS: for every j, chunk `rank` of peer_send[j] (peer j's send buffer) is
 * copied to recv + j * chunk_bytes.  peer_send is a HOST array of n_ranks device pointers.  On NVLink 5
 * remote loads win when the links are busy in one direction only (786 vs 716 GB/s per GPU measured); when all
 * ranks exchange at once the push form is faster (704 vs 665).  The caller makes sure every peer's send buffer
 * is ready before the launch and stays untouched until all ranks are done. */
int lcb_alltoall_pull(void *const *peer_send, void *recv, size_t chunk_bytes, int n_ranks, int rank,
                      lcbStream stream);

/* One rank's half of an all-to-all on the COPY ENGINES, for ranks that live in different processes (one per
 * GPU): n_ranks - 1 peer copies of chunk_bytes, rank r sending chunk (r + s) mod n to rank (r + s) mod n at step
 * s, plus the local chunk by the copy kernel (on local_stream if it is not NULL, so that it runs beside the
 * engine copies).  Engine copies only reach their rate (about 775 GB/s per direction against 707 for SM-issued
 * stores) when every GPU has exactly ONE sender at a time, so the ranks keep in lock-step through flags in
 * each other's memory: after a copy the sender posts `epoch` into a flag word of the rank that needs that
 * receiver next, and that rank's copy waits for it with a one-thread kernel.  The wait is bounded by timeout_ms
 * (1..10000); when it runs out the kernel raises bit 1 of the sticky error word (lcb_device_error_word) and
 * the copies go on unsynchronised.
 *   peer_recv[j]   rank j's receive buffer (n_ranks * chunk_bytes), mapped into this process;
 *   flags          this rank's flag words: n_ranks unsigned ints, zero before the first call;
 *   peer_flags[j]  rank j's flag words mapped into this process (HOST array of n_ranks device pointers);
 *   epoch          1, 2, 3 ... : the same value on every rank for the same call, increased by one per call.
 * With n_ranks <= 2 no flags are needed (they may be NULL).  ref: none (single-GPU reference, librecuda.cpp:61). */
int lcb_alltoall_engines(void *const *peer_recv, const void *send, size_t chunk_bytes, int n_ranks, int rank,
                         void *flags, void *const *peer_flags, unsigned int epoch, unsigned int timeout_ms,
                         lcbStream stream, lcbStream local_stream);
/* The schedule of that exchange as a pure function (no GPU): for `step` in [1, n_ranks) of `rank` it gives the
 * destination rank of the copy, the own flag word to wait on first (-1: none) and whether the value awaited is
 * the previous call's epoch, and the rank and flag word to post to afterwards (-1: none).  lcb_alltoall_engines
 * follows exactly this; the tests replay it with arbitrary copy durations to show that no GPU ever has two
 * senders and that nobody waits for ever. */
int lcb_alltoall_engines_step(int n_ranks, int rank, int step, int *dest, int *wait_slot, int *wait_previous_call,
                              int *post_rank, int *post_slot);
/* The two flag primitives it is built from.  lcb_flag_post: once everything earlier on `stream` has finished,
 * store `value` to the 4-byte aligned word `flag` (any memory this GPU may write, a peer's included).
 * lcb_flag_wait: work later on `stream` starts when the word has reached `value` (counters only grow), or
 * after timeout_ms (1..10000) with bit 1 of the sticky error word raised. */
int lcb_flag_post(void *flag, unsigned int value, lcbStream stream);
int lcb_flag_wait(const void *flag, unsigned int value, unsigned int timeout_ms, lcbStream stream);

/* One GPU's part of a ring broadcast root -> d1 -> d2 -> ..., fused into one kernel: for every chunk of
 * chunk_bytes it waits until flags_in[chunk] has reached `epoch` (skipped on the root: flags_in NULL), copies
 * the chunk from `local` into `next` with remote stores, and stores `epoch` into flags_next[chunk] (skipped on
 * the last GPU: next NULL, which then only waits for its chunks).  The GPUs of a chain run one such kernel each
 * at the same time; flags_* are arrays of one unsigned int per chunk in the memory of the GPU that waits on
 * them, zero before the first use, epochs grow from call to call.  `bytes` and both buffers are multiples of
 * 16; a wait is bounded by timeout_ms (1..10000: then bit 1 of the sticky error word, and the kernel returns).
 * ctas = 0: one CTA per SM (two in the chunk-per-CTA form).  A chunk is the work of one warp (tunable "bcast_ring_warp" = 1, the default;
 * chunks of 8-32 KiB, handed to the warps by ticket unless "bcast_ring_tickets" = 0) or of one CTA (= 0; chunks
 * from 128 KiB); every GPU of a chain must run the same form.  One broadcast at a time per GPU: the ticket
 * counters and the abort word are per GPU.
 * ref: none (single-GPU reference, librecuda.cpp:61). */
int lcb_bcast_ring_hop(const void *local, void *next, const void *flags_in, void *flags_next, size_t bytes, size_t chunk_bytes,
                       unsigned int epoch, unsigned int timeout_ms, int ctas, lcbStream stream);

/* Broadcast down two complementary binary trees, one per half of the buffer, instead of one chain: the depth is
 * 1 + log2(n_ranks - 1) hops instead of n_ranks - 1, every GPU still receives each byte once and sends at most one
 * buffer's worth.  lcb_bcast_tree_plan is the topology as a pure function (no GPU): for `rank` it gives
 * parents[0..1] (the rank it receives the first / second half from; -1 on the root) and children[0..3]
 * (children[0..1]: where it forwards the first half, children[2..3]: the second; -1 = none).  The non-root ranks
 * in the order root+1, root+2, ... form a heap for the first half and the same heap in reverse order for the
 * second, so a rank with children in one tree has none in the other.
 * lcb_bcast_tree_node is one GPU's kernel: for every chunk of chunk_bytes (one warp each, as in the ring's
 * chunk-per-warp form) it waits for flags_in[chunk] (skipped on the root: flags_in NULL), stores the chunk into
 * the children's buffers and posts children_flags[k][chunk].  children / children_flags are arrays of four
 * pointers laid out like the plan's children (NULL = none; whole buffers and whole flag arrays, indexed like
 * `local` and flags_in); chunks below split_chunk belong to the first half.  Alignment, epochs, timeout and the
 * error word are those of lcb_bcast_ring_hop.  ctas = 0: one CTA per SM.  ref: none (single-GPU reference). */
int lcb_bcast_tree_plan(int n_ranks, int root, int rank, int *parents, int *children);
int lcb_bcast_tree_node(const void *local, const void *flags_in, void *const *children, void *const *children_flags,
                        size_t bytes, size_t chunk_bytes, size_t split_chunk, unsigned int epoch, unsigned int timeout_ms,
                        int ctas, lcbStream stream);

/* Copies `bytes` bytes (a multiple of 16; both addresses 16-byte aligned) from ordinary device memory to a
 * MULTICAST address with multimem stores: NVSwitch writes the data into the memory of every GPU bound to the
 * multicast object at that offset, while it leaves the storing GPU only once.  mc_dst must be an address of a
 * multicast mapping (cuMulticastCreate / cuMemMap) that this GPU may access; only stores are issued on it.
 * ctas = 0: one short CTA per 32 KiB tile; > 0: that many looping CTAs.
 * ref: none (the reference is single-GPU, librecuda.cpp:61). */
int lcb_multicast_store(void *mc_dst, const void *src, size_t bytes, int ctas, lcbStream stream);

/* ---- verification helpers that run on the device (used by tests and the benchmark) ------------- */

/* dst[0..bytes) <- the seeded byte stream: 64-bit word i = mix64(seed + (i+1) * 0x9E3779B97F4A7C15),
 * little-endian, mix64 = the splitmix64 finaliser.  dst 8-byte aligned. */
int lcb_fill_splitmix64(void *dst, size_t bytes, uint64_t seed, lcbStream stream);
/* The same stream from its 64-bit word `first_word` on: dst[0..bytes) <- bytes [8 * first_word, 8 * first_word
 * + bytes) of what lcb_fill_splitmix64 would write with this seed, so a window deep inside a multi-GiB
 * stream can be regenerated without the part before it. */
int lcb_fill_splitmix64_at(void *dst, size_t bytes, uint64_t seed, uint64_t first_word, lcbStream stream);

/* result[0] <- number of positions where a[i] != b[i]; result[1] <- smallest such i (UINT64_MAX if
 * none).  `result` is device memory for two uint64_t and is overwritten. */
int lcb_compare_bytes(const void *a, const void *b, size_t bytes, uint64_t *result, lcbStream stream);

/* out[0] <- order-independent 64-bit checksum of the buffer: sum over 8-byte words w_i of
 * mix64(w_i + i * 0x9E3779B97F4A7C15) modulo 2^64 (a trailing partial word is zero-extended).
 * `scratch` is device memory for at least lcb_checksum_scratch_bytes() bytes; `out` one uint64_t.
 * src 8-byte aligned. */
int lcb_checksum64(const void *src, size_t bytes, uint64_t *scratch, uint64_t *out, lcbStream stream);
size_t lcb_checksum_scratch_bytes(void);

/* lcb_checksum64 for callers that cannot allocate device memory.  No counterpart in the reference.
 * Same result as lcb_checksum64, but the scratch (one ticket counter + 1024 partial sums, about 8 KiB) is a
 * fixed array compiled into the library, so nothing is allocated here or by the caller: meant for a check
 * that runs when the application's own pool already owns all free HBM, or from a plug-in whose host forbids
 * allocating calls.  Limits and rules:
 *   - `bytes` above lcb_checksum64_noalloc_max_bytes() (64 GiB) is rejected with 1 and a line on stderr;
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress); make that
 *     first call before any stream capture begins;
 *   - every call on a device shares the one array (it is re-zeroed where needed at the start of a call), so
 *     two calls that may run at the same time on the GPU -- different streams, no ordering -- race: order them;
 *   - each GPU that loads the library holds the array until the process exits.
 * src 8-byte aligned; `out` is device memory for one uint64_t. */
int lcb_checksum64_noalloc(const void *src, size_t bytes, uint64_t *out, lcbStream stream);
size_t lcb_checksum64_noalloc_max_bytes(void);

/* Reads and clears the per-device sticky word that kernels set when a bounded wait gave up: bit 0 an mbarrier
 * wait of the bulk-copy ring, bit 1 a wait for another GPU's flag; 0 = no error.  Synchronises the device. */
int lcb_device_error_word(unsigned int *out);
/* The same word as last mirrored into host memory by the kernels, read WITHOUT synchronising or clearing:
 * what a host that has just finished a stream wait consults (libreCuStreamAwait and libreCuEventSynchronize
 * do).  0 until lcb_preload has run on the device. */
int lcb_device_error_peek(unsigned int *out);

/* Exercises the give-up path of the kernels' bounded waits without any fault: one thread waits, at most
 * max_tries (1..100000) tries, on a barrier nothing completes, then sets bit 0 of the sticky error word and
 * returns.  Afterwards lcb_device_error_word reports 1 and the device is fully usable. */
int lcb_selftest_wait_timeout(unsigned int max_tries, lcbStream stream);

/* Loads the default copy / memset / fill kernels onto the current device now instead of at their first
 * launch.  ref: loadMemcpyKernelsIfNeeded, driverapi/src/memcopy.cpp:23-75, called from context creation
 * (driverapi/src/librecuda.cpp:622). */
int lcb_preload(void);

/* Library / build identification: "lcb200 <version> sm_100a". */
const char *lcb_version(void);

/* Override one launch tunable by name (thread counts, unroll, bulk-ring depth ...; the names are the
 * fields of the Tuning record in the kernel sources; "reset" restores the shipped configuration).
 * For sweeps; returns 1 for an unknown name. */
int lcb_tune(const char *name, int value);
/* Current value of a tunable (-1 for an unknown name). */
int lcb_tune_get(const char *name);

/* CUDA-event stopwatch on a raw stream: start/stop record events on `stream`, elapsed waits for the
 * stop event and returns milliseconds. */
int lcb_timer_create(void **timer_out);
int lcb_timer_start(void *timer, lcbStream stream);
int lcb_timer_stop(void *timer, lcbStream stream);
int lcb_timer_elapsed_ms(void *timer, float *ms_out);
int lcb_timer_destroy(void *timer);
int lcb_stream_synchronize(lcbStream stream);
/* Work submitted to `waiter` after this call starts only when everything submitted to `signaller` before it
 * has finished (an event recorded on one stream and awaited by the other; the host does not block). */
int lcb_stream_wait_stream(lcbStream waiter, lcbStream signaller);

/* The CUDA runtime's own device-to-device copy and memset on the same stream, exported only so that the
 * benchmark can time them beside this library's kernels.  Nothing in the library calls them. */
int lcb_vendor_memcpy_d2d(void *dst, const void *src, size_t bytes, lcbStream stream);
int lcb_vendor_memset_d8(void *dst, unsigned char value, size_t bytes, lcbStream stream);

#ifdef __cplusplus
}
#endif
#endif /* LCB200_KERNELS_H */
