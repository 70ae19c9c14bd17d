/* lcb_oracle.c -- CPU restatement of the reference's data-movement path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or calls this file; it is the
 * checker used by tests/, by the smoke test and by the CPU-baseline leg of the benchmark.
 *
 * What it restates (paths are relative to the reference project):
 *  - the DtoD dispatcher memcpyD2D, driverapi/src/memcopy.cpp:77-158 (which of the three kernels run,
 *    with which grids and which byte ranges), and the three kernels it launches,
 *    driverapi/kernels/memcpy/memcpy.cu:5-27, executed thread by thread on the host;
 *  - the reference's own acceptance criterion for the path: byte equality with host memory after
 *    HtoD -> DtoD... -> DtoH (tests/dma_chronological_consistency/main.cpp:33-36,56-85), i.e. plain
 *    memcpy / memset / host loops over the same seeded bytes;
 *  - the grid-indexed fill fixture tests/indexing/write_float.cu:1-4 generalised to out[i] = float(i),
 *    and the multiply-add stage used between HtoD and DtoH in the stream-ordering configuration.
 *
 * Pinning: tests check this file against (1) the reference's golden vectors G1..G3
 * (tests/dma_chronological_consistency, tests/memcopy, tests/indexing) and (2) the reference's own
 * memcopy.cpp + memcpy.cu compiled for the host (oracle/_ref, built by oracle/build_ref.sh), launch plan
 * by launch plan and byte by byte.
 */
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#define ORC_GOLDEN 0x9E3779B97F4A7C15ull

static inline uint64_t orc_mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

/* Seeded byte stream: 64-bit word i = mix64(seed + (i+1) * golden), little-endian.  The stream is keyed by
 * position, so any window of it can be produced without the bytes before it: orc_fill_window writes the n
 * bytes that start at word `first_word` of the stream (a window deep inside a multi-GiB buffer costs only
 * its own length). */
void orc_fill_window(uint8_t *dst, size_t n, uint64_t seed, uint64_t first_word) {
    size_t nw = n / 8, i;
    for (i = 0; i < nw; ++i) {
        uint64_t w = orc_mix64(seed + (first_word + (uint64_t)i + 1) * ORC_GOLDEN);
        memcpy(dst + 8 * i, &w, 8);
    }
    if (n & 7) {
        uint64_t w = orc_mix64(seed + (first_word + (uint64_t)nw + 1) * ORC_GOLDEN);
        memcpy(dst + 8 * nw, &w, n & 7);
    }
}

void orc_fill_bytes(uint8_t *dst, size_t n, uint64_t seed) { orc_fill_window(dst, n, seed, 0); }

/* Uniform floats in [0,1): top 24 bits of word i scaled by 2^-24. */
void orc_fill_f32(float *dst, size_t n, uint64_t seed) {
    size_t i;
    for (i = 0; i < n; ++i) {
        uint64_t w = orc_mix64(seed + (uint64_t)(i + 1) * ORC_GOLDEN);
        dst[i] = (float)(w >> 40) * (1.0f / 16777216.0f);
    }
}

/* ---------------------------------------------------------------------------------------------
 * memcpyD2D restated (driverapi/src/memcopy.cpp:77-158).
 * ------------------------------------------------------------------------------------------- */
typedef struct {
    int kernel;        /* 1 = HighBW, 2 = LowLatency, 3 = Trailing */
    uint64_t grid_x;
    uint64_t grid_y;
    uint64_t offset;   /* byte offset of dst/src handed to the kernel */
    uint64_t n;        /* the kernel's `n` argument (words for 2, bytes for 3, unused for 1) */
} orc_launch_t;

#define ORC_BLOCK 256ull
#define ORC_THREAD_COPY 16ull
#define ORC_MAX_GRID_X 65535ull
#define ORC_HIGHBW_GRAN 4096ull
#define ORC_FINISH_GRAN 4ull

static uint64_t ceil_div(uint64_t a, uint64_t b) { return (a + b - 1) / b; }

/* Fills plan[0..3) and returns the number of launches, in launch order. */
int orc_ref_d2d_plan(uint64_t size, orc_launch_t *plan) {
    int n = 0;
    int high_bw = size > 1024ull * 1024ull;                      /* memcopy.cpp:82, strict */
    int k1 = high_bw;                                            /* :87 */
    int k2 = !high_bw || (size % ORC_HIGHBW_GRAN) != 0;          /* :88 */
    int k3 = (size % ORC_FINISH_GRAN) != 0;                      /* :89 */
    if (k1) {                                                    /* :93-111 */
        plan[n].kernel = 1;
        plan[n].grid_x = size / (ORC_THREAD_COPY * ORC_BLOCK);
        plan[n].grid_y = ceil_div(plan[n].grid_x, ORC_MAX_GRID_X);
        plan[n].offset = 0;
        plan[n].n = 0;
        ++n;
    }
    if (k2) {                                                    /* :113-136 */
        uint64_t copied = high_bw ? (size / ORC_HIGHBW_GRAN) * ORC_HIGHBW_GRAN : 0;
        uint64_t words = (size - copied) / 4;
        plan[n].kernel = 2;
        plan[n].grid_x = ceil_div(words, ORC_BLOCK);
        plan[n].grid_y = 1;
        plan[n].offset = copied;
        plan[n].n = words;
        ++n;
    }
    if (k3) {                                                    /* :138-155 */
        uint64_t copied = (size / ORC_HIGHBW_GRAN) * ORC_HIGHBW_GRAN;
        uint64_t rem = size - copied;
        plan[n].kernel = 3;
        plan[n].grid_x = ceil_div(rem, ORC_BLOCK);
        plan[n].grid_y = 1;
        plan[n].offset = copied;
        plan[n].n = rem;
        ++n;
    }
    return n;
}

/* The three kernels of driverapi/kernels/memcpy/memcpy.cu:5-27, one host loop iteration per thread.
 * `limit` bounds every access to the caller's buffers: for sizes >= 256 MiB the reference's HighBW grid
 * (grid_x is not clamped to 65535 while grid_y grows) addresses blocks past the end of the buffers;
 * the emulation skips those and reports how many bytes they would have touched. */
uint64_t orc_ref_d2d_run(uint8_t *dst, const uint8_t *src, uint64_t size) {
    orc_launch_t plan[3];
    int n = orc_ref_d2d_plan(size, plan), l;
    uint64_t oob = 0;
    for (l = 0; l < n; ++l) {
        const orc_launch_t *p = &plan[l];
        uint8_t *d = dst + p->offset;
        const uint8_t *s = src + p->offset;
        uint64_t by, bx, t;
        if (p->kernel == 1) {
            for (by = 0; by < p->grid_y; ++by)
                for (bx = 0; bx < p->grid_x; ++bx) {
                    uint64_t blk = by * p->grid_x + bx;              /* memcpy.cu:6 */
                    if ((blk + 1) * 4096 > size) { oob += 4096; continue; }
                    for (t = 0; t < ORC_BLOCK; ++t) {
                        uint64_t idx = ((ORC_BLOCK * blk) << 2) + t;  /* word index */
                        int i;
                        for (i = 0; i < 4; ++i) {                    /* memcpy.cu:9-12 */
                            memcpy(d + 4 * idx, s + 4 * idx, 4);
                            idx += ORC_BLOCK;
                        }
                    }
                }
        } else if (p->kernel == 2) {
            for (bx = 0; bx < p->grid_x; ++bx)
                for (t = 0; t < ORC_BLOCK; ++t) {
                    uint64_t tid = ORC_BLOCK * bx + t;               /* memcpy.cu:16-19 */
                    if (tid < p->n) memcpy(d + 4 * tid, s + 4 * tid, 4);
                }
        } else {
            for (bx = 0; bx < p->grid_x; ++bx)
                for (t = 0; t < ORC_BLOCK; ++t) {
                    uint64_t tid = ORC_BLOCK * bx + t;               /* memcpy.cu:23-26 */
                    if (tid < p->n) d[tid] = s[tid];
                }
        }
    }
    return oob;
}

/* ---------------------------------------------------------------------------------------------
 * host statements of the operations (what the reference's tests compare against)
 * ------------------------------------------------------------------------------------------- */
void orc_memcpy(uint8_t *dst, const uint8_t *src, size_t n) { memcpy(dst, src, n); }
void orc_memset_d8(uint8_t *dst, uint8_t v, size_t n) { memset(dst, v, n); }
void orc_memset_d16(uint16_t *dst, uint16_t v, size_t n) { size_t i; for (i = 0; i < n; ++i) dst[i] = v; }
void orc_memset_d32(uint32_t *dst, uint32_t v, size_t n) { size_t i; for (i = 0; i < n; ++i) dst[i] = v; }
void orc_index_fill_f32(float *dst, size_t n) { size_t i; for (i = 0; i < n; ++i) dst[i] = (float)i; }
/* two roundings: product, then sum (this file is compiled with -ffp-contract=off) */
void orc_axpb_f32(float *y, const float *x, float a, float b, size_t n) {
    size_t i;
    for (i = 0; i < n; ++i) { volatile float p = a * x[i]; y[i] = p + b; }
}

/* Order-independent checksum: sum of mix64(word_i + i * golden), trailing partial word zero-extended. */
uint64_t orc_checksum64(const uint8_t *src, size_t n) {
    size_t nw = n / 8, i;
    uint64_t acc = 0, w;
    for (i = 0; i < nw; ++i) { memcpy(&w, src + 8 * i, 8); acc += orc_mix64(w + (uint64_t)i * ORC_GOLDEN); }
    if (n & 7) { w = 0; memcpy(&w, src + 8 * nw, n & 7); acc += orc_mix64(w + (uint64_t)nw * ORC_GOLDEN); }
    return acc;
}

/* Shard boundaries of a partitioned copy: `parts` contiguous shards, interior boundaries multiples of
 * `align` (power of two), the last shard takes the tail.  offsets has parts+1 entries. */
int orc_partition(uint64_t total, int parts, uint64_t align, uint64_t *offsets) {
    int g;
    uint64_t per;
    if (parts < 1 || align == 0 || (align & (align - 1))) return 1;
    per = ceil_div(ceil_div(total, (uint64_t)parts), align) * align;
    for (g = 0; g <= parts; ++g) {
        uint64_t o = per * (uint64_t)g;
        offsets[g] = (o > total || g == parts) ? total : o;
    }
    return 0;
}

/* All-to-all on host buffers: recv[j][r*chunk .. ) = send[r][j*chunk .. ) for all r, j. */
void orc_alltoall(uint8_t *const *recv, const uint8_t *const *send, size_t chunk, int n) {
    int r, j;
    for (r = 0; r < n; ++r)
        for (j = 0; j < n; ++j) memcpy(recv[j] + (size_t)r * chunk, send[r] + (size_t)j * chunk, chunk);
}

/* ---------------------------------------------------------------------------------------------
 * multithreaded CPU baseline: T threads, contiguous slices, returns best-of-`reps` seconds
 * ------------------------------------------------------------------------------------------- */
typedef struct {
    uint8_t *dst;
    const uint8_t *src;
    size_t n;
    int op;  /* 0 memcpy, 1 memset */
    int value;
} orc_job_t;

static void *orc_worker(void *arg) {
    orc_job_t *j = (orc_job_t *)arg;
    if (j->op == 0) memcpy(j->dst, j->src, j->n);
    else memset(j->dst, j->value, j->n);
    return NULL;
}

static double now_s(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

double orc_mt_run(uint8_t *dst, const uint8_t *src, size_t n, int op, int value, int threads, int reps) {
    double best = 1e30;
    int r, t;
    pthread_t *th;
    orc_job_t *jobs;
    if (threads < 1) threads = 1;
    th = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)threads);
    jobs = (orc_job_t *)malloc(sizeof(orc_job_t) * (size_t)threads);
    for (r = 0; r < reps; ++r) {
        size_t per = ((n / (size_t)threads) + 63) & ~(size_t)63;
        double t0 = now_s(), dt;
        for (t = 0; t < threads; ++t) {
            size_t lo = per * (size_t)t, hi = lo + per;
            if (lo > n) lo = n;
            if (hi > n || t == threads - 1) hi = n;
            jobs[t].dst = dst + lo;
            jobs[t].src = src ? src + lo : NULL;
            jobs[t].n = hi - lo;
            jobs[t].op = op;
            jobs[t].value = value;
            pthread_create(&th[t], NULL, orc_worker, &jobs[t]);
        }
        for (t = 0; t < threads; ++t) pthread_join(th[t], NULL);
        dt = now_s() - t0;
        if (dt < best) best = dt;
    }
    free(th);
    free(jobs);
    return best;
}
