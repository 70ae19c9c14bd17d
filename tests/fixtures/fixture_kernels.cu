// Fixture kernels for the libreCuLaunchKernel tests, compiled to tests/fixtures/_bin/fixture_kernels.cubin
// for sm_100a by __graft_entry__.build().  They play the role of the reference's test kernels
// (tests/indexing/write_float.cu, tests/write_float/write_float.cu, tests/kernel_struct_param/
// read_from_struct.cu, tests/dynamic_shared_mem/write_float.cu, tests/async_kernels/write_float.cu) but are
// written for the configurations this repository checks.
#include <cstddef>

// out[i] = float(i) over a 2-D grid of 256-thread blocks; block id = blockIdx.y * gridDim.x + blockIdx.x.
extern "C" __global__ void index_fill_2d(float *out, size_t n) {
    const size_t i = ((size_t)blockIdx.y * gridDim.x + blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) out[i] = (float)i;
}

// y = 2x + 1 with separate multiply and add roundings
extern "C" __global__ void axpb(float *y, const float *x, float a, float b, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = __fadd_rn(__fmul_rn(a, x[i]), b);
}

extern "C" __global__ void store_value(float *dst, float value) { *dst = value; }

__device__ int fixture_global = 0x69;

// scalar parameters of three sizes plus a module-scope variable
extern "C" __global__ void store_sum(float *dst, short a, float b) { *dst = (float)a + b + (float)fixture_global; }

struct fixture_struct {
    int x, y, z;
    int w, h, d;
    char text[33];
    char last;
};

extern "C" __global__ void read_struct(fixture_struct s, int *out) {
    out[0] = s.w;
    out[1] = (int)s.last;
}

// touches dynamic shared memory well past 4 KiB
extern "C" __global__ void smem_sum(float *dst, short a, float b) {
    extern __shared__ float buf[];
    buf[1024] = (float)a;
    buf[1025] = b;
    __syncthreads();
    *dst = buf[1024] + buf[1025];
}

// busy kernel: spins for `cycles` clock ticks, then dst[0] += 1 (non-atomic: ordering tests rely on it)
extern "C" __global__ void spin_then_increment(float *dst, long long cycles) {
    const long long t0 = clock64();
    while (clock64() - t0 < cycles) {
    }
    *dst = *dst + 1.0f;
}

extern "C" __global__ void empty_kernel() {}
