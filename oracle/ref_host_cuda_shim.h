// Force-included ahead of the reference's CUDA source (driverapi/kernels/memcpy/memcpy.cu) when it is
// compiled as plain host C++ for the oracle: maps the CUDA execution-space keywords and built-in index
// variables onto host globals that the emulated launch loop in ref_shim.cpp sets before each call.
// TEST INFRASTRUCTURE ONLY.
#pragma once
#include <cstddef>
#include <cstdint>
#define __global__
struct orc_dim3 {
    unsigned int x, y, z;
};
extern orc_dim3 blockIdx, threadIdx, gridDim, blockDim;
