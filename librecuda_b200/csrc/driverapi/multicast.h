// NVLink multicast windows: per group of GPUs, one slab of device memory on every member, all bound to one
// multicast object, so that a multimem store issued by any member lands in every member's slab (NVSwitch
// replicates it).  The slabs are staging memory owned by the library; user buffers are never bound.
// Plain interface (no CUDA driver types) because <cuda.h> and librecuda.h cannot share a translation unit.
#pragma once

#include <cstddef>

namespace lcu {

struct McWindow {
    int n = 0;               // members
    int devs[16] = {};       // their device ordinals, in group order
    size_t bytes = 0;        // usable bytes of every slab (and of the multicast mapping)
    void *local[16] = {};    // local[k]: ordinary address of member k's slab (mapped for member k)
    void *mc = nullptr;      // multicast address: a multimem store at mc + x reaches local[k] + x for every k
};

// Window over exactly these devices with at least `min_bytes` per slab: cached per process, created on first
// use, re-created larger when needed.  Returns 0 and *out, -1 when the driver or a device has no multicast
// support (callers fall back to another path), or a positive CUresult.
int mc_window_acquire(const int *devs, int n, size_t min_bytes, const McWindow **out);

// Unbinds and frees every window; safe to call more than once.  Runs from libreCuCtxDestroy of a member and
// at process exit, so that no slab is still bound when the process goes away.
void mc_release_all();

}  // namespace lcu
