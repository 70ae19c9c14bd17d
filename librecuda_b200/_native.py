"""ctypes binding of libdriverapi.so: the `lcb_*` kernel layer (include/lcb200_kernels.h) and the
`libreCu*` API (include/librecuda.h).

There is no fallback: if the shared object has not been built, importing this module raises.  Build it
with `python -m librecuda_b200.build`.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libdriverapi.so"

if not LIB_PATH.exists():
    raise ImportError(
        f"{LIB_PATH} is missing: the native CUDA library has not been built "
        "(run `python -m librecuda_b200.build`); there is no CPU fallback"
    )

lib = C.CDLL(str(LIB_PATH))

vp, sz, u64, u32, i32 = C.c_void_p, C.c_size_t, C.c_uint64, C.c_uint32, C.c_int
vpp = C.POINTER(C.c_void_p)

# name -> (restype, argtypes); every symbol the two public headers declare
LCB_FUNCTIONS = {
    "lcb_copy_d2d": (i32, [vp, vp, sz, vp]),
    "lcb_copy_d2d_ex": (i32, [vp, vp, sz, i32, i32, vp]),
    "lcb_copy_d2d_describe": (i32, [vp, vp, sz, i32, i32, C.c_char_p, sz]),
    "lcb_memset_d8": (i32, [vp, C.c_ubyte, sz, vp]),
    "lcb_memset_d16": (i32, [vp, C.c_ushort, sz, vp]),
    "lcb_memset_d32": (i32, [vp, C.c_uint, sz, vp]),
    "lcb_memset_ex": (i32, [vp, C.c_uint, i32, sz, i32, i32, vp]),
    "lcb_index_fill_f32": (i32, [vp, sz, vp]),
    "lcb_axpb_f32": (i32, [vp, vp, C.c_float, C.c_float, sz, vp]),
    "lcb_alltoall_push": (i32, [vpp, vp, sz, i32, i32, vp]),
    "lcb_alltoall_pull": (i32, [vpp, vp, sz, i32, i32, vp]),
    "lcb_multicast_store": (i32, [vp, vp, sz, i32, vp]),
    "lcb_alltoall_engines": (i32, [vpp, vp, sz, i32, i32, vp, vpp, C.c_uint, C.c_uint, vp, vp]),
    "lcb_alltoall_engines_step": (i32, [i32, i32, i32] + [C.POINTER(i32)] * 5),
    "lcb_bcast_ring_hop": (i32, [vp, vp, vp, vp, sz, sz, C.c_uint, C.c_uint, i32, vp]),
    "lcb_bcast_tree_plan": (i32, [i32, i32, i32, C.POINTER(i32), C.POINTER(i32)]),
    "lcb_bcast_tree_node": (i32, [vp, vp, vpp, vpp, sz, sz, sz, C.c_uint, C.c_uint, i32, vp]),
    "lcb_flag_post": (i32, [vp, C.c_uint, vp]),
    "lcb_flag_wait": (i32, [vp, C.c_uint, C.c_uint, vp]),
    "lcb_fill_splitmix64": (i32, [vp, sz, u64, vp]),
    "lcb_fill_splitmix64_at": (i32, [vp, sz, u64, u64, vp]),
    "lcb_compare_bytes": (i32, [vp, vp, sz, vp, vp]),
    "lcb_checksum64": (i32, [vp, sz, vp, vp, vp]),
    "lcb_checksum_scratch_bytes": (sz, []),
    "lcb_checksum64_noalloc": (i32, [vp, sz, vp, vp]),
    "lcb_checksum64_noalloc_max_bytes": (sz, []),
    "lcb_device_error_word": (i32, [C.POINTER(C.c_uint)]),
    "lcb_device_error_peek": (i32, [C.POINTER(C.c_uint)]),
    "lcb_preload": (i32, []),
    "lcb_selftest_wait_timeout": (i32, [C.c_uint, vp]),
    "lcb_version": (C.c_char_p, []),
    "lcb_tune": (i32, [C.c_char_p, i32]),
    "lcb_tune_get": (i32, [C.c_char_p]),
    "lcb_timer_create": (i32, [vpp]),
    "lcb_timer_start": (i32, [vp, vp]),
    "lcb_timer_stop": (i32, [vp, vp]),
    "lcb_timer_elapsed_ms": (i32, [vp, C.POINTER(C.c_float)]),
    "lcb_timer_destroy": (i32, [vp]),
    "lcb_stream_synchronize": (i32, [vp]),
    "lcb_stream_wait_stream": (i32, [vp, vp]),
    "lcb_vendor_memcpy_d2d": (i32, [vp, vp, sz, vp]),
    "lcb_vendor_memset_d8": (i32, [vp, C.c_ubyte, sz, vp]),
}

LIBRECU_FUNCTIONS = {
    # reference surface (30)
    "libreCuInit": (i32, [i32]),
    "libreCuDeviceGetCount": (i32, [C.POINTER(i32)]),
    "libreCuDeviceGet": (i32, [vpp, i32]),
    "libreCuGetErrorString": (i32, [i32, C.POINTER(C.c_char_p)]),
    "libreCuCtxCreate_v2": (i32, [vpp, i32, vp]),
    "libreCuCtxDestroy": (i32, [vp]),
    "libreCuCtxSetCurrent": (i32, [vp]),
    "libreCuCtxGetCurrent": (i32, [vpp]),
    "libreCuMemAlloc": (i32, [vpp, sz, C.c_bool]),
    "libreCuMemCpy": (i32, [vp, vp, sz, vp, C.c_bool]),
    "libreCuMemFree": (i32, [vp]),
    "libreCuStreamCreate": (i32, [vpp, u32]),
    "libreCuStreamDestroy": (i32, [vp]),
    "libreCuDeviceGetName": (i32, [C.c_char_p, i32, vp]),
    "libreCuDeviceGetAttribute": (i32, [C.POINTER(i32), i32, vp]),
    "libreCuFuncSetAttribute": (i32, [vp, i32, i32]),
    "libreCuModuleLoadData": (i32, [vpp, vp, sz]),
    "libreCuModuleGetFunctionCount": (i32, [C.POINTER(u32), vp]),
    "libreCuModuleEnumerateFunctions": (i32, [vpp, u32, vp]),
    "libreCuFuncGetName": (i32, [C.POINTER(C.c_char_p), vp]),
    "libreCuModuleGetFunction": (i32, [vpp, vp, C.c_char_p]),
    "libreCuLaunchKernel": (i32, [vp, u32, u32, u32, u32, u32, u32, u32, vp, vpp, sz, vpp, C.c_bool]),
    "libreCuEventCreate": (i32, [vpp, u32]),
    "libreCuEventRecord": (i32, [vp, vp]),
    "libreCuEventSynchronize": (i32, [vp]),
    "libreCuEventElapsedTime": (i32, [C.POINTER(C.c_float), vp, vp]),
    "libreCuEventDestroy": (i32, [vp]),
    "libreCuStreamCommence": (i32, [vp]),
    "libreCuStreamAwait": (i32, [vp]),
    "libreCuModuleUnload": (i32, [vp]),
    # additive
    "libreCuMemcpyHtoD": (i32, [vp, vp, sz, vp]),
    "libreCuMemcpyHtoDAsync": (i32, [vp, vp, sz, vp]),
    "libreCuMemcpyDtoH": (i32, [vp, vp, sz, vp]),
    "libreCuMemcpyDtoHAsync": (i32, [vp, vp, sz, vp]),
    "libreCuMemcpyDtoD": (i32, [vp, vp, sz, vp]),
    "libreCuMemcpyDtoDAsync": (i32, [vp, vp, sz, vp]),
    "libreCuMemAllocHost": (i32, [vpp, sz]),
    "libreCuMemFreeHost": (i32, [vp]),
    "libreCuMemsetD8": (i32, [vp, C.c_ubyte, sz, vp]),
    "libreCuMemsetD8Async": (i32, [vp, C.c_ubyte, sz, vp]),
    "libreCuMemsetD16": (i32, [vp, C.c_ushort, sz, vp]),
    "libreCuMemsetD16Async": (i32, [vp, C.c_ushort, sz, vp]),
    "libreCuMemsetD32": (i32, [vp, C.c_uint, sz, vp]),
    "libreCuMemsetD32Async": (i32, [vp, C.c_uint, sz, vp]),
    "libreCuStreamWaitEvent": (i32, [vp, vp]),
    "libreCuEventQuery": (i32, [vp]),
    "libreCuEventGetTimestamp": (i32, [C.POINTER(u64), vp]),
    "libreCuDeviceCanAccessPeer": (i32, [C.POINTER(i32), vp, vp]),
    "libreCuCtxEnablePeerAccess": (i32, [vp, C.c_uint]),
    "libreCuMemcpyPeer": (i32, [vp, vp, sz, vp, C.c_bool]),
    "libreCuPartitionPlan": (i32, [sz, i32, sz, C.POINTER(sz)]),
    "libreCuMemcpyPartitioned": (i32, [vpp, vp, sz, i32, sz, vpp]),
    "libreCuAllToAllPush": (i32, [vpp, vp, sz, i32, i32, vp]),
    "libreCuAllToAllPull": (i32, [vpp, vp, sz, i32, i32, vp]),
    "libreCuAllToAllEngines": (i32, [vpp, vp, sz, i32, i32, vpp, C.c_uint, C.c_uint, vp]),
    "libreCuAllToAll": (i32, [vpp, vpp, sz, i32, vpp, i32]),
    "libreCuBroadcast": (i32, [vpp, i32, sz, i32, vpp, i32]),
    "libreCuBroadcastLastForm": (i32, [C.POINTER(i32)]),
    "libreCuIpcGetMemHandle": (i32, [vp, vp]),
    "libreCuIpcOpenMemHandle": (i32, [vpp, vp]),
    "libreCuIpcCloseMemHandle": (i32, [vp]),
    "libreCuStreamGetNativeHandle": (i32, [vpp, vp]),
}

STATUS_VARIABLES = {
    "LIBRECUDA_SUCCESS": 0,
    "LIBRECUDA_ERROR_INVALID_VALUE": 1,
    "LIBRECUDA_ERROR_OUT_OF_MEMORY": 2,
    "LIBRECUDA_ERROR_NOT_INITIALIZED": 3,
    "LIBRECUDA_ERROR_INVALID_DEVICE": 101,
    "LIBRECUDA_ERROR_INVALID_IMAGE": 200,
    "LIBRECUDA_ERROR_INVALID_CONTEXT": 201,
    "LIBRECUDA_ERROR_NOT_FOUND": 500,
    "LIBRECUDA_ERROR_NOT_READY": 600,
    "LIBRECUDA_ERROR_LAUNCH_OUT_OF_RESOURCES": 701,
    "LIBRECUDA_ERROR_COMPAT_NOT_SUPPORTED_ON_DEVICE": 804,
    "LIBRECUDA_ERROR_UNKNOWN": 999,
}

for _name, (_res, _args) in {**LCB_FUNCTIONS, **LIBRECU_FUNCTIONS}.items():
    _fn = getattr(lib, _name)  # AttributeError here = a declared symbol is not exported
    _fn.restype = _res
    _fn.argtypes = _args

IPC_HANDLE_SIZE = 72
