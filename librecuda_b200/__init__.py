"""librecuda_b200 -- B200-native (sm_100a) data-movement path behind the LibreCUDA `libreCu*` C API.

The product is the shared library `lib/libdriverapi.so` (hand-written CUDA kernels + a C++ host layer);
this package only binds it for Python callers, tests and the benchmark.  Importing `librecuda_b200.api`
raises if the library has not been built: there is no CPU fallback.
"""
__version__ = "0.1"
