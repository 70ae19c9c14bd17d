// Status codes of the libreCu* API.
//
// Binary contract kept from the reference (driverapi/include/librecuda_status.h:6,20-22 and
// driverapi/include/librecuda_all_statuses.h:1-12): libreCudaStatus_t is a plain int and every
// status is an exported `extern "C"` *variable* (not an enum / macro), so callers compiled against
// the reference header resolve the same data symbols from this library.
//
// The validation macros keep the reference's stderr line format
// ("[LibreCuda Debug]: file:line: condition", librecuda_status.h:8-17).
#ifndef LIBRECUDA_B200_STATUS_H
#define LIBRECUDA_B200_STATUS_H

#include <iostream>

typedef int libreCudaStatus_t;

extern "C" {
extern libreCudaStatus_t LIBRECUDA_SUCCESS;                              // 0
extern libreCudaStatus_t LIBRECUDA_ERROR_INVALID_VALUE;                  // 1
extern libreCudaStatus_t LIBRECUDA_ERROR_OUT_OF_MEMORY;                  // 2
extern libreCudaStatus_t LIBRECUDA_ERROR_NOT_INITIALIZED;                // 3
extern libreCudaStatus_t LIBRECUDA_ERROR_INVALID_DEVICE;                 // 101
extern libreCudaStatus_t LIBRECUDA_ERROR_INVALID_IMAGE;                  // 200
extern libreCudaStatus_t LIBRECUDA_ERROR_INVALID_CONTEXT;                // 201
extern libreCudaStatus_t LIBRECUDA_ERROR_NOT_FOUND;                      // 500
extern libreCudaStatus_t LIBRECUDA_ERROR_NOT_READY;                      // 600
extern libreCudaStatus_t LIBRECUDA_ERROR_LAUNCH_OUT_OF_RESOURCES;        // 701
extern libreCudaStatus_t LIBRECUDA_ERROR_COMPAT_NOT_SUPPORTED_ON_DEVICE; // 804
extern libreCudaStatus_t LIBRECUDA_ERROR_UNKNOWN;                        // 999
}

#define LIBRECUDA_DEBUG(msg) std::cerr << "[LibreCuda Debug]: " << msg << std::endl
#define LIBRECUDA_STR2_(x) #x
#define LIBRECUDA_STR_(x) LIBRECUDA_STR2_(x)

// Print "file:line: condition" and return `err` from the enclosing function when `condition` fails.
#define LIBRECUDA_VALIDATE(condition, err)                                               \
    do {                                                                                 \
        if (!(condition)) {                                                              \
            LIBRECUDA_DEBUG(__FILE__ ":" LIBRECUDA_STR_(__LINE__) ": " #condition);      \
            return (err);                                                                \
        }                                                                                \
    } while (0)

#define LIBRECUDA_SUCCEED() return LIBRECUDA_SUCCESS
#define LIBRECUDA_FAIL(status) return (status)

// Early-return a non-success status of a callee.
#define LIBRECUDA_ERR_PROPAGATE(expr)                                    \
    do {                                                                 \
        libreCudaStatus_t librecuda_status_tmp_ = (expr);                \
        if (librecuda_status_tmp_ != LIBRECUDA_SUCCESS) {                \
            return librecuda_status_tmp_;                                \
        }                                                                \
    } while (0)

#endif  // LIBRECUDA_B200_STATUS_H
