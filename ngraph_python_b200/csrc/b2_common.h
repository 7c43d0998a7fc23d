// Shared host-side helpers of the b200ng library: error reporting and CUDA status checks.
#ifndef B2_COMMON_H
#define B2_COMMON_H

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <string>

#include "../../include/b200ng.h"

namespace b2 {

std::string& last_error_ref();

inline int fail(int code, const char* fmt, ...) {
    char buf[2048];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    last_error_ref() = buf;
    return code;
}

}  // namespace b2

#define B2_CUDA(call)                                                                     \
    do {                                                                                  \
        cudaError_t e__ = (call);                                                         \
        if (e__ != cudaSuccess)                                                           \
            return b2::fail(B2_ERR_CUDA, "%s failed: %s (%s:%d)", #call,                  \
                            cudaGetErrorString(e__), __FILE__, __LINE__);                 \
    } while (0)

#define B2_REQUIRE(cond, ...)                                   \
    do {                                                        \
        if (!(cond)) return b2::fail(B2_ERR_INVALID, __VA_ARGS__); \
    } while (0)

#endif  // B2_COMMON_H
