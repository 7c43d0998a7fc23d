// Library-level entry points: version, error string, device count.
#include "b2_common.h"

namespace b2 {
std::string& last_error_ref() {
    static thread_local std::string err;
    return err;
}
}  // namespace b2

extern "C" const char* b2_last_error(void) { return b2::last_error_ref().c_str(); }

extern "C" int b2_version(void) { return 100; }

extern "C" int b2_device_count(void) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return b2::fail(B2_ERR_CUDA, "cudaGetDeviceCount: %s", cudaGetErrorString(e));
    }
    return n;
}
