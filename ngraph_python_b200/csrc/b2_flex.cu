// Flex16 host<->device conversions and statistics, as device kernels.
//
// The reference converts on the host with numpy before every upload
// (ngraph/transformers/flexgputransform.py:178-208): value / scale, clip to [-2^15, 2^15-1],
// float->int16 assignment (truncation toward zero), maxabs = int(max |clipped|).  Here the fp32
// data is uploaded as it is and converted on the device with the same arithmetic, so the PCIe
// copy is the only host-side work.
#include "b2_common.h"
#include "b2_ew_device.cuh"

namespace {

const int kThreads = 256;

__global__ void __launch_bounds__(kThreads)
k_host_quantize(const float* __restrict__ src, short* __restrict__ dst, long long n,
                const b2_flex_scale* __restrict__ table, int slot, int* __restrict__ stats) {
    __shared__ int ismem[32];
    const float inv = table[slot].inv_scale;
    int stat = 0;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float v = src[i] * inv;                       // power-of-two scaling: exact
        v = fminf(fmaxf(v, -32768.0f), 32767.0f);     // clip (NaN -> -32768 like fmaxf/fminf)
        const int m = (int)v;                         // truncation toward zero
        stat = b2_absmax(stat, m);
        dst[i] = (short)m;
    }
    b2_block_stat(stat, stats + slot, ismem);
}

__global__ void __launch_bounds__(kThreads)
k_dequantize(const short* __restrict__ src, float* __restrict__ dst, long long n,
             const b2_flex_scale* __restrict__ table, int slot) {
    const float s = table[slot].scale;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        dst[i] = s * (float)src[i];
}

__global__ void __launch_bounds__(kThreads)
k_absmax_bits(const float* __restrict__ src, long long n, int* __restrict__ out) {
    __shared__ int ismem[32];
    int stat = 0;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        stat = max(stat, b2_absbits(src[i]));
    b2_block_stat(stat, out, ismem);
}

unsigned grid_for(long long n) {
    long long g = (n + kThreads - 1) / kThreads;
    if (g < 1) g = 1;
    if (g > 148 * 16) g = 148 * 16;
    return (unsigned)g;
}

}  // namespace

extern "C" int b2_flex_host_quantize(const float* src, int16_t* dst, int64_t n,
                                     const b2_flex_scale* table, int32_t slot, int32_t* stats,
                                     void* stream) {
    B2_REQUIRE(src && dst && table && stats && slot >= 0 && n >= 0, "bad argument");
    if (n == 0) return B2_OK;
    k_host_quantize<<<grid_for(n), kThreads, 0, (cudaStream_t)stream>>>(src, dst, n, table, slot,
                                                                       stats);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

extern "C" int b2_flex_dequantize(const int16_t* src, float* dst, int64_t n,
                                  const b2_flex_scale* table, int32_t slot, void* stream) {
    B2_REQUIRE(src && dst && table && slot >= 0 && n >= 0, "bad argument");
    if (n == 0) return B2_OK;
    k_dequantize<<<grid_for(n), kThreads, 0, (cudaStream_t)stream>>>(src, dst, n, table, slot);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

extern "C" int b2_absmax_bits_f32(const float* src, int64_t n, int32_t* out, void* stream) {
    B2_REQUIRE(src && out && n >= 0, "bad argument");
    if (n == 0) return B2_OK;
    k_absmax_bits<<<grid_for(n), kThreads, 0, (cudaStream_t)stream>>>(src, n, out);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

// End of a call: the statistics array and the status word go to the host in ONE small kernel that
// stores them into pinned host memory the device can address (zero-copy), and the statistics are
// cleared for the next call.  Replaces two device-to-host copies and a memset per call -- inside
// a replayed CUDA graph those are three more serialised nodes, each with its own latency.
namespace {
__global__ void __launch_bounds__(kThreads)
k_publish(int* __restrict__ stats, int n, const int* __restrict__ status,
          volatile int* __restrict__ host_stats, volatile int* __restrict__ host_status) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        host_stats[i] = stats[i];
        stats[i] = 0;
    }
    if (threadIdx.x == 0 && status && host_status) *host_status = *status;
    __threadfence_system();
}
}  // namespace

extern "C" int b2_flex_publish(int32_t* stats, int32_t n, const int32_t* status,
                               int32_t* host_stats, int32_t* host_status, void* stream) {
    B2_REQUIRE(n >= 0 && (n == 0 || (stats && host_stats)), "bad argument");
    B2_REQUIRE((status == nullptr) == (host_status == nullptr), "status source and destination go together");
    k_publish<<<1, kThreads, 0, (cudaStream_t)stream>>>(stats, n, status, host_stats, host_status);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}
