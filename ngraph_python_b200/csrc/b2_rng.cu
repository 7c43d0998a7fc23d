// Random fill: out[i] ~ U[low, high) or N(loc, scale).
//
// Takes the place of RngFillKernel / FlexRngFillKernel (ngraph/transformers/gpu/tensor_ops.py:
// 621-661, 713-740), which fill the tensor through pycuda's generator (fill_uniform /
// fill_normal) and then scale and shift it with a second elementwise pass.  Here one kernel draws,
// scales, shifts and -- for flex16 storage -- quantises with the output's exponent, measuring the
// range on a tensor's first write like every other flex kernel of this library.
//
// Generator: Philox-4x32 with 10 rounds (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as
// easy as 1, 2, 3", SC'11), counter-based: element group g of a launch uses counter
// (g, 0, offset_lo, offset_hi) under the key (seed_lo, seed_hi) and yields four 32-bit words, i.e.
// four uniforms or (Box-Muller) four normals.  A given (seed, offset) always reproduces the same
// tensor, on any grid size.  So that every execution of an op draws fresh numbers (the
// reference's test_rng_repetition) -- also when the launch is replayed from a CUDA graph, where
// arguments are frozen -- the offset can live on the device: *device_counter is added to `offset`
// and advanced by one after the fill.
#include <cstdint>

#include "b2_common.h"

namespace {

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
    const uint32_t m0 = 0xD2511F53u, m1 = 0xCD9E8D57u;
    const uint32_t hi0 = __umulhi(m0, c[0]), lo0 = m0 * c[0];
    const uint32_t hi1 = __umulhi(m1, c[2]), lo1 = m1 * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

__device__ __forceinline__ void philox4x32_10(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        philox_round(c, k0, k1);
        k0 += 0x9E3779B9u;          // Weyl sequence of the key schedule
        k1 += 0xBB67AE85u;
    }
}

// 24 random bits -> [0, 1) exactly representable, never 1
__device__ __forceinline__ float u01(uint32_t w) { return (float)(w >> 8) * (1.0f / 16777216.0f); }

template <typename T>
__global__ void __launch_bounds__(256)
rng_fill_kernel(T* __restrict__ out, long long n, int normal, float a, float b,
                unsigned long long seed, unsigned long long offset,
                const unsigned long long* __restrict__ counter,
                const b2_flex_scale* __restrict__ table, int slot, int* stats,
                unsigned long long* probe_out, int probe) {
    const bool flex = sizeof(T) == 2;
    if (counter) offset += *counter;
    const float q = flex && !probe ? table[slot].inv_scale : 1.0f;
    float fstat = 0.0f, fmax = 0.0f;
    const long long groups = (n + 3) / 4;
    for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < groups;
         g += (long long)gridDim.x * blockDim.x) {
        uint32_t c[4] = {(uint32_t)g, (uint32_t)((unsigned long long)g >> 32), (uint32_t)offset,
                         (uint32_t)(offset >> 32)};
        philox4x32_10(c, (uint32_t)seed, (uint32_t)(seed >> 32));
        float v[4];
        if (normal) {
            // Box-Muller on two pairs; 1 - u is in (0, 1], so the logarithm is finite
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float r = sqrtf(-2.0f * logf(1.0f - u01(c[2 * h])));
                float s, co;
                sincospif(2.0f * u01(c[2 * h + 1]), &s, &co);
                v[2 * h] = a + b * (r * co);
                v[2 * h + 1] = a + b * (r * s);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float x = a + (b - a) * u01(c[j]);
                v[j] = x < b || !(a < b) ? x : a;      // rounding may land on `high`: fold it back
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const long long i = 4 * g + j;
            if (i >= n) break;
            if (!flex) {
                out[i] = (T)v[j];
            } else if (probe) {
                fmax = fmaxf(fmax, fabsf(v[j]));
            } else {
                float m = v[j] * q;
                m = fminf(fmaxf(m, -32768.0f), 32767.0f);
                fstat = fmaxf(fstat, fabsf(m));
                out[i] = (T)(__float_as_int(m + 12582912.0f) - 0x4B400000);   // round to nearest even
            }
        }
    }
    if (flex) {
        if (probe) {
            unsigned bits = __float_as_uint(fmax);
            for (int o = 16; o > 0; o >>= 1) bits = max(bits, __shfl_xor_sync(0xffffffffu, bits, o));
            if ((threadIdx.x & 31) == 0 && bits) atomicMax(probe_out, (unsigned long long)bits);
        } else {
            int stat = (int)rintf(fstat);
            for (int o = 16; o > 0; o >>= 1) stat = max(stat, __shfl_xor_sync(0xffffffffu, stat, o));
            if ((threadIdx.x & 31) == 0 && stat) atomicMax(stats + slot, stat);
        }
    }
}

__global__ void rng_advance_kernel(unsigned long long* counter) { *counter += 1; }

}  // namespace

extern "C" int b2_rng_fill(void* out, int32_t flex, int64_t n, int32_t distribution, float a,
                           float b, uint64_t seed, uint64_t offset, uint64_t* device_counter,
                           const b2_flex_scale* table, int32_t slot, int32_t* stats,
                           uint64_t* probe_out, int32_t probe, void* stream) {
    B2_REQUIRE(out && n >= 0, "bad argument");
    B2_REQUIRE(distribution == B2_RNG_UNIFORM || distribution == B2_RNG_NORMAL,
               "unsupported distribution: %d", distribution);
    if (flex) {
        B2_REQUIRE(table && slot >= 0, "a flex16 fill needs the scale table");
        B2_REQUIRE(probe ? probe_out != nullptr : stats != nullptr, "missing statistics destination");
    }
    if (n == 0) return B2_OK;
    long long blocks = ((n + 3) / 4 + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int normal = distribution == B2_RNG_NORMAL;
    if (flex)
        rng_fill_kernel<short><<<(unsigned)blocks, 256, 0, st>>>(
            (short*)out, n, normal, a, b, seed, offset, (const unsigned long long*)device_counter,
            table, slot, stats, (unsigned long long*)probe_out, probe ? 1 : 0);
    else
        rng_fill_kernel<float><<<(unsigned)blocks, 256, 0, st>>>(
            (float*)out, n, normal, a, b, seed, offset, (const unsigned long long*)device_counter,
            nullptr, -1, nullptr, nullptr, 0);
    B2_CUDA(cudaGetLastError());
    // a probe launch measures the very numbers the storing launch will write: same counter
    if (device_counter && !probe) {
        rng_advance_kernel<<<1, 1, 0, st>>>((unsigned long long*)device_counter);
        B2_CUDA(cudaGetLastError());
    }
    return B2_OK;
}
