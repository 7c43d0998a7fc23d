// N-d strided copy / transpose ("dimshuffle").
//
// Takes the place of DimShuffleKernel and the generated copy_transpose kernels
// (ngraph/transformers/gpu/tensor_ops.py:119-204, gpu/kernels/cuda/copy_transpose.py:78-282): a
// copy between two tensors of the same extents whose axes lie in different orders in memory, any
// rank.  The reference generates one kernel per shape with magic-number index arithmetic; here one
// compiled kernel takes the (collapsed) extents and both stride sets as arguments.
//
// The host first drops axes of extent 1 and merges neighbours that both tensors walk
// contiguously.  Then:
//   * if the axis that is contiguous in the source is also the contiguous one in the destination
//     (or no transposition is involved), threads run along it: both sides coalesced, the other
//     axes come from the block index;
//   * otherwise the plane spanned by the source-contiguous axis x and the destination-contiguous
//     axis y is cut into 32 x 32 tiles that go through shared memory (33-word rows, no bank
//     conflicts): loads run along x, stores along y, both in full 128-byte (64-byte for 16-bit
//     elements) rows.  Every block loops over its share of (tile, other axes) combinations.
// The kernel is bandwidth-bound: bytes moved = 2 x tensor size.
#include <cstdint>

#include "b2_common.h"

namespace {

constexpr int kMaxRank = B2_DIMSHUFFLE_MAX_RANK;

struct ShuffleParams {
    int rank;                 // collapsed rank, >= 1
    int ax, ay;               // tile axes (ay < 0: plain copy along ax)
    long long len[kMaxRank];
    long long ss[kMaxRank];   // source strides (elements)
    long long ds[kMaxRank];   // destination strides (elements)
    long long tiles_x, tiles_y, outer;   // outer = product of the other extents
};

template <typename T>
__global__ void __launch_bounds__(256)
dimshuffle_tiled_kernel(const T* __restrict__ src, T* __restrict__ dst, ShuffleParams p) {
    __shared__ T tile[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;      // 32 x 8
    const long long per_outer = p.tiles_x * p.tiles_y;
    const long long total = per_outer * p.outer;
    for (long long b = blockIdx.x; b < total; b += gridDim.x) {
        long long o = b / per_outer;
        const long long t = b - o * per_outer;
        const long long tyi = t / p.tiles_x, txi = t - tyi * p.tiles_x;
        long long soff = 0, doff = 0;
        for (int a = p.rank - 1; a >= 0; --a) {
            if (a == p.ax || a == p.ay) continue;
            const long long i = o % p.len[a];
            o /= p.len[a];
            soff += i * p.ss[a];
            doff += i * p.ds[a];
        }
        const long long x0 = txi * 32, y0 = tyi * 32;
        // load: lanes along x (contiguous in the source)
        {
            const long long x = x0 + tx;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const long long y = y0 + ty + 8 * j;
                if (x < p.len[p.ax] && y < p.len[p.ay])
                    tile[ty + 8 * j][tx] = src[soff + x * p.ss[p.ax] + y * p.ss[p.ay]];
            }
        }
        __syncthreads();
        // store: lanes along y (contiguous in the destination)
        {
            const long long y = y0 + tx;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const long long x = x0 + ty + 8 * j;
                if (x < p.len[p.ax] && y < p.len[p.ay])
                    dst[doff + x * p.ds[p.ax] + y * p.ds[p.ay]] = tile[tx][ty + 8 * j];
            }
        }
        __syncthreads();
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
dimshuffle_rows_kernel(const T* __restrict__ src, T* __restrict__ dst, ShuffleParams p) {
    // threads along axis ax in chunks of 256; the other axes from the block index
    const long long chunks = p.tiles_x;
    const long long total = chunks * p.outer;
    for (long long b = blockIdx.x; b < total; b += gridDim.x) {
        long long o = b / chunks;
        const long long x = (b - o * chunks) * 256 + threadIdx.x;
        long long soff = 0, doff = 0;
        for (int a = p.rank - 1; a >= 0; --a) {
            if (a == p.ax) continue;
            const long long i = o % p.len[a];
            o /= p.len[a];
            soff += i * p.ss[a];
            doff += i * p.ds[a];
        }
        if (x < p.len[p.ax]) dst[doff + x * p.ds[p.ax]] = src[soff + x * p.ss[p.ax]];
    }
}

template <typename T>
int launch(const void* src, void* dst, const ShuffleParams& p, cudaStream_t st) {
    long long blocks;
    if (p.ay >= 0) blocks = p.tiles_x * p.tiles_y * p.outer;
    else blocks = p.tiles_x * p.outer;
    const long long cap = 148LL * 32;
    const unsigned grid = (unsigned)(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
    if (p.ay >= 0)
        dimshuffle_tiled_kernel<T><<<grid, 256, 0, st>>>((const T*)src, (T*)dst, p);
    else
        dimshuffle_rows_kernel<T><<<grid, 256, 0, st>>>((const T*)src, (T*)dst, p);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

}  // namespace

extern "C" int b2_dimshuffle(const void* src, void* dst, int32_t elem_bytes, int32_t rank,
                             const int64_t* shape, const int64_t* src_strides,
                             const int64_t* dst_strides, void* stream) {
    B2_REQUIRE(src && dst, "null tensor");
    B2_REQUIRE(rank >= 0 && rank <= kMaxRank, "rank %d outside 0..%d", rank, kMaxRank);
    B2_REQUIRE(rank == 0 || (shape && src_strides && dst_strides), "null shape or strides");
    B2_REQUIRE(elem_bytes == 1 || elem_bytes == 2 || elem_bytes == 4 || elem_bytes == 8,
               "element size %d is not 1, 2, 4 or 8 bytes", elem_bytes);
    // drop unit axes, merge neighbours both tensors walk contiguously
    ShuffleParams p;
    p.rank = 0;
    for (int a = 0; a < rank; ++a) {
        B2_REQUIRE(shape[a] >= 0 && dst_strides[a] >= 0 && src_strides[a] >= 0,
                   "negative extent or stride");
        if (shape[a] == 0) return B2_OK;
        if (shape[a] == 1) continue;
        const int q = p.rank;
        if (q > 0 && p.ss[q - 1] == src_strides[a] * shape[a] &&
            p.ds[q - 1] == dst_strides[a] * shape[a]) {
            p.len[q - 1] *= shape[a];
            p.ss[q - 1] = src_strides[a];
            p.ds[q - 1] = dst_strides[a];
        } else {
            p.len[q] = shape[a]; p.ss[q] = src_strides[a]; p.ds[q] = dst_strides[a];
            ++p.rank;
        }
    }
    if (p.rank == 0) { p.rank = 1; p.len[0] = 1; p.ss[0] = 1; p.ds[0] = 1; }
    // axis contiguous in the source / in the destination (smallest non-zero stride otherwise)
    int sx = -1, dx = -1;
    for (int a = 0; a < p.rank; ++a) {
        if (p.ss[a] > 0 && (sx < 0 || p.ss[a] < p.ss[sx])) sx = a;
        if (dx < 0 || p.ds[a] < p.ds[dx]) dx = a;
    }
    if (sx < 0) sx = dx;                               // source broadcast along every axis
    long long outer = 1;
    if (sx == dx || p.ds[dx] != 1 || p.ss[sx] != 1) {
        // no transposition to tile: run along the destination's fastest axis
        p.ax = dx; p.ay = -1;
        p.tiles_x = (p.len[dx] + 255) / 256; p.tiles_y = 1;
        for (int a = 0; a < p.rank; ++a) if (a != dx) outer *= p.len[a];
    } else {
        p.ax = sx; p.ay = dx;
        p.tiles_x = (p.len[sx] + 31) / 32; p.tiles_y = (p.len[dx] + 31) / 32;
        for (int a = 0; a < p.rank; ++a) if (a != sx && a != dx) outer *= p.len[a];
    }
    p.outer = outer;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (elem_bytes) {
        case 1: return launch<uint8_t>(src, dst, p, st);
        case 2: return launch<uint16_t>(src, dst, p, st);
        case 4: return launch<uint32_t>(src, dst, p, st);
        default: return launch<unsigned long long>(src, dst, p, st);
    }
}
