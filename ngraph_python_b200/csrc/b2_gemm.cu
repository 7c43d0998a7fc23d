// C-ABI entry points of the dense GEMM (the kernels and their launch helpers are in
// b2_gemm_impl.cuh, which the convolution entry points share).
#define B2_GEMM_OWNS_TILE_KERNEL
#include "b2_gemm_impl.cuh"

int b2_gemm_launch_on_planes(int mode, unsigned char* base, const void* shapes, const void* params,
                             cudaStream_t st, int splits, void* workspace) {
    const Shapes& s = *static_cast<const Shapes*>(shapes);
    const GemmParams& p = *static_cast<const GemmParams*>(params);
    return mode == MODE_FLEX16
        ? launch_on_planes<MODE_FLEX16>(base, s, p, st, splits, workspace)
        : launch_on_planes<MODE_F32X3>(base, s, p, st, splits, workspace);
}

extern "C" int b2_gemm_scratch_bytes(int32_t flex, int32_t M, int32_t N, int32_t K, size_t* bytes) {
    B2_REQUIRE(bytes && M > 0 && N > 0 && K > 0, "bad argument");
    const int mode = flex ? MODE_FLEX16 : MODE_F32X3;
    *bytes = gemm_scratch_need(mode, shapes_for(mode, M, N, K));
    return B2_OK;
}

extern "C" int b2_gemm_f32(const float* A, int64_t a_row_stride, int64_t a_k_stride, const float* B,
                           int64_t b_k_stride, int64_t b_col_stride, float* C, int64_t ldc,
                           int32_t M, int32_t N, int32_t K, void* scratch, size_t scratch_bytes,
                           int32_t* status, void* stream) {
    return run_gemm<float, MODE_F32X3>(A, a_row_stride, a_k_stride, B, b_k_stride, b_col_stride, C,
                                       ldc, M, N, K, nullptr, 0, 0, 0, nullptr, scratch,
                                       scratch_bytes, nullptr, status, 0, (cudaStream_t)stream);
}

extern "C" int b2_gemm_flex16(const int16_t* A, int64_t a_row_stride, int64_t a_k_stride,
                              const int16_t* B, int64_t b_k_stride, int64_t b_col_stride,
                              int16_t* C, int64_t ldc, int32_t M, int32_t N, int32_t K,
                              const b2_flex_scale* table, int32_t slotA, int32_t slotB,
                              int32_t slotC, int32_t* stats, void* scratch, size_t scratch_bytes,
                              uint64_t* probe_out, int32_t* status, int32_t probe, void* stream) {
    B2_REQUIRE(table && slotA >= 0 && slotB >= 0 && slotC >= 0, "flex GEMM needs the scale table");
    B2_REQUIRE(probe ? probe_out != nullptr : stats != nullptr, "missing statistics destination");
    return run_gemm<short, MODE_FLEX16>(A, a_row_stride, a_k_stride, B, b_k_stride, b_col_stride, C,
                                        ldc, M, N, K, table, slotA, slotB, slotC, stats, scratch,
                                        scratch_bytes, (unsigned long long*)probe_out, status,
                                        probe ? 1 : 0, (cudaStream_t)stream);
}

// ---- self-test of the bounded-wait path ----------------------------------------------------------
// Every device-side wait of the tile kernels (on an mbarrier that a TMA copy, an MMA commit or
// another warp completes) gives up after a fixed number of polls, sets the caller's status word
// and lets the kernel finish normally -- tensor memory freed, nothing left spinning.  This kernel
// runs exactly that path on purpose and harmlessly: it waits, with the kernels' own wait routine,
// on a barrier that nothing will ever complete, for `poll_limit` polls, then reports and cleans up
// as the tile kernels do.  No fault, no trap, no endless loop: the context stays usable.
namespace {
__global__ void __launch_bounds__(64)
bounded_wait_selftest_kernel(int poll_limit, int* status, int* waited_out) {
    __shared__ unsigned long long bar;
    __shared__ unsigned holder;
    __shared__ int failed;
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);                    // one arrival expected; nobody arrives
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) tmem_alloc(&holder, 32);    // held across the wait, like the tile kernels
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (threadIdx.x == 32 && !mbar_wait_limit(&bar, 0, poll_limit)) atomicExch(&failed, 1);
    __syncthreads();
    if (threadIdx.x == 0 && failed) {
        if (status) atomicExch(status, 1);
        if (waited_out) *waited_out = poll_limit;
    }
    if (warp == 0) tmem_dealloc(holder, 32);
}
}  // namespace

extern "C" int b2_selftest_bounded_wait(int32_t poll_limit, int32_t* status, int32_t* polls_waited,
                                        void* stream) {
    B2_REQUIRE(poll_limit > 0 && poll_limit <= (1 << 16), "poll limit must be in 1..65536");
    B2_REQUIRE(status, "null status word");
    bounded_wait_selftest_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(poll_limit, status, polls_waited);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}
