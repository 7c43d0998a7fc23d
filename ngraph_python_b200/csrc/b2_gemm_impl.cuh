// Dense GEMM on the 5th-generation tensor cores: C[M,N] = op(A)[M,K] * op(B)[K,N]
//
// Takes the place of the reference's GEMMKernel and its maxas SASS kernels
// (ngraph/transformers/gpu/gemm.py:26-263, gpu/kernels/sass/sgemm_*.sass, fgemm_*.sass).
//
//   flex16: operands are int16 mantissas.  Each is split exactly into a signed high byte and an
//           unsigned low byte, a = 256*ah + al, and the product is formed from four int8 tensor-core
//           products with int32 accumulation in tensor memory:
//               sum a*b = 65536*sum(ah*bh) + 256*(sum(ah*bl) + sum(al*bh)) + sum(al*bl)
//           Three accumulators (HH, cross, LL) stay exact in int32 for K <= 32768; the epilogue
//           recombines them in int64, applies the power-of-two rescale 2^(decC-decA-decB) with
//           round-to-nearest-even in integer arithmetic, saturates to int16 and folds max|mantissa|.
//           (The reference accumulates int16 products in fp32 FFMA, fgemm_common_128x128.sass:
//           188-228, which is inexact above 2^24; this path is exact.)
//           When the caller supplies row sums of A ("merged" form, used by the dense GEMM entry
//           point) the low plane of B is stored as the signed byte bl - 128, so that both planes of
//           B are signed and lie behind one another in shared memory as ONE 2*BN-row operand:
//               A_hi x [B_hi | B_lo'] -> HH | X          A_lo x [B_hi | B_lo'] -> X | LL
//           two N = 2*BN instructions per k-step instead of four of N = BN (a quarter less operand
//           traffic from shared memory); the epilogue adds back 128 * sum_k a[m,k].
//   fp32:   3xTF32: a = a_hi + a_lo with a_hi rounded to tf32, and
//               a*b ~= a_hi*b_hi + a_hi*b_lo + a_lo*b_hi        (relative error ~2^-21)
//           three kind::tf32 products into one fp32 accumulator.  The tensor core's fp32
//           accumulation truncates, and the bias grows with the length of the accumulation
//           chain (measured: 5e-4 relative at K = 40000), so the chain is cut every 16 k-blocks
//           (512 elements): the MMA warp alternates between two accumulator buffers in tensor
//           memory and the epilogue warps add each finished buffer into registers with ordinary
//           round-to-nearest fp32 adds while the next chunk is being multiplied.
//
// Structure of the main kernel (one CTA per 128x128 output tile, 192 threads):
//   warp 0   : TMA producer -- 2-D tiled bulk tensor copies of the four operand planes of a
//              k-block (4 x 16 KB, 128-byte swizzle) into a 3-stage shared-memory ring;
//   warp 1   : allocates tensor memory, one lane issues tcgen05.mma (8, 12 or 16 per k-block) and
//              commits each stage back to the producer;
//   warps 2-5: epilogue -- tcgen05.ld of the accumulators (each warp owns 32 lanes = 32 rows),
//              recombination / rescale / store.
// A pre-pass writes the operand planes K-major (and transposes when the source is not), zero
// padded to tile multiples, into caller-provided scratch.
//
// Every mbarrier wait is bounded; when one runs out the kernel records it in `status` and
// finishes without hanging.  No cluster multicast is used anywhere.
#ifndef B2_GEMM_IMPL_CUH
#define B2_GEMM_IMPL_CUH
#include <cuda.h>

#include <mutex>

#include "b2_common.h"

// The tile kernel is compiled once, in the translation unit that defines B2_GEMM_OWNS_TILE_KERNEL
// (b2_gemm.cu); every other includer reaches it through this function.  Shapes and GemmParams
// live in this header's unnamed namespace -- each translation unit has its own, identical, type --
// so they cross the boundary as untyped pointers.
__attribute__((visibility("hidden")))
int b2_gemm_launch_on_planes(int mode, unsigned char* base, const void* shapes, const void* params,
                             cudaStream_t st, int splits, void* workspace);

namespace {

constexpr int kBlockM = 128;          // UMMA M; the N tile (16/32/64/128) is a template parameter
constexpr int kKBytes = 128;            // bytes of K per k-block row: one 128B swizzle atom
constexpr int kPlaneBytes = 128 * kKBytes;   // 16 KB: 128 rows x 128 B
__host__ __device__ constexpr int stage_bytes(int bn) { return 2 * kPlaneBytes + 2 * bn * kKBytes; }  // A0 A1 B0 B1
constexpr int kStages = 3;
constexpr int kThreads = 192;
__host__ __device__ constexpr int smem_bytes(int bn) { return kStages * stage_bytes(bn) + 1024 /*alignment*/ + 256 /*barriers*/; }
// tensor-memory columns: a power of two >= 32 that holds the accumulators (3 x BN or BN)
__host__ __device__ constexpr int tmem_cols(int mode, int bn) {
    int need = (mode == 0 ? 3 : 1) * bn, c = 32;
    while (c < need) c *= 2;
    return c;
}
// the dense GEMM kernel keeps two fp32 accumulator buffers (see the head of this file)
__host__ __device__ constexpr int gemm_tmem_cols(int mode, int bn) {
    return mode == 0 ? tmem_cols(0, bn) : tmem_cols(1, 2 * bn);
}
constexpr int kChunkKb = 16;            // fp32: k-blocks per accumulation chain

enum { MODE_FLEX16 = 0, MODE_F32X3 = 1 };

// ---- PTX wrappers ------------------------------------------------------------------------------
__device__ __forceinline__ unsigned smem_u32(const void* p) {
    return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait: gives up after `limit` polls (each poll suspends up to a hardware time limit)
__device__ __forceinline__ bool mbar_wait_limit(unsigned long long* bar, unsigned parity, int limit) {
    for (int i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
constexpr int kWaitPolls = 1 << 20;     // what every wait of the kernels allows itself
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
    return mbar_wait_limit(bar, parity, kWaitPolls);
}
// the same for warps that wait long and share an instruction scheduler with the MMA-issuing
// thread: back off between polls so that the polling does not take its issue slots
__device__ __forceinline__ bool mbar_wait_relaxed(unsigned long long* bar, unsigned parity) {
    for (int i = 0; i < (1 << 20); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(64);
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y,
                                            unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_alloc(unsigned* holder, unsigned cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(holder)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(unsigned taddr, unsigned cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(smem_u32(bar)) : "memory");
}
template <int MODE>
__device__ __forceinline__ void tc_mma(unsigned tmem_d, unsigned long long adesc,
                                       unsigned long long bdesc, unsigned idesc, unsigned accumulate) {
    if (MODE == MODE_FLEX16) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
    }
}
// 16 consecutive 32-bit columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld16(unsigned taddr, unsigned* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 B stored
// consecutively (8-row groups 1024 B apart).  Fields: start>>4 [0,14), LBO>>4 [16,30) (=1 for
// swizzled K-major), SBO>>4 [32,46) (=64), version [46,48) = 1, layout type [61,64) = 2.
__device__ __forceinline__ unsigned long long make_smem_desc(const void* p) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_u32(p) >> 4) & 0x3FFF);
    d |= (unsigned long long)1 << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= (unsigned long long)1 << 46;
    d |= (unsigned long long)2 << 61;
    return d;
}
// Instruction descriptor: D format [4,6), A format [7,10), B format [10,13), K-major both,
// N>>3 [17,23), M>>4 [24,29).
__host__ __device__ constexpr unsigned make_idesc(unsigned dfmt, unsigned afmt, unsigned bfmt,
                                                  unsigned bn) {
    return (dfmt << 4) | (afmt << 7) | (bfmt << 10) | ((bn >> 3) << 17) |
           ((unsigned)(kBlockM >> 4) << 24);
}

struct GemmParams {
    int M, N, num_kb;
    long long ldc;
    void* C;
    const b2_flex_scale* table;
    int slotA, slotB, slotC;
    int* stats;
    unsigned long long* probe_out;   // probe: max |exact integer product sum|
    int* status;
    int probe;
    int c_colmajor;                  // 0: C[row*ldc + col]; 1: C[col*ldc + row]
    const int* rowsum;               // flex16 merged form: sum_k a[m,k] per row of A, else null
    // split-K: grid.z slices of kb_per_split k-blocks each write raw sums (int64 for flex16, float
    // for fp32) to partial[z][Mp][Np]; splitk_finish_kernel adds the slices in a fixed order
    void* partial;
    int kb_per_split, Mp, Np;
};

// round-to-nearest-even of v / 2^sh (sh > 0), or v * 2^-sh (sh <= 0), saturated to int16
__device__ __forceinline__ int rescale_i64(long long v, int sh) {
    long long q;
    if (sh <= 0) {
        // scale up: anything with |v| >= 2^16 saturates for every left shift
        const int l = -sh;
        const long long a = v < 0 ? -v : v;
        if (a >= 65536 || (l >= 16 && a != 0)) q = v > 0 ? 32767 : -32768;
        else q = v << l;
    } else if (sh >= 62) {
        q = 0;
    } else {
        const long long half = 1LL << (sh - 1);
        const long long lsb = (v >> sh) & 1;
        q = (v + half - 1 + lsb) >> sh;
    }
    q = q > 32767 ? 32767 : (q < -32768 ? -32768 : q);
    return (int)q;
}

// The same for 1 <= sh <= 31 (every realistic exponent combination) in 32-bit pieces: the low
// word of v >> sh by a funnel shift, the remainder by a mask, the tie rule from both, and the
// saturation from whether the 64-bit quotient is the sign extension of its low word.
// About a third of the instructions of the general form; callers test the range once per kernel.
__device__ __forceinline__ int rescale_i64_fast(long long v, int sh, unsigned mask, unsigned half) {
    const unsigned lo = (unsigned)v;
    const int hi = (int)(v >> 32);
    const unsigned q0lo = __funnelshift_r(lo, (unsigned)hi, sh);   // low word of floor(v / 2^sh)
    const int q0hi = hi >> sh;
    const unsigned rem = lo & mask;
    const unsigned up = (rem > half || (rem == half && (q0lo & 1u))) ? 1u : 0u;
    const unsigned qlo = q0lo + up;
    const int qhi = q0hi + (qlo < up ? 1 : 0);
    const int q32 = (int)qlo;
    if (qhi != (q32 >> 31)) return qhi < 0 ? -32768 : 32767;
    return q32 > 32767 ? 32767 : (q32 < -32768 ? -32768 : q32);
}

template <int MODE, int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap mapA0, const __grid_constant__ CUtensorMap mapA1,
            const __grid_constant__ CUtensorMap mapB0, const __grid_constant__ CUtensorMap mapB1,
            const GemmParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    constexpr int kStageBytes = stage_bytes(BN);
    constexpr int kBPlane = BN * kKBytes;
    constexpr int kTmemCols = gemm_tmem_cols(MODE, BN);
    unsigned long long* full_bar = (unsigned long long*)(smem + kStages * kStageBytes);
    unsigned long long* empty_bar = full_bar + kStages;
    unsigned long long* tmem_full = empty_bar + kStages;        // [2]
    unsigned long long* tmem_empty = tmem_full + 2;             // [2] (fp32 only)
    unsigned* tmem_holder = (unsigned*)(tmem_empty + 2);
    int* fail_flag = (int*)(tmem_holder + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * kBlockM, n0 = blockIdx.x * BN;
    const int kElems = MODE == MODE_FLEX16 ? kKBytes : kKBytes / 4;   // elements of K per k-block
    const int kb0 = p.partial ? blockIdx.z * p.kb_per_split : 0;
    const int nkb = p.partial ? min(p.kb_per_split, p.num_kb - kb0) : p.num_kb;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&tmem_full[b], 1); mbar_init(&tmem_empty[b], 4); }
        *fail_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_holder, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_holder;

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % kStages;
                if (kb >= kStages && !mbar_wait(&empty_bar[s], ((kb / kStages) - 1) & 1)) {
                    atomicExch(fail_flag, 1);
                    break;
                }
                unsigned char* st = smem + s * kStageBytes;
                mbar_expect_tx(&full_bar[s], kStageBytes);
                const int kx = (kb0 + kb) * kElems;
                tma_load_2d(st + 0 * kPlaneBytes, &mapA0, kx, m0, &full_bar[s]);
                tma_load_2d(st + 1 * kPlaneBytes, &mapA1, kx, m0, &full_bar[s]);
                tma_load_2d(st + 2 * kPlaneBytes, &mapB0, kx, n0, &full_bar[s]);
                tma_load_2d(st + 2 * kPlaneBytes + kBPlane, &mapB1, kx, n0, &full_bar[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // flex16: planes are (hi = signed, lo = unsigned) bytes; accumulators HH | X | LL
            const unsigned id_ss = make_idesc(2, 1, 1, BN), id_su = make_idesc(2, 1, 0, BN),
                           id_us = make_idesc(2, 0, 1, BN), id_uu = make_idesc(2, 0, 0, BN);
            const unsigned id_tf = make_idesc(1, 2, 2, BN);
            const unsigned id_ss2 = make_idesc(2, 1, 1, 2 * BN), id_us2 = make_idesc(2, 0, 1, 2 * BN);
            const bool merged = MODE == MODE_FLEX16 && p.rowsum != nullptr;
            bool ok = true;
            for (int kb = 0; kb < nkb && ok; ++kb) {
                const int s = kb % kStages;
                if (!mbar_wait(&full_bar[s], (kb / kStages) & 1)) { atomicExch(fail_flag, 1); ok = false; break; }
                tc_fence_after();
                unsigned char* st = smem + s * kStageBytes;
                const unsigned long long dA0 = make_smem_desc(st + 0 * kPlaneBytes);
                const unsigned long long dA1 = make_smem_desc(st + 1 * kPlaneBytes);
                const unsigned long long dB0 = make_smem_desc(st + 2 * kPlaneBytes);
                const unsigned long long dB1 = make_smem_desc(st + 2 * kPlaneBytes + kBPlane);
                // fp32: accumulation chains of kChunkKb k-blocks alternate between two buffers
                const int chunk = MODE == MODE_F32X3 ? kb / kChunkKb : 0;
                const int kin = MODE == MODE_F32X3 ? kb % kChunkKb : kb;
                const unsigned tmem_acc = tmem_base + (MODE == MODE_F32X3 ? (chunk & 1) * BN : 0);
                if (MODE == MODE_F32X3 && kin == 0 && chunk >= 2) {
                    if (!mbar_wait(&tmem_empty[chunk & 1], ((chunk >> 1) - 1) & 1)) {
                        atomicExch(fail_flag, 1); ok = false; break;
                    }
                    tc_fence_after();
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const unsigned long long adv = (unsigned long long)((k * 32) >> 4);
                    const unsigned acc = (kin > 0 || k > 0) ? 1u : 0u;
                    if (merged && acc) {
                        // B_hi and B_lo' are adjacent: one descriptor spans both
                        tc_mma<MODE>(tmem_base + 0, dA0 + adv, dB0 + adv, id_ss2, 1u);      // HH | X
                        tc_mma<MODE>(tmem_base + BN, dA1 + adv, dB0 + adv, id_us2, 1u);     // X | LL
                    } else if (merged) {
                        // first k-step: the three accumulators start from different instructions
                        tc_mma<MODE>(tmem_base + 0, dA0 + adv, dB0 + adv, id_ss, 0u);
                        tc_mma<MODE>(tmem_base + BN, dA0 + adv, dB1 + adv, id_ss, 0u);
                        tc_mma<MODE>(tmem_base + BN, dA1 + adv, dB0 + adv, id_us, 1u);
                        tc_mma<MODE>(tmem_base + 2 * BN, dA1 + adv, dB1 + adv, id_us, 0u);
                    } else if (MODE == MODE_FLEX16) {
                        tc_mma<MODE>(tmem_base + 0, dA0 + adv, dB0 + adv, id_ss, acc);      // HH
                        tc_mma<MODE>(tmem_base + BN, dA0 + adv, dB1 + adv, id_su, acc);     // X += ah*bl
                        tc_mma<MODE>(tmem_base + BN, dA1 + adv, dB0 + adv, id_us, 1u);      // X += al*bh
                        tc_mma<MODE>(tmem_base + 2 * BN, dA1 + adv, dB1 + adv, id_uu, acc); // LL
                    } else {
                        tc_mma<MODE>(tmem_acc, dA0 + adv, dB0 + adv, id_tf, acc);           // hi*hi
                        tc_mma<MODE>(tmem_acc, dA0 + adv, dB1 + adv, id_tf, 1u);            // hi*lo
                        tc_mma<MODE>(tmem_acc, dA1 + adv, dB0 + adv, id_tf, 1u);            // lo*hi
                    }
                }
                tc_commit(&empty_bar[s]);       // stage reusable once these MMAs have read it
                if (MODE == MODE_F32X3 && (kin == kChunkKb - 1 || kb == nkb - 1))
                    tc_commit(&tmem_full[chunk & 1]);      // this chain is complete
            }
            if (MODE == MODE_FLEX16) tc_commit(&tmem_full[0]);     // accumulators complete
        }
    } else {
        // epilogue warps 2..5: TMEM lane quarter = warp % 4
        const int quarter = warp & 3;
        const int row = m0 + quarter * 32 + lane;
        bool ok = true;
        if (MODE == MODE_FLEX16) {
            ok = mbar_wait(&tmem_full[0], 0);
            if (!ok) atomicExch(fail_flag, 1);
            tc_fence_after();
        }
        const unsigned lane_addr = tmem_base + ((unsigned)(quarter * 32) << 16);
        if (MODE == MODE_FLEX16) {
            const float f = p.table[p.slotA].scale * p.table[p.slotB].scale *
                            (p.probe ? 1.0f : p.table[p.slotC].inv_scale);
            const int sh = -ilogbf(f);          // f = 2^-sh exactly
            const bool fast = sh >= 1 && sh <= 31;
            const unsigned rmask = fast ? (1u << sh) - 1u : 0u, rhalf = fast ? 1u << (sh - 1) : 0u;
            int stat = 0;
            unsigned long long pmax = 0;
            short* crow = (short*)p.C + (long long)row * p.ldc;
            // the row-sum term belongs to the whole contraction: slice 0 carries it
            const long long fix = (p.rowsum && row < p.M && (!p.partial || blockIdx.z == 0))
                                      ? 128LL * (long long)p.rowsum[row] : 0LL;
            for (int c0 = 0; c0 < BN; c0 += 16) {
                unsigned hh[16], xx[16], ll[16];
                tmem_ld16(lane_addr + c0, hh);
                tmem_ld16(lane_addr + BN + c0, xx);
                tmem_ld16(lane_addr + 2 * BN + c0, ll);
                tmem_ld_wait();
                if (!ok || row >= p.M) continue;
                if (p.partial) {
                    long long* dst = (long long*)p.partial +
                                     ((long long)blockIdx.z * p.Mp + row) * p.Np + n0 + c0;
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        dst[j] = ((long long)(int)hh[j] << 16) + ((long long)(int)xx[j] << 8) +
                                 (long long)(int)ll[j] + fix;
                    continue;
                }
                int q[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const long long v = ((long long)(int)hh[j] << 16) + ((long long)(int)xx[j] << 8) +
                                        (long long)(int)ll[j] + fix;
                    if (p.probe) {
                        const unsigned long long a = (unsigned long long)(v < 0 ? -v : v);
                        pmax = a > pmax ? a : pmax;
                    } else {
                        q[j] = fast ? rescale_i64_fast(v, sh, rmask, rhalf) : rescale_i64(v, sh);
                        const int a = q[j] < 0 ? -q[j] : q[j];
                        stat = a > stat ? a : stat;
                    }
                }
                if (!p.probe) {
                    const int col = n0 + c0;
                    if (p.c_colmajor) {
                        // lanes hold consecutive rows: each column is a coalesced 64-byte store
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (col + j < p.N)
                                ((short*)p.C)[(long long)(col + j) * p.ldc + row] = (short)q[j];
                    } else if (col + 16 <= p.N && ((p.ldc & 7) == 0) && (((uintptr_t)p.C & 15) == 0)) {
                        int4 w0, w1;
                        w0.x = (q[0] & 0xffff) | (q[1] << 16); w0.y = (q[2] & 0xffff) | (q[3] << 16);
                        w0.z = (q[4] & 0xffff) | (q[5] << 16); w0.w = (q[6] & 0xffff) | (q[7] << 16);
                        w1.x = (q[8] & 0xffff) | (q[9] << 16); w1.y = (q[10] & 0xffff) | (q[11] << 16);
                        w1.z = (q[12] & 0xffff) | (q[13] << 16); w1.w = (q[14] & 0xffff) | (q[15] << 16);
                        *reinterpret_cast<int4*>(crow + col) = w0;
                        *reinterpret_cast<int4*>(crow + col + 8) = w1;
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (col + j < p.N) crow[col + j] = (short)q[j];
                    }
                }
            }
            if (p.partial) {
                // statistics are taken by the finishing kernel
            } else if (p.probe) {
                for (int o = 16; o > 0; o >>= 1) {
                    const unsigned long long t = __shfl_xor_sync(0xffffffffu, pmax, o);
                    pmax = t > pmax ? t : pmax;
                }
                if (lane == 0 && pmax) atomicMax(p.probe_out, pmax);
            } else {
                for (int o = 16; o > 0; o >>= 1) {
                    const int t = __shfl_xor_sync(0xffffffffu, stat, o);
                    stat = t > stat ? t : stat;
                }
                if (lane == 0 && stat) atomicMax(p.stats + p.slotC, stat);
            }
        } else {
            // add every finished accumulation chain into registers (round-to-nearest adds)
            float sum[BN];
#pragma unroll
            for (int j = 0; j < BN; ++j) sum[j] = 0.f;
            const int nchunks = (nkb + kChunkKb - 1) / kChunkKb;
            for (int chunk = 0; chunk < nchunks; ++chunk) {
                const int b = chunk & 1;
                if (ok && !mbar_wait(&tmem_full[b], (chunk >> 1) & 1)) {
                    atomicExch(fail_flag, 1);
                    ok = false;
                }
                tc_fence_after();
#pragma unroll
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    unsigned acc[16];
                    tmem_ld16(lane_addr + b * BN + c0, acc);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) sum[c0 + j] += __uint_as_float(acc[j]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&tmem_empty[b]);
            }
            float* crow = (float*)p.C + (long long)row * p.ldc;
            if (ok && row < p.M) {
#pragma unroll
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    const int col = n0 + c0;
                    if (p.partial) {
                        float* dst = (float*)p.partial + ((long long)blockIdx.z * p.Mp + row) * p.Np + col;
#pragma unroll
                        for (int j = 0; j < 16; j += 4)
                            *reinterpret_cast<float4*>(dst + j) =
                                make_float4(sum[c0 + j], sum[c0 + j + 1], sum[c0 + j + 2], sum[c0 + j + 3]);
                    } else if (p.c_colmajor) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (col + j < p.N)
                                ((float*)p.C)[(long long)(col + j) * p.ldc + row] = sum[c0 + j];
                    } else if (col + 16 <= p.N && ((p.ldc & 3) == 0) && (((uintptr_t)p.C & 15) == 0)) {
#pragma unroll
                        for (int j = 0; j < 16; j += 4)
                            *reinterpret_cast<float4*>(crow + col + j) =
                                make_float4(sum[c0 + j], sum[c0 + j + 1], sum[c0 + j + 2], sum[c0 + j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (col + j < p.N) crow[col + j] = sum[c0 + j];
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
    if (threadIdx.x == 0 && *fail_flag && p.status) atomicExch(p.status, 1);
}

// ---- split-K second stage ----------------------------------------------------------------------
// Adds the slices of one output element in a fixed order (deterministic), then finishes it like
// the tile kernel's epilogue: flex16 rescale + saturate + statistics (or the probe maximum), fp32
// store.  A block of 8 warps owns 32 consecutive elements: warp w adds the slices w, w+8, ... of
// its lane's element, the eight partial sums are combined in warp order through shared memory.
template <int MODE>
__global__ void __launch_bounds__(256)
splitk_finish_kernel(const GemmParams p, int splits) {
    __shared__ long long part64[8][32];
    __shared__ float part32[8][32];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const long long total = (long long)p.M * p.N;
    const long long slice = (long long)p.Mp * p.Np;
    int stat = 0;
    unsigned long long pmax = 0;
    int sh = 0;
    if (MODE == MODE_FLEX16) {
        const float f = p.table[p.slotA].scale * p.table[p.slotB].scale *
                        (p.probe ? 1.0f : p.table[p.slotC].inv_scale);
        sh = -ilogbf(f);
    }
    for (long long base = (long long)blockIdx.x * 32; base < total; base += (long long)gridDim.x * 32) {
        const long long i = base + lane;
        const bool live = i < total;
        const int row = live ? (int)(i / p.N) : 0, col = live ? (int)(i % p.N) : 0;
        const long long src = (long long)row * p.Np + col;
        if (MODE == MODE_FLEX16) {
            long long v = 0;
            if (live)
                for (int z = w; z < splits; z += 8) v += ((const long long*)p.partial)[z * slice + src];
            part64[w][lane] = v;
        } else {
            float v = 0.f;
            if (live)
                for (int z = w; z < splits; z += 8) v += ((const float*)p.partial)[z * slice + src];
            part32[w][lane] = v;
        }
        __syncthreads();
        if (w == 0 && live) {
            const long long dst = p.c_colmajor ? (long long)col * p.ldc + row
                                               : (long long)row * p.ldc + col;
            if (MODE == MODE_FLEX16) {
                long long v = 0;
#pragma unroll
                for (int k = 0; k < 8; ++k) v += part64[k][lane];
                if (p.probe) {
                    const unsigned long long a = (unsigned long long)(v < 0 ? -v : v);
                    pmax = a > pmax ? a : pmax;
                } else {
                    const int q = rescale_i64(v, sh);
                    const int a = q < 0 ? -q : q;
                    stat = a > stat ? a : stat;
                    ((short*)p.C)[dst] = (short)q;
                }
            } else {
                float v = 0.f;
#pragma unroll
                for (int k = 0; k < 8; ++k) v += part32[k][lane];
                ((float*)p.C)[dst] = v;
            }
        }
        __syncthreads();
    }
    if (MODE == MODE_FLEX16 && w == 0) {
        if (p.probe) {
            for (int o = 16; o > 0; o >>= 1) {
                const unsigned long long t = __shfl_xor_sync(0xffffffffu, pmax, o);
                pmax = t > pmax ? t : pmax;
            }
            if (lane == 0 && pmax) atomicMax(p.probe_out, pmax);
        } else {
            for (int o = 16; o > 0; o >>= 1) {
                const int t = __shfl_xor_sync(0xffffffffu, stat, o);
                stat = t > stat ? t : stat;
            }
            if (lane == 0 && stat) atomicMax(p.stats + p.slotC, stat);
        }
    }
}

// ---- pre-pass: operand planes, K-major, zero padded ---------------------------------------------
// src element (r, k) of op(X) is src[r * rs + k * cs]; planes are [rows_p][kp] with kp contiguous.
//   flex16: plane0 = high byte (signed), plane1 = low byte XOR lo_xor (lo_xor = 0x80 stores the
//           signed byte lo - 128); rowsum (optional) accumulates sum_k of the int16 values per row.
//   fp32:   plane0 = value rounded to tf32, plane1 = remainder.
// Three kernels: K contiguous with 16-byte aligned rows (vector loads, no staging), rows contiguous
// with aligned columns (64x64 / 64x32 tiles transposed through shared memory, vector loads and
// stores), and a 32x32-tile kernel without any alignment requirement.

__device__ __forceinline__ void tf32_split(float a, float& hi, float& lo) {
    unsigned hb;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hb) : "f"(a));
    hi = __uint_as_float(hb);
    lo = a - hi;
}

__device__ __forceinline__ void add_rowsum(int* rowsum, int r, int rows, int v, int group) {
    // lanes of a group (a power of two, aligned) hold partial sums of the same row
    for (int o = group >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & (group - 1)) == 0 && r < rows && v != 0) atomicAdd(rowsum + r, v);
}

// K contiguous: one thread = 16 int16 (two 16-byte loads) or 4 floats of one row
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
split_rows_kernel(const T* __restrict__ src, long long rs, int rows, int k, int rows_p, int kp,
                  void* __restrict__ plane0, void* __restrict__ plane1, unsigned lo_xor,
                  int* __restrict__ rowsum) {
    constexpr int kPer = MODE == MODE_FLEX16 ? 16 : 4;
    const int upr = kp / kPer;                                   // units per row
    const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;
    const bool live = idx < (long long)rows_p * upr;
    const int r = live ? (int)(idx / upr) : rows_p;
    const int kk = live ? (int)(idx % upr) * kPer : 0;
    const long long o = (long long)r * kp + kk;
    if (MODE == MODE_FLEX16) {
        unsigned w[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (live && r < rows) {
            const short* sp = (const short*)src + (long long)r * rs + kk;
            if (kk + 16 <= k) {
                const int4 a = __ldg((const int4*)sp), b = __ldg((const int4*)sp + 1);
                w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
                w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
            } else {
                for (int j = 0; j < 16 && kk + j < k; ++j)
                    w[j >> 1] |= (unsigned)(unsigned short)sp[j] << ((j & 1) * 16);
            }
        }
        int sum = 0;
        unsigned hi[4], lo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            hi[j] = __byte_perm(w[2 * j], w[2 * j + 1], 0x7531);
            lo[j] = __byte_perm(w[2 * j], w[2 * j + 1], 0x6420) ^ (lo_xor * 0x01010101u);
            sum += ((int)(w[2 * j] << 16) >> 16) + ((int)w[2 * j] >> 16) +
                   ((int)(w[2 * j + 1] << 16) >> 16) + ((int)w[2 * j + 1] >> 16);
        }
        if (live) {
            *(int4*)((unsigned char*)plane0 + o) = make_int4(hi[0], hi[1], hi[2], hi[3]);
            *(int4*)((unsigned char*)plane1 + o) = make_int4(lo[0], lo[1], lo[2], lo[3]);
        }
        if (rowsum) {
            const int r0 = __shfl_sync(0xffffffffu, r, 0);
            if (__all_sync(0xffffffffu, r == r0)) add_rowsum(rowsum, r, rows, sum, 32);
            else if (r < rows && sum != 0) atomicAdd(rowsum + r, sum);
        }
    } else {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live && r < rows) {
            const float* sp = (const float*)src + (long long)r * rs + kk;
            if (kk + 4 <= k) v = __ldg((const float4*)sp);
            else {
                if (kk + 0 < k) v.x = sp[0];
                if (kk + 1 < k) v.y = sp[1];
                if (kk + 2 < k) v.z = sp[2];
            }
        }
        float4 h, l;
        tf32_split(v.x, h.x, l.x); tf32_split(v.y, h.y, l.y);
        tf32_split(v.z, h.z, l.z); tf32_split(v.w, h.w, l.w);
        if (live) {
            *(float4*)((float*)plane0 + o) = h;
            *(float4*)((float*)plane1 + o) = l;
        }
    }
}

// rows contiguous in the source (element (r, k) at src[k * cs + r]): tiles of 64 rows x 64 k
// (flex16) or 64 rows x 32 k (fp32) are read with 16-byte loads along r, transposed through shared
// memory and written with 16- / 32-byte stores along k.
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
split_cols_kernel(const T* __restrict__ src, long long cs, int rows, int k, int rows_p, int kp,
                  void* __restrict__ plane0, void* __restrict__ plane1, unsigned lo_xor,
                  int* __restrict__ rowsum) {
    constexpr int kTileK = MODE == MODE_FLEX16 ? 64 : 32;
    constexpr int kPitch = MODE == MODE_FLEX16 ? 66 : 65;       // elements; odd word pitch
    __shared__ T tile[kTileK * kPitch];
    const int tid = threadIdx.x;
    const int r0 = blockIdx.y * 64, k0 = blockIdx.x * kTileK;
    if (MODE == MODE_FLEX16) {
        // load: 8 rows per thread per k; 8 threads cover 64 rows, 32 k per pass
        for (int i = 0; i < 2; ++i) {
            const int kk = (tid >> 3) + 32 * i, r8 = (tid & 7) * 8;
            unsigned w[4] = {0, 0, 0, 0};
            if (k0 + kk < k) {
                const short* sp = (const short*)src + (long long)(k0 + kk) * cs + r0 + r8;
                if (r0 + r8 + 8 <= rows) {
                    const int4 a = __ldg((const int4*)sp);
                    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
                } else {
                    for (int j = 0; j < 8 && r0 + r8 + j < rows; ++j)
                        w[j >> 1] |= (unsigned)(unsigned short)sp[j] << ((j & 1) * 16);
                }
            }
            unsigned* dst = (unsigned*)((short*)tile + kk * kPitch + r8);
            dst[0] = w[0]; dst[1] = w[1]; dst[2] = w[2]; dst[3] = w[3];
        }
        __syncthreads();
        const int r = tid >> 2, kc = (tid & 3) * 16;
        unsigned hi[4], lo[4];
        int sum = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            unsigned h = 0, l = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int m = ((short*)tile)[(kc + 4 * j + b) * kPitch + r];
                sum += m;
                l |= (unsigned)(m & 0xff) << (8 * b);
                h |= (unsigned)((m >> 8) & 0xff) << (8 * b);
            }
            hi[j] = h;
            lo[j] = l ^ (lo_xor * 0x01010101u);
        }
        if (r0 + r < rows_p && k0 + kc < kp) {
            const long long o = (long long)(r0 + r) * kp + k0 + kc;
            *(int4*)((unsigned char*)plane0 + o) = make_int4(hi[0], hi[1], hi[2], hi[3]);
            *(int4*)((unsigned char*)plane1 + o) = make_int4(lo[0], lo[1], lo[2], lo[3]);
        }
        if (rowsum) add_rowsum(rowsum, r0 + r, rows, sum, 4);
    } else {
        // load: 4 rows per thread per k; 16 threads cover 64 rows, 16 k per pass
        for (int i = 0; i < 2; ++i) {
            const int kk = (tid >> 4) + 16 * i, r4 = (tid & 15) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (k0 + kk < k) {
                const float* sp = (const float*)src + (long long)(k0 + kk) * cs + r0 + r4;
                if (r0 + r4 + 4 <= rows) v = __ldg((const float4*)sp);
                else {
                    if (r0 + r4 + 0 < rows) v.x = sp[0];
                    if (r0 + r4 + 1 < rows) v.y = sp[1];
                    if (r0 + r4 + 2 < rows) v.z = sp[2];
                }
            }
            float* dst = (float*)tile + kk * kPitch + r4;
            dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
        }
        __syncthreads();
        const int r = tid >> 2, kc = (tid & 3) * 8;
        float h[8], l[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) tf32_split(((float*)tile)[(kc + j) * kPitch + r], h[j], l[j]);
        if (r0 + r < rows_p && k0 + kc < kp) {
            const long long o = (long long)(r0 + r) * kp + k0 + kc;
            *(float4*)((float*)plane0 + o) = make_float4(h[0], h[1], h[2], h[3]);
            *(float4*)((float*)plane0 + o + 4) = make_float4(h[4], h[5], h[6], h[7]);
            *(float4*)((float*)plane1 + o) = make_float4(l[0], l[1], l[2], l[3]);
            *(float4*)((float*)plane1 + o + 4) = make_float4(l[4], l[5], l[6], l[7]);
        }
    }
}

// no alignment requirement: 32x32 tiles through shared memory so that both the read and the write
// are coalesced whichever of rs / cs is 1.
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
split_planes_kernel(const T* __restrict__ src, long long rs, long long cs, int rows, int k,
                    int rows_p, int kp, void* __restrict__ plane0, void* __restrict__ plane1,
                    unsigned lo_xor, int* __restrict__ rowsum) {
    __shared__ T tile[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;     // 32 x 8
    const int r0 = blockIdx.y * 32, k0 = blockIdx.x * 32;
    const bool k_contig = (cs == 1);
    for (int i = ty; i < 32; i += 8) {
        // read so that the contiguous source direction runs along tx
        const int r = k_contig ? r0 + i : r0 + tx;
        const int kk = k_contig ? k0 + tx : k0 + i;
        T v = 0;
        if (r < rows && kk < k) v = src[(long long)r * rs + (long long)kk * cs];
        if (k_contig) tile[i][tx] = v; else tile[tx][i] = v;
    }
    __syncthreads();
    for (int i = ty; i < 32; i += 8) {
        const int r = r0 + i, kk = k0 + tx;
        const T v = tile[i][tx];
        if (MODE == MODE_FLEX16 && rowsum) add_rowsum(rowsum, r, rows, (int)v, 32);
        if (r >= rows_p || kk >= kp) continue;
        const long long o = (long long)r * kp + kk;
        if (MODE == MODE_FLEX16) {
            const int m = (int)v;
            const int lo = m & 0xff;                 // unsigned low byte
            const int hi = (m - lo) >> 8;            // signed high byte: m = 256*hi + lo
            ((signed char*)plane0)[o] = (signed char)hi;
            ((unsigned char*)plane1)[o] = (unsigned char)(lo ^ lo_xor);
        } else {
            float hi, lo;
            tf32_split((float)v, hi, lo);
            ((float*)plane0)[o] = hi;
            ((float*)plane1)[o] = lo;
        }
    }
}

// Picks the pre-pass kernel for one operand.
template <typename T, int MODE>
int split_operand(const T* src, long long rs, long long cs, int rows, int k, int rows_p, int kp,
                  void* plane0, void* plane1, unsigned lo_xor, int* rowsum, cudaStream_t st) {
    const bool base16 = ((uintptr_t)src & 15) == 0;
    const int vec = 16 / (int)sizeof(T);
    if (cs == 1 && base16 && rs % vec == 0) {
        const long long units = (long long)rows_p * (kp / (MODE == MODE_FLEX16 ? 16 : 4));
        split_rows_kernel<T, MODE><<<(unsigned)((units + 255) / 256), 256, 0, st>>>(
            src, rs, rows, k, rows_p, kp, plane0, plane1, lo_xor, rowsum);
    } else if (rs == 1 && base16 && cs % vec == 0) {
        const int tk = MODE == MODE_FLEX16 ? 64 : 32;
        dim3 g((kp + tk - 1) / tk, (rows_p + 63) / 64);
        split_cols_kernel<T, MODE><<<g, 256, 0, st>>>(src, cs, rows, k, rows_p, kp, plane0, plane1,
                                                     lo_xor, rowsum);
    } else {
        dim3 g((kp + 31) / 32, (rows_p + 31) / 32);
        split_planes_kernel<T, MODE><<<g, 256, 0, st>>>(src, rs, cs, rows, k, rows_p, kp, plane0,
                                                       plane1, lo_xor, rowsum);
    }
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::mutex g_gemm_mutex;

int get_encode() {
    std::lock_guard<std::mutex> lock(g_gemm_mutex);
    if (g_encode) return B2_OK;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    B2_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    if (!fn || qres != cudaDriverEntryPointSuccess)
        return b2::fail(B2_ERR_UNAVAILABLE, "driver lacks cuTensorMapEncodeTiled");
    g_encode = (EncodeTiledFn)fn;
    return B2_OK;
}

// plane: [rows_p][kp] elements of `esize` bytes, K contiguous; box = 128 rows x 128 bytes
int make_map(CUtensorMap* map, void* base, int rows_p, int kp, int esize, int box_rows) {
    cuuint64_t dims[2] = {(cuuint64_t)kp, (cuuint64_t)rows_p};
    cuuint64_t strides[1] = {(cuuint64_t)kp * esize};
    cuuint32_t box[2] = {(cuuint32_t)(kKBytes / esize), (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, esize == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                          2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return b2::fail(B2_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
    return B2_OK;
}

inline int round_up(int v, int m) { return (v + m - 1) / m * m; }
inline size_t align1k(size_t v) { return (v + 1023) & ~(size_t)1023; }

struct Shapes { int Mp, Np, Kp, esize, bn; size_t bytes, a_bytes, rowsum_off; };

inline int pick_bn(int N) { return N <= 16 ? 16 : N <= 32 ? 32 : N <= 64 ? 64 : 128; }

Shapes shapes_for(int mode, int M, int N, int K) {
    Shapes s;
    s.esize = mode == MODE_FLEX16 ? 1 : 4;
    s.bn = pick_bn(N);
    s.Mp = round_up(M, kBlockM);
    s.Np = round_up(N, s.bn);
    s.Kp = round_up(K, kKBytes / s.esize);
    s.a_bytes = 2ull * (size_t)s.Mp * s.Kp * s.esize;
    s.bytes = s.a_bytes + 2ull * (size_t)s.Np * s.Kp * s.esize;
    s.rowsum_off = s.bytes;                  // int32 row sums of A (flex16 merged form)
    if (mode == MODE_FLEX16) s.bytes += (size_t)s.Mp * sizeof(int);
    return s;
}

#ifdef B2_GEMM_OWNS_TILE_KERNEL
template <int MODE, int BN>
int launch_tile(const CUtensorMap& mA0, const CUtensorMap& mA1, const CUtensorMap& mB0,
                const CUtensorMap& mB1, const GemmParams& p, const Shapes& s, int splits,
                cudaStream_t st) {
    static bool attr_set = false;
    if (!attr_set) {
        B2_CUDA(cudaFuncSetAttribute(gemm_kernel<MODE, BN>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(BN)));
        attr_set = true;
    }
    dim3 grid(s.Np / BN, s.Mp / kBlockM, splits);
    gemm_kernel<MODE, BN><<<grid, kThreads, smem_bytes(BN), st>>>(mA0, mA1, mB0, mB1, p);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

#endif

// bytes of split-K workspace for `splits` slices (0 when the GEMM runs in one slice)
inline size_t splitk_bytes(int mode, const Shapes& s, int splits) {
    return splits > 1 ? (size_t)splits * s.Mp * s.Np * (mode == MODE_FLEX16 ? 8 : 4) : 0;
}

// Number of K slices: at least enough that a flex16 slice keeps exact int32 sums (256 k-blocks =
// 32768 elements), and, when `fill` is set, enough to give every SM a tile.
inline int pick_splits(int mode, const Shapes& s, bool fill) {
    const int num_kb = s.Kp / (kKBytes / s.esize);
    int splits = 1;
    if (mode == MODE_FLEX16) splits = (num_kb + 255) / 256;
    if (fill) {
        const int tiles = (s.Mp / kBlockM) * (s.Np / s.bn);
        int want = (2 * 148 + tiles - 1) / tiles;
        const int max_by_k = num_kb / 4 > 0 ? num_kb / 4 : 1;      // at least 4 k-blocks a slice
        if (want > max_by_k) want = max_by_k;
        if (want > splits) splits = want;
    }
    return splits;
}

// scratch of the dense GEMM entry points: operand planes (+ row sums), then the split-K slices
inline size_t gemm_scratch_need(int mode, const Shapes& s) {
    return align1k(s.bytes) + splitk_bytes(mode, s, pick_splits(mode, s, false));
}

// Launches the tile kernel on operand planes that are already in scratch:
// A planes at `base`, B planes behind them.  With splits > 1, `workspace` (splitk_bytes) receives
// the slices and a finishing kernel writes C.
#ifdef B2_GEMM_OWNS_TILE_KERNEL
template <int MODE>
int launch_on_planes(unsigned char* base, const Shapes& s, GemmParams p, cudaStream_t st,
                     int splits = 1, void* workspace = nullptr) {
    int rc = get_encode();
    if (rc) return rc;
    const size_t a_plane = (size_t)s.Mp * s.Kp * s.esize, b_plane = (size_t)s.Np * s.Kp * s.esize;
    void* A0 = base; void* A1 = base + a_plane;
    void* B0 = base + 2 * a_plane; void* B1 = base + 2 * a_plane + b_plane;
    CUtensorMap mA0, mA1, mB0, mB1;
    if ((rc = make_map(&mA0, A0, s.Mp, s.Kp, s.esize, 128))) return rc;
    if ((rc = make_map(&mA1, A1, s.Mp, s.Kp, s.esize, 128))) return rc;
    if ((rc = make_map(&mB0, B0, s.Np, s.Kp, s.esize, s.bn))) return rc;
    if ((rc = make_map(&mB1, B1, s.Np, s.Kp, s.esize, s.bn))) return rc;
    p.num_kb = s.Kp / (kKBytes / s.esize);
    p.Mp = s.Mp; p.Np = s.Np;
    p.partial = nullptr; p.kb_per_split = p.num_kb;
    if (splits > 1) {
        B2_REQUIRE(workspace, "split-K needs a workspace");
        p.partial = workspace;
        p.kb_per_split = (p.num_kb + splits - 1) / splits;
        splits = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;      // no empty slice
    }
    switch (s.bn) {
        case 16: rc = launch_tile<MODE, 16>(mA0, mA1, mB0, mB1, p, s, splits, st); break;
        case 32: rc = launch_tile<MODE, 32>(mA0, mA1, mB0, mB1, p, s, splits, st); break;
        case 64: rc = launch_tile<MODE, 64>(mA0, mA1, mB0, mB1, p, s, splits, st); break;
        default: rc = launch_tile<MODE, 128>(mA0, mA1, mB0, mB1, p, s, splits, st); break;
    }
    if (rc || !p.partial) return rc;
    long long blocks = ((long long)p.M * p.N + 31) / 32;
    if (blocks > 148 * 16) blocks = 148 * 16;
    splitk_finish_kernel<MODE><<<(unsigned)blocks, 256, 0, st>>>(p, splits);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}
#else
template <int MODE>
int launch_on_planes(unsigned char* base, const Shapes& s, GemmParams p, cudaStream_t st,
                     int splits = 1, void* workspace = nullptr) {
    return b2_gemm_launch_on_planes(MODE, base, &s, &p, st, splits, workspace);
}
#endif

// A flex16 product far smaller than one wave of tensor-core tiles (the 10 x 64 x 256 classifier
// of a small network): one thread per result, exact int64 sum, the tile kernel's rescale -- one
// launch instead of the operand pre-passes and a mostly empty 128-row tile.
__global__ void __launch_bounds__(256)
small_gemm_flex16_kernel(const short* __restrict__ A, long long a_rs, long long a_cs,
                         const short* __restrict__ B, long long b_ks, long long b_ns,
                         short* __restrict__ C, long long ldc, int M, int N, int K,
                         const b2_flex_scale* __restrict__ table, int slotA, int slotB, int slotC,
                         int* stats, unsigned long long* probe_out, int probe) {
    const float f = table[slotA].scale * table[slotB].scale * (probe ? 1.0f : table[slotC].inv_scale);
    const int sh = -ilogbf(f);
    int stat = 0;
    unsigned long long pmax = 0;
    const long long total = (long long)M * N;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int m = (int)(i / N), n = (int)(i - (long long)m * N);
        const short* a = A + m * a_rs;
        const short* b = B + n * b_ns;
        long long acc = 0;
#pragma unroll 4
        for (int k = 0; k < K; ++k) acc += (long long)((int)a[k * a_cs] * (int)b[k * b_ks]);
        if (probe) {
            const unsigned long long v = (unsigned long long)(acc < 0 ? -acc : acc);
            pmax = v > pmax ? v : pmax;
        } else {
            const int q = rescale_i64(acc, sh);
            const int v = q < 0 ? -q : q;
            stat = v > stat ? v : stat;
            C[m * ldc + n] = (short)q;
        }
    }
    if (probe) {
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long t = __shfl_xor_sync(0xffffffffu, pmax, o);
            pmax = t > pmax ? t : pmax;
        }
        if ((threadIdx.x & 31) == 0 && pmax) atomicMax(probe_out, pmax);
    } else {
        for (int o = 16; o > 0; o >>= 1) {
            const int t = __shfl_xor_sync(0xffffffffu, stat, o);
            stat = t > stat ? t : stat;
        }
        if ((threadIdx.x & 31) == 0 && stat) atomicMax(stats + slotC, stat);
    }
}

inline bool small_gemm(int mode, int M, int N, int K) {
    return mode == MODE_FLEX16 && (long long)M * N <= 8192 && K <= 1024;
}

template <typename T, int MODE>
int run_gemm(const T* A, long long a_rs, long long a_cs, const T* B, long long b_ks, long long b_ns,
             void* C, long long ldc, int M, int N, int K, const b2_flex_scale* table, int slotA,
             int slotB, int slotC, int* stats, void* scratch, size_t scratch_bytes,
             unsigned long long* probe_out, int* status, int probe, cudaStream_t st) {
    B2_REQUIRE(A && B && C && M > 0 && N > 0 && K > 0, "bad GEMM argument");
    B2_REQUIRE(a_rs == 1 || a_cs == 1, "A must be contiguous along M or K");
    B2_REQUIRE(b_ks == 1 || b_ns == 1, "B must be contiguous along K or N");
    if (small_gemm(MODE, M, N, K)) {
        const int blocks = (int)(((long long)M * N + 255) / 256);
        small_gemm_flex16_kernel<<<blocks, 256, 0, st>>>(
            (const short*)A, a_rs, a_cs, (const short*)B, b_ks, b_ns, (short*)C, ldc, M, N, K, table,
            slotA, slotB, slotC, stats, probe_out, probe);
        B2_CUDA(cudaGetLastError());
        return B2_OK;
    }
    const Shapes s = shapes_for(MODE, M, N, K);
    const int splits = pick_splits(MODE, s, false);     // > 1 only for flex16 with K > 32768
    const size_t need = gemm_scratch_need(MODE, s);
    B2_REQUIRE(scratch && scratch_bytes >= need && ((uintptr_t)scratch & 1023) == 0,
               "GEMM needs %zu bytes of 1024-byte aligned scratch, got %zu", need, scratch_bytes);
    unsigned char* base = (unsigned char*)scratch;
    const size_t a_plane = (size_t)s.Mp * s.Kp * s.esize, b_plane = (size_t)s.Np * s.Kp * s.esize;
    void* A0 = base; void* A1 = base + a_plane;
    void* B0 = base + 2 * a_plane; void* B1 = base + 2 * a_plane + b_plane;
    int* rowsum = nullptr;
    unsigned lo_xor = 0;
    if (MODE == MODE_FLEX16) {
        rowsum = (int*)(base + s.rowsum_off);
        lo_xor = 0x80;
        B2_CUDA(cudaMemsetAsync(rowsum, 0, (size_t)s.Mp * sizeof(int), st));
    }
    int rc = split_operand<T, MODE>(A, a_rs, a_cs, M, K, s.Mp, s.Kp, A0, A1, 0, rowsum, st);
    if (rc) return rc;
    // op(B)^T: rows = N, element (n, k) = B[k * b_ks + n * b_ns]
    rc = split_operand<T, MODE>(B, b_ns, b_ks, N, K, s.Np, s.Kp, B0, B1, lo_xor, nullptr, st);
    if (rc) return rc;
    GemmParams p;
    p.M = M; p.N = N; p.num_kb = 0;
    p.ldc = ldc; p.C = C; p.table = table; p.slotA = slotA; p.slotB = slotB; p.slotC = slotC;
    p.stats = stats; p.probe_out = probe_out; p.status = status; p.probe = probe;
    p.c_colmajor = 0;
    p.rowsum = rowsum;
    return launch_on_planes<MODE>(base, s, p, st, splits, base + align1k(s.bytes));
}

}  // namespace

#endif  // B2_GEMM_IMPL_CUH
