// Convolution forward (and average pooling) for tensors in the reference's C,D,H,W,N layout.
//
// Takes the place of ConvFpropKernel / FlexConvFpropKernel and the direct-convolution SASS they
// select (ngraph/transformers/gpu/conv.py:24-100, gpu/flex_conv.py:49-200,
// gpu/kernels/sass/?conv_xprop_*.sass), and of the avg-pooling forward kernel
// (gpu/pool.py:27-220, gpu/kernels/cuda/pooling.py:291-438).
//
// fprop:  O[K,M,P,Q,N] = sum_{c,t,r,s} F[C,T,R,S,K] * I[C,D,H,W,N]
// is run as one GEMM on the tensor cores, O^T[(p,q,n), k] = Icol[(p,q,n),(c,r,s)] * F[(c,r,s), k]:
//   * a gather pre-pass writes the rows of Icol (one row per output pixel and image, the filter
//     window unrolled along K, zero where the window hangs over the border) directly as the two
//     operand planes the GEMM kernel streams with TMA (int8 hi/lo for flex16, tf32 hi/lo for
//     fp32), so the input is read once and no separate split pass is needed;
//   * the filter planes come from the same split kernel the GEMM uses (F is already [(c,r,s)][k]);
//   * the tile kernel's epilogue stores column-major, which is exactly the K,P,Q,N layout: for a
//     fixed output channel the 32 lanes of a warp hold 32 consecutive images -> coalesced stores.
// N (batch) is the GEMM-M direction (128 rows per tile), the output channels are the GEMM-N
// direction with a 16/32/64/128-wide tile, so the small channel counts of ResNet-20 do not pad
// the tensor-core tile to 128.
//
// The two training contractions (ConvBpropKernel / ConvUpdateKernel, gpu/conv.py:121-312,
// FlexConvBpropKernel / FlexConvUpdateKernel, gpu/flex_conv.py:203-621; readable specification
// ngraph/transformers/cpu/cpuengine.py:256-271 and :395-418) run on the same tile kernel:
//   bprop:  gI^T[(h,w,n), c] = Ecol[(h,w,n),(k,r,s)] * F[(c,r,s),k] read as [(k,r,s)][c], where the
//           gather takes E[k,p,q,n] with p = (h + pad - r*dil) / str when that division is exact
//           and p lies inside the output, zero otherwise (the transposed, flipped convolution);
//   update: U[(c,r,s), k] = Icol^T[(c,r,s),(p,q,n)] * E[k,(p,q,n)]: the contraction runs over all
//           output positions and images (262144 for a 32x32 layer at batch 256), so it is cut
//           into K slices spread over the SMs; the slices are added in a fixed order by a second
//           kernel (deterministic, and exact for flex16: every slice is an exact integer).
#include <cstdlib>

#include "b2_gemm_impl.cuh"

namespace {

struct ConvGeom {
    int C, H, W, N, K, R, S, P, Q, pad_h, pad_w, str_h, str_w, dil_h, dil_w;
    // depth (the reference's D / T / M axes): handled by the gather + GEMM path only; the tile
    // kernels take convolutions with D = T = M = 1
    int D, T, M, pad_d, str_d, dil_d;
    // the streamed tensor of an implicit-GEMM pass may be a zero-dilated view of a smaller one
    // (the input gradient of a strided convolution): element (h, w) is source (h/up_h, w/up_w)
    // where both divide and the quotient is inside src_h x src_w, zero elsewhere
    int up_h, up_w, src_h, src_w;
};

int geom_from(const b2_conv_dims* d, ConvGeom* g) {
    B2_REQUIRE(d, "null dims");
    B2_REQUIRE(d->C > 0 && d->H > 0 && d->W > 0 && d->N > 0 && d->K > 0 && d->R > 0 && d->S > 0 &&
               d->P > 0 && d->Q > 0 && d->str_h > 0 && d->str_w > 0 && d->dil_h > 0 && d->dil_w > 0 &&
               d->D > 0 && d->T > 0 && d->M > 0 && d->str_d > 0 && d->dil_d > 0 && d->pad_d >= 0 &&
               d->pad_h >= 0 && d->pad_w >= 0,
               "bad convolution dimensions");
    B2_REQUIRE((long long)d->D * d->H * d->W < (1 << 24) && (long long)d->M * d->P * d->Q < (1 << 24),
               "convolution extents too large");
    g->C = d->C; g->H = d->H; g->W = d->W; g->N = d->N; g->K = d->K; g->R = d->R; g->S = d->S;
    g->P = d->P; g->Q = d->Q; g->pad_h = d->pad_h; g->pad_w = d->pad_w; g->str_h = d->str_h;
    g->str_w = d->str_w; g->dil_h = d->dil_h; g->dil_w = d->dil_w;
    g->up_h = g->up_w = 1; g->src_h = g->H; g->src_w = g->W;
    g->D = d->D; g->T = d->T; g->M = d->M; g->pad_d = d->pad_d; g->str_d = d->str_d;
    g->dil_d = d->dil_d;
    return B2_OK;
}

inline bool flat_depth(const ConvGeom& g) {
    return g.D == 1 && g.T == 1 && g.M == 1 && g.pad_d == 0;
}

// Gather + split.  Rows of the planes: r = ((m*P + p)*Q + q)*N + n ; columns:
// kidx = ((c*T + t)*R + r_)*S + s_.
// A block owns 32 consecutive rows (32 images of one output pixel when N is a multiple of 32) and
// walks the columns in chunks of 128 bytes of plane row.  Per chunk the tap decomposition of each
// column is computed once into shared memory; loads run along n (contiguous in the input), the
// write phase emits one 16-byte vector per thread and plane (contiguous along the plane row).
// BPROP = true gathers the rows of Ecol instead: row = (h*W + w)*N + n of the INPUT gradient,
// column = (k*R + r_)*S + s_, source E[k, p, q, n] (see the head of this file).
template <typename T, int MODE, bool BPROP>
__global__ void __launch_bounds__(256)
im2col_planes_kernel(const T* __restrict__ I, ConvGeom g, int rows, int kg, int rows_p, int kp,
                     void* __restrict__ plane0, void* __restrict__ plane1) {
    constexpr int CK = MODE == MODE_FLEX16 ? 128 : 32;
    __shared__ T tile[CK][33];
    __shared__ int tab_c[CK], tab_h[CK], tab_w[CK], tab_d[CK];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int r0 = blockIdx.x * 32;
    const int r = r0 + tx;
    const bool rvalid = r < rows;
    int n = 0, h0 = 0, w0 = 0, d0 = 0;
    if (rvalid) {
        n = r % g.N;
        const int pq = r / g.N;
        if (BPROP) {
            const int hw = pq % (g.H * g.W);
            d0 = pq / (g.H * g.W) + g.pad_d;
            h0 = hw / g.W + g.pad_h;
            w0 = hw % g.W + g.pad_w;
        } else {
            const int q = pq % g.Q, mp = pq / g.Q, pp = mp % g.P;
            d0 = (mp / g.P) * g.str_d - g.pad_d;
            h0 = pp * g.str_h - g.pad_h;
            w0 = q * g.str_w - g.pad_w;
        }
    }
    const int RS = g.R * g.S, TRS = g.T * RS;
    const int wr = threadIdx.x >> 3, vec = threadIdx.x & 7;
    const int orow = r0 + wr;
    for (int kc = 0; kc < kp; kc += CK) {
        __syncthreads();
        if (threadIdx.x < CK) {
            const int kidx = kc + threadIdx.x;
            if (kidx < kg) {
                const int c = kidx / TRS, trs = kidx - c * TRS;
                const int ft = trs / RS, rs = trs - ft * RS;
                const int fr = rs / g.S, fs = rs - fr * g.S;
                tab_c[threadIdx.x] = c * (BPROP ? g.M * g.P * g.Q : g.D * g.H * g.W) * g.N;
                tab_d[threadIdx.x] = ft * g.dil_d;
                tab_h[threadIdx.x] = fr * g.dil_h;
                tab_w[threadIdx.x] = fs * g.dil_w;
            } else {
                tab_c[threadIdx.x] = -1;
            }
        }
        __syncthreads();
        for (int i = ty; i < CK; i += 8) {
            T v = 0;
            const int tc = tab_c[i];
            if (tc >= 0 && rvalid) {
                if (BPROP) {
                    const int th = h0 - tab_h[i], tw = w0 - tab_w[i], td = d0 - tab_d[i];
                    if (th >= 0 && tw >= 0 && td >= 0 && th % g.str_h == 0 && tw % g.str_w == 0 &&
                        td % g.str_d == 0) {
                        const int pp = th / g.str_h, q = tw / g.str_w, mm = td / g.str_d;
                        if (pp < g.P && q < g.Q && mm < g.M)
                            v = I[(long long)tc + (((long long)mm * g.P + pp) * g.Q + q) * g.N + n];
                    }
                } else {
                    const int h = h0 + tab_h[i], w = w0 + tab_w[i], dd = d0 + tab_d[i];
                    if (h >= 0 && h < g.H && w >= 0 && w < g.W && dd >= 0 && dd < g.D)
                        v = I[(long long)tc + (((long long)dd * g.H + h) * g.W + w) * g.N + n];
                }
            }
            tile[i][tx] = v;
        }
        __syncthreads();
        if (orow < rows_p) {
            if (MODE == MODE_FLEX16) {
                unsigned hi[4] = {0, 0, 0, 0}, lo[4] = {0, 0, 0, 0};
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int m = (int)tile[vec * 16 + j][wr];
                    const int l = m & 0xff;
                    const int h8 = ((m - l) >> 8) & 0xff;
                    hi[j >> 2] |= (unsigned)h8 << (8 * (j & 3));
                    lo[j >> 2] |= (unsigned)l << (8 * (j & 3));
                }
                const long long o = (long long)orow * kp + kc + vec * 16;
                *reinterpret_cast<uint4*>((unsigned char*)plane0 + o) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<uint4*>((unsigned char*)plane1 + o) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            } else {
                float hi[4], lo[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float a = (float)tile[vec * 4 + j][wr];
                    unsigned hb;
                    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hb) : "f"(a));
                    hi[j] = __uint_as_float(hb);
                    lo[j] = a - hi[j];
                }
                const long long o = (long long)orow * kp + kc + vec * 4;
                *reinterpret_cast<float4*>((float*)plane0 + o) = make_float4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<float4*>((float*)plane1 + o) = make_float4(lo[0], lo[1], lo[2], lo[3]);
            }
        }
    }
}

// ================================================================================================
// Implicit GEMM (flex16): no unrolled copy of the input.
//
// For batches that are a multiple of 128 the tile kernel reads the activations straight from
// their C,H,W,N layout.  A tile is one output pixel (p,q) x 128 images; its reduction runs over
// chunks of `cu` input channels.  For every chunk ONE 4-d TMA box [cu channels][R][S][128 images]
// per operand plane is fetched at (n0, q*str - pad, p*str - pad, c0): the whole filter window of
// those channels in a single copy, zero fill outside the image doing the padding.  It lands in
// shared memory as an MN-major (images contiguous) 128-byte-swizzled operand whose K rows are in
// (channel, r, s) order -- the natural order of the C,R,S,K filter tensor -- padded to a multiple
// of 32 rows (one MMA step).
//
// At 16..64 output channels an MMA's time is the read of its A operand from shared memory (4 KB
// per instruction whatever N is), so the four byte products are folded into TWO instructions per
// k-step.  The filters' low plane is stored as the signed byte bl - 128, which makes both filter
// planes signed and lets them lie behind one another as one operand of 2*bn rows:
//     A_hi x [B_hi | B_lo'] -> HH | X            A_lo x [B_hi | B_lo'] -> X | LL
// The bias costs 128 * (sum of the activations under the window); that sum comes out of the same
// instructions through one extra filter column whose planes are (0, +1) on every K row: its X and
// LL accumulators are sum(a_hi) and sum(a_lo).  Because that column is 1 on the padding rows too,
// whatever bytes lie there cancel exactly (their true filter value is 0 = 256*0 + (-128) + 128).
//
// The filter planes of the CTA's output channels are loaded ONCE per CTA and stay resident in
// shared memory.  CTAs are persistent: each walks many tiles, the producer warp runs ahead across
// tile boundaries through a ring of stages, and up to four accumulator sets in tensor memory let
// the epilogues of earlier tiles (sixteen warps) overlap the MMAs of later ones.
// The only pre-pass is an elementwise split of the activations into the two operand planes, and a
// fused elementwise kernel that produces the activations can write the planes itself.
// ================================================================================================
struct ConvTileParams {
    int P, Q, N, K;
    int pad_h, pad_w, str_h, str_w;
    int cu;                       // channels per chunk
    int cchunks;                  // chunks per tile = stages per tile
    int kc_pad;                   // K rows per chunk, padded to a multiple of 32
    int box_bytes;                // bytes one activation box delivers (cu*R*S*128)
    int npanels;                  // 128-byte K panels of the resident filter planes
    int nstages;                  // ring depth
    int bn;                       // columns per accumulator: kt output channels + the sum column
    int kt;                       // output channels per CTA column (blockIdx.y)
    int nbuf;                     // accumulator sets in tensor memory: 1, 2, 3 (or 4)
    int n_mma;                    // MMA-issuing threads: 1..3, at most nbuf
    int tmem_cols;                // power of two >= 3*bn*nbuf
    int num_tiles, nblk;
    long long ldc;
    void* O;
    const b2_flex_scale* table;
    int slotA, slotB, slotC;
    int* stats;
    unsigned long long* probe_out;
    int* status;
    int probe;
    long long* dbg;      // optional per-role cycle counters of CTA 0 (profiling aid), else null
    // fused epilogue (all optional): y = relu?(conv + bias[k] + residual) in fp32, quantised once
    // with the output's exponent; stored as int16 and / or as the byte planes the next
    // convolution reads
    int fused;                    // 0: plain integer rescale of the convolution
    const short* bias; int slot_bias;
    const short* residual; int slot_res;      // same K,P,Q,N layout as the output
    int relu;
    int write_i16;
    unsigned char* out_planes; long long out_plane_bytes;
};

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, int c0, int c1,
                                            int c2, int c3, unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3, %4, %5}], [%6];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_u32(bar))
        : "memory");
}
// one 32-bit column of this thread's TMEM lane
__device__ __forceinline__ unsigned tmem_ld1(unsigned taddr) {
    unsigned r;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr) : "memory");
    return r;
}
// 8 consecutive 32-bit columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld8(unsigned taddr, unsigned* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void prefetch_map(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
}
// instruction descriptor with a run-time N
__device__ __forceinline__ unsigned make_idesc_n(unsigned dfmt, unsigned afmt, unsigned bfmt,
                                                 unsigned n) {
    return (dfmt << 4) | (afmt << 7) | (bfmt << 10) | ((n >> 3) << 17) |
           ((unsigned)(kBlockM >> 4) << 24);
}

constexpr int kConvMaxStages = 8;
constexpr int kConvThreads = 640;           // producer, MMA, sixteen epilogue warps, two more MMA warps
constexpr int kConvSmemMax = 232448;        // 227 KB: the most one CTA can have
constexpr int kConvSmemFixed = 1024 /*alignment*/ + 1024 /*barriers, bias*/;

__global__ void __launch_bounds__(kConvThreads, 1)
conv_implicit_kernel(const __grid_constant__ CUtensorMap mapI0,
                     const __grid_constant__ CUtensorMap mapI1,
                     const __grid_constant__ CUtensorMap mapB, const ConvTileParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int bn = p.bn;
    const int panel_bytes = 2 * bn * kKBytes;                  // [B_hi rows | B_lo' rows] x 128 B
    const int acc_cols = 3 * bn;                               // HH | X | LL
    const int act_stage = p.kc_pad * 128;                      // bytes per plane per stage
    unsigned char* filt = smem;                                // [npanels][2*bn][128]
    unsigned char* ring = smem + p.npanels * panel_bytes;      // [nstages][2 planes][act_stage]
    // one set of "stage filled" barriers per MMA-issuing warp: a waiter must see every phase of
    // a barrier in turn (a parity wait cannot tell phase n from phase n+2), and an issuer only
    // ever looks at the stages of its own tiles
    unsigned long long* full_bar =
        (unsigned long long*)(ring + (size_t)p.nstages * 2 * act_stage);   // [4][kConvMaxStages]
    unsigned long long* empty_bar = full_bar + 4 * kConvMaxStages;
    unsigned long long* tmem_full = empty_bar + kConvMaxStages;   // [4]
    // "set drained" barriers, one per (issuing thread, set): the epilogue signals the thread that
    // will fill the set next, so each thread meets every phase of its own barriers in turn
    unsigned long long* tmem_empty = tmem_full + 4;               // [4 issuers][4 sets]
    unsigned long long* filt_bar = tmem_empty + 16;
    unsigned* tmem_holder = (unsigned*)(filt_bar + 1);
    int* fail_flag = (int*)(tmem_holder + 1);
    float* bias_s = (float*)(fail_flag + 2);                      // [bn] bias of this CTA's channels, real values

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int epi_w = p.nbuf == 3 ? 1 : 4 / p.nbuf;   // epilogue warps per lane quarter and accumulator set

    // Programmatic dependent launch: the next kernel of the stream, if it was launched the same
    // way, may take the SMs this grid leaves while its last CTAs still work, and do its set-up;
    // it reads and writes global memory only after its own griddepcontrol.wait below.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x == 0) {
        prefetch_map(&mapI0); prefetch_map(&mapI1); prefetch_map(&mapB);
        for (int s = 0; s < kConvMaxStages; ++s) {
            for (int i = 0; i < 4; ++i) mbar_init(&full_bar[i * kConvMaxStages + s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 4; ++b) {
            mbar_init(&tmem_full[b], 1);
            for (int i = 0; i < 4; ++i) mbar_init(&tmem_empty[i * 4 + b], 4 * epi_w);
        }
        mbar_init(filt_bar, 1);
        *fail_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_holder, p.tmem_cols);
    // everything before this line touches no global memory; everything after it sees the
    // completed work of all earlier kernels of the stream
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x >= 64 && threadIdx.x < 64 + bn) {
        const int col = blockIdx.y * p.kt + (threadIdx.x - 64);
        bias_s[threadIdx.x - 64] = (p.fused && p.bias && (threadIdx.x - 64) < p.kt && col < p.K)
                                       ? (float)p.bias[col] * p.table[p.slot_bias].scale *
                                             (p.probe ? 1.0f : p.table[p.slotC].inv_scale)
                                       : 0.0f;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_holder;

    if (warp == 0) {
        if (lane == 0) {
            // the filter planes of this CTA's output channels: once, resident
            mbar_expect_tx(filt_bar, p.npanels * panel_bytes);
            for (int j = 0; j < p.npanels; ++j)
                tma_load_2d(filt + j * panel_bytes, &mapB, j * kKBytes, blockIdx.y * 2 * bn, filt_bar);
            int s = 0, ti = 0;
            const int n_mma = p.n_mma;
            unsigned empty_parity = 1;         // the first pass over the ring finds every stage free
            bool ok = true;
            const long long t_start = clock64();
            long long t_wait = 0;
            for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++ti) {
                unsigned long long* fb = full_bar + (ti % n_mma) * kConvMaxStages;   // its consumer's
                const int pq = tile / p.nblk, nb = tile - pq * p.nblk;
                const int pp = pq / p.Q, q = pq - pp * p.Q;
                const int n0 = nb * 128;
                const int h0 = pp * p.str_h - p.pad_h, w0 = q * p.str_w - p.pad_w;
                for (int cc = 0; cc < p.cchunks; ++cc) {
                    const long long tw = clock64();
                    if (!mbar_wait_relaxed(&empty_bar[s], empty_parity)) {
                        atomicExch(fail_flag, 1); ok = false; break;
                    }
                    t_wait += clock64() - tw;
                    unsigned char* sa = ring + (size_t)s * 2 * act_stage;
                    mbar_expect_tx(&fb[s], 2 * p.box_bytes);
                    tma_load_4d(sa, &mapI0, n0, w0, h0, cc * p.cu, &fb[s]);
                    tma_load_4d(sa + act_stage, &mapI1, n0, w0, h0, cc * p.cu, &fb[s]);
                    if (++s == p.nstages) { s = 0; empty_parity ^= 1u; }
                }
            }
            if (p.dbg && blockIdx.x == 0 && blockIdx.y == 0) {
                p.dbg[0] = clock64() - t_start; p.dbg[1] = t_wait;
            }
        }
    } else if (warp == 1 || warp >= 18) {
        // up to three MMA-issuing threads take the tiles in turn (when there are accumulator sets
        // for them): an MMA instruction costs its issuing thread about a hundred cycles whatever
        // its N and whatever the operand layout (a K-major, channel-innermost variant of this
        // kernel was measured slower), and at 16..64 output channels that latency is what bounds
        // a tile.  Three keep up with the operand fetch; a fourth would need a 21st warp, and at
        // 672 threads the register file leaves the epilogue 80 registers (it spills and the
        // kernel is slower than with two).
        const int mma_id = warp == 1 ? 0 : warp - 17;
        const int n_mma = p.n_mma;
        if (lane == 0) {
            // bit 15: A is MN-major.  A_hi is signed, A_lo unsigned, both filter planes signed.
            const unsigned mn = 1u << 15;
            const unsigned id_s2 = make_idesc_n(2, 1, 1, 2 * bn) | mn, id_u2 = make_idesc_n(2, 0, 1, 2 * bn) | mn;
            const unsigned id_s1 = make_idesc_n(2, 1, 1, bn) | mn, id_u1 = make_idesc_n(2, 0, 1, bn) | mn;
            int ti = 0;
            bool ok = mma_id < n_mma && mbar_wait(filt_bar, 0);
            if (!ok && mma_id < n_mma) atomicExch(fail_flag, 1);
            const int ksteps = p.kc_pad >> 5;
            // Matrix descriptors as (low word, constant high word): only the start address
            // (bits 0-13, in 16-byte units) changes from one MMA to the next, so the loop keeps
            // a few running integers instead of rebuilding 64-bit descriptors.
            const unsigned long long desc_hi = (unsigned long long)((1024u >> 4) | (1u << 14) | (2u << 29)) << 32;
            const unsigned filt_lo = ((smem_u32(filt) >> 4) & 0x3FFF) | (1u << 16);     // K-major: LBO field 1
            const unsigned lo_rows = (unsigned)((bn * kKBytes) >> 4);                   // B_lo' behind B_hi
            const unsigned panel_units = (unsigned)(panel_bytes >> 4);
            const unsigned ring_lo = (smem_u32(ring) >> 4) & 0x3FFF;                  // MN-major: LBO field 0
            const unsigned stage_units = (unsigned)((2 * act_stage) >> 4), plane_units = (unsigned)(act_stage >> 4);
            int s = 0;
            unsigned phase_bits = 0, stage_lo = ring_lo;       // bit s: parity of my next phase of stage s
            unsigned empty_bits = 0;                           // bit b: the same for set b's "drained" barrier
            unsigned long long* fb = full_bar + mma_id * kConvMaxStages;
            const long long t_start = clock64();
            long long t_wait_e = 0, t_wait_f = 0, t_mma = 0, t_commit = 0;
            for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++ti) {
                if (ti % n_mma != mma_id) {
                    // the other issuing thread's tile: step over its stages (their "filled"
                    // barriers are the other thread's own)
                    for (int cc = 0; cc < p.cchunks; ++cc) {
                        stage_lo += stage_units;
                        if (++s == p.nstages) { s = 0; stage_lo = ring_lo; }
                    }
                    continue;
                }
                const int buf = ti % p.nbuf;
                const unsigned acc_base = tmem_base + buf * acc_cols;
                const long long tw = clock64();
                if (ti >= p.nbuf) {
                    if (!mbar_wait(&tmem_empty[mma_id * 4 + buf], (empty_bits >> buf) & 1u)) {
                        atomicExch(fail_flag, 1); ok = false; break;
                    }
                    empty_bits ^= 1u << buf;
                }
                t_wait_e += clock64() - tw;
                tc_fence_after();
                int idx = 0;                                   // 32-byte column block of the filter planes
                for (int cc = 0; cc < p.cchunks; ++cc) {
                    const long long tw2 = clock64();
                    if (!mbar_wait(&fb[s], (phase_bits >> s) & 1u)) {
                        atomicExch(fail_flag, 1); ok = false; break;
                    }
                    phase_bits ^= 1u << s;
                    t_wait_f += clock64() - tw2;
                    tc_fence_after();
                    unsigned a_lo = stage_lo;
                    const long long tm0 = clock64();
                    for (int k = 0; k < ksteps; ++k, ++idx, a_lo += 256u) {
                        const unsigned boff = (unsigned)(idx >> 2) * panel_units + (unsigned)(idx & 3) * 2u;
                        const unsigned long long dB = desc_hi | (filt_lo + boff);
                        const unsigned long long dA0 = desc_hi | a_lo;
                        const unsigned long long dA1 = desc_hi | (a_lo + plane_units);
                        if (idx > 0) {
                            tc_mma<MODE_FLEX16>(acc_base, dA0, dB, id_s2, 1u);            // HH | X
                            tc_mma<MODE_FLEX16>(acc_base + bn, dA1, dB, id_u2, 1u);       // X | LL
                        } else {
                            // first k-step of a tile: the accumulators start from different products
                            const unsigned long long dBl = desc_hi | (filt_lo + boff + lo_rows);
                            tc_mma<MODE_FLEX16>(acc_base, dA0, dB, id_s1, 0u);
                            tc_mma<MODE_FLEX16>(acc_base + bn, dA0, dBl, id_s1, 0u);
                            tc_mma<MODE_FLEX16>(acc_base + bn, dA1, dB, id_u1, 1u);
                            tc_mma<MODE_FLEX16>(acc_base + 2 * bn, dA1, dBl, id_u1, 0u);
                        }
                    }
                    const long long tm1 = clock64();
                    tc_commit(&empty_bar[s]);
                    stage_lo += stage_units;
                    if (++s == p.nstages) { s = 0; stage_lo = ring_lo; }
                    t_mma += tm1 - tm0; t_commit += clock64() - tm1;
                }
                const long long tc0 = clock64();
                tc_commit(&tmem_full[buf]);
                t_commit += clock64() - tc0;
            }
            if (p.dbg && blockIdx.x == 0 && blockIdx.y == 0 && mma_id == 0) {
                p.dbg[2] = clock64() - t_start; p.dbg[3] = t_wait_e; p.dbg[4] = t_wait_f;
                p.dbg[8] = t_mma; p.dbg[9] = t_commit;
            }
        }
    } else {
        // epilogue warps 2..17: TMEM lane quarter = warp % 4.  Accumulator set b is drained by the
        // warps whose slot (0..3) falls into [b*epi_w, (b+1)*epi_w); they take the 16-column
        // chunks of its output channels in turn.
        const int quarter = warp & 3;
        const int slot = (warp - 2) >> 2;
        const int set = slot / epi_w, part = slot % epi_w;
        const int ncol0 = blockIdx.y * p.kt;                  // first output channel of this CTA
        int kt = p.K - ncol0;                                  // output channels this CTA owns
        if (kt > p.kt) kt = p.kt;
        int stat = 0;
        unsigned long long pmax = 0;
        const int n_mma_e = p.n_mma;
        const int n_my = (p.num_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
        const float f = p.table[p.slotA].scale * p.table[p.slotB].scale *
                        (p.probe ? 1.0f : p.table[p.slotC].inv_scale);
        const int sh = -ilogbf(f);
        // fused epilogue: every term carries the output's 1/step (a power of two, so the scaled
        // sum is the real-valued sum times that power, bit for bit); the probe keeps real values
        const float q_out = p.probe ? 1.0f : p.table[p.slotC].inv_scale;
        const float f_conv = p.table[p.slotA].scale * p.table[p.slotB].scale * q_out;
        const float s_res = p.residual ? p.table[p.slot_res].scale * q_out : 0.0f;
        float fmax_probe = 0.0f, fstat = 0.0f;
        const bool fast = sh >= 1 && sh <= 31;
        const unsigned rmask = fast ? (1u << sh) - 1u : 0u, rhalf = fast ? 1u << (sh - 1) : 0u;
        int ti = 0;
        bool ok = true;
        const long long t_start = clock64();
        long long t_wait = 0, t_ld = 0, t_arr = 0, t_all = 0;
        for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++ti) {
            const int buf = ti % p.nbuf;
            if (buf != set) continue;
            const long long row = (long long)tile * 128 + quarter * 32 + lane;   // (pq*N + n)
            // the residual of the first piece is fetched while the tile is still being multiplied
            short rz[8];
            if (p.fused && p.residual) {
                const int cc0 = part * 8;
                const long long base = (long long)(ncol0 + cc0) * p.ldc + row;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    rz[j] = cc0 + j < kt ? p.residual[base + (long long)j * p.ldc] : (short)0;
            }
            const long long tw = clock64();
            if (ok && !mbar_wait_relaxed(&tmem_full[buf], (ti / p.nbuf) & 1)) { atomicExch(fail_flag, 1); ok = false; }
            t_wait += clock64() - tw;
            tc_fence_after();
            const unsigned lane_addr = tmem_base + buf * acc_cols + ((unsigned)(quarter * 32) << 16);
            // 128 * (sum of this row's activations), from the extra column p.kt
            const long long te0 = clock64();
            const int s_hi = (int)tmem_ld1(lane_addr + bn + p.kt);
            const int s_lo = (int)tmem_ld1(lane_addr + 2 * bn + p.kt);
            tmem_ld_wait();
            const long long fix = 128LL * (256LL * (long long)s_hi + (long long)s_lo);
            const float fixf = (float)fix;
            if (p.fused) {
                // fp32 epilogue: the exact integer sum scaled to a real value, bias and residual
                // added, ReLU, ONE quantisation with the output's exponent.  Eight columns at a
                // time (the register budget of a 608-thread CTA), loads first, then arithmetic,
                // then stores: eight independent chains.
                {
                    // the warps that share a lane quarter take the 8-column pieces in turn
                    for (int cc0 = part * 8; cc0 < kt; cc0 += 8 * epi_w) {
                        unsigned hh[8], xx[8], ll[8];
                        tmem_ld8(lane_addr + cc0, hh);
                        tmem_ld8(lane_addr + bn + cc0, xx);
                        tmem_ld8(lane_addr + 2 * bn + cc0, ll);
                        const long long base = (long long)(ncol0 + cc0) * p.ldc + row;
                        const int live = kt - cc0;
                        float y[8];
                        if (p.residual) {
#pragma unroll
                            for (int j = 0; j < 8; ++j) y[j] = (float)rz[j] * s_res;
                            // and the next piece's, one piece ahead of its use
                            const int nx = cc0 + 8 * epi_w;
                            if (nx < kt) {
                                const long long nbase = (long long)(ncol0 + nx) * p.ldc + row;
#pragma unroll
                                for (int j = 0; j < 8; ++j)
                                    rz[j] = nx + j < kt ? p.residual[nbase + (long long)j * p.ldc] : (short)0;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 8; ++j) y[j] = 0.0f;
                        }
                        tmem_ld_wait();
                        if (!ok) continue;
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            // three exact-or-correctly-rounded conversions instead of a 64-bit sum:
                            // the fp32 result is quantised to 16 bits right after
                            const float acc = fmaf((float)(int)hh[j], 65536.0f,
                                                   fmaf((float)(int)xx[j], 256.0f, (float)(int)ll[j] + fixf));
                            y[j] += fmaf(acc, f_conv, bias_s[cc0 + j]);
                        }
                        if (p.relu) {
#pragma unroll
                            for (int j = 0; j < 8; ++j) y[j] = fmaxf(y[j], 0.0f);      // also NaN -> 0
                        } else if (!p.probe) {
#pragma unroll
                            for (int j = 0; j < 8; ++j) y[j] = (y[j] != y[j]) ? 0.0f : fmaxf(y[j], -32768.0f);
                        }
                        if (p.probe) {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                if (j < live) fmax_probe = fmaxf(fmax_probe, fabsf(y[j]));
                            continue;
                        }
                        // y is already in units of the output's step (see f_conv): clamp, round to
                        // nearest even by the magic-number add; the low 16 bits of the sum are the
                        // mantissa, so the bytes are stored straight from it
                        int m[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            y[j] = fminf(y[j], 32767.0f);
                            m[j] = __float_as_int(y[j] + 12582912.0f);
                        }
                        if (live >= 8) {
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                fstat = fmaxf(fstat, fabsf(y[j]));
                                const long long at = base + (long long)j * p.ldc;
                                if (p.write_i16) ((short*)p.O)[at] = (short)m[j];
                                if (p.out_planes) {
                                    p.out_planes[at] = (unsigned char)(m[j] >> 8);
                                    p.out_planes[p.out_plane_bytes + at] = (unsigned char)m[j];
                                }
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                if (j < live) {
                                    fstat = fmaxf(fstat, fabsf(y[j]));
                                    const long long at = base + (long long)j * p.ldc;
                                    if (p.write_i16) ((short*)p.O)[at] = (short)m[j];
                                    if (p.out_planes) {
                                        p.out_planes[at] = (unsigned char)(m[j] >> 8);
                                        p.out_planes[p.out_plane_bytes + at] = (unsigned char)m[j];
                                    }
                                }
                            }
                        }
                    }
                }
            } else
            for (int c0 = part * 16; c0 < kt; c0 += 16 * epi_w) {
                unsigned hh[16], xx[16], ll[16];
                tmem_ld16(lane_addr + c0, hh);
                tmem_ld16(lane_addr + bn + c0, xx);
                tmem_ld16(lane_addr + 2 * bn + c0, ll);
                tmem_ld_wait();
                t_ld += clock64() - te0;
                if (!ok) continue;
                short* out = (short*)p.O + (long long)(ncol0 + c0) * p.ldc + row;
                long long v[16];
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    v[j] = ((long long)(int)hh[j] << 16) + ((long long)(int)xx[j] << 8) +
                           (long long)(int)ll[j] + fix;
                if (p.probe) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const unsigned long long a = (unsigned long long)(v[j] < 0 ? -v[j] : v[j]);
                        if (c0 + j < kt) pmax = a > pmax ? a : pmax;
                    }
                    continue;
                }
                // all sixteen values first, then the stores: independent chains for the scheduler
                int q[16];
                if (fast) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) q[j] = rescale_i64_fast(v[j], sh, rmask, rhalf);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) q[j] = rescale_i64(v[j], sh);
                }
                const int live = kt - c0;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (j < live) {
                        const int a = q[j] < 0 ? -q[j] : q[j];
                        stat = a > stat ? a : stat;
                        out[(long long)j * p.ldc] = (short)q[j];
                    }
                }
            }
            // this warp has read its part of the accumulator set
            const long long te1 = clock64();
            tc_fence_before();
            __syncwarp();
            // tell the thread that fills this set next (tile ti + nbuf of this CTA, if there is one)
            if (lane == 0 && ti + p.nbuf < n_my)
                mbar_arrive(&tmem_empty[((ti + p.nbuf) % n_mma_e) * 4 + buf]);
            t_arr += clock64() - te1;
            t_all += clock64() - te0;
        }
        if (p.dbg && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 64) {
            p.dbg[5] = clock64() - t_start; p.dbg[6] = t_wait; p.dbg[7] = ti;
            p.dbg[10] = t_ld; p.dbg[11] = t_arr; p.dbg[12] = t_all;
        }
        if (p.probe) {
            // fused: the bit pattern of max |y| (fp32); plain: max |integer sum|
            if (p.fused) pmax = (unsigned long long)__float_as_uint(fmax_probe);
            for (int o = 16; o > 0; o >>= 1) {
                const unsigned long long t = __shfl_xor_sync(0xffffffffu, pmax, o);
                pmax = t > pmax ? t : pmax;
            }
            if (lane == 0 && pmax) atomicMax(p.probe_out, pmax);
        } else {
            // fused epilogue: the largest |value| before rounding (rounding is monotonic)
            const int fs = (int)rintf(fstat);
            stat = fs > stat ? fs : stat;
            for (int o = 16; o > 0; o >>= 1) {
                const int t = __shfl_xor_sync(0xffffffffu, stat, o);
                stat = t > stat ? t : stat;
            }
            if (lane == 0 && stat) atomicMax(p.stats + p.slotC, stat);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, p.tmem_cols);
    }
    if (threadIdx.x == 0 && *fail_flag && p.status) atomicExch(p.status, 1);
}

// activations -> two operand planes in the same C,H,W,N layout (elementwise)
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
split_same_layout_kernel(const T* __restrict__ src, long long n, void* __restrict__ plane0,
                         void* __restrict__ plane1, unsigned lo_xor = 0) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    if (MODE == MODE_FLEX16 && (n & 7) == 0 && (((uintptr_t)src | (uintptr_t)plane0 |
                                                  (uintptr_t)plane1) & 15) == 0) {
        // eight mantissas per thread: one 16-byte load, two 8-byte stores
        for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < n / 8; v += stride) {
            const int4 w = __ldcs(reinterpret_cast<const int4*>(src) + v);
            const unsigned x[4] = {(unsigned)w.x, (unsigned)w.y, (unsigned)w.z, (unsigned)w.w};
            unsigned hi[2] = {0, 0}, lo[2] = {0, 0};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                // each word holds two int16: low byte of each -> lo plane; (m - lo) >> 8 is just
                // the high byte of the two's-complement pattern
                const unsigned l2 = __byte_perm(x[j], 0, 0x4420);   // bytes 0 and 2
                const unsigned h2 = __byte_perm(x[j], 0, 0x4431);   // bytes 1 and 3
                lo[j >> 1] |= (l2 & 0xffffu) << (16 * (j & 1));
                hi[j >> 1] |= (h2 & 0xffffu) << (16 * (j & 1));
            }
            reinterpret_cast<uint2*>(plane0)[v] = make_uint2(hi[0], hi[1]);
            reinterpret_cast<uint2*>(plane1)[v] = make_uint2(lo[0] ^ lo_xor, lo[1] ^ lo_xor);
        }
        return;
    }
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        if (MODE == MODE_FLEX16) {
            const int m = (int)src[i];
            const int lo = m & 0xff;
            ((signed char*)plane0)[i] = (signed char)((m - lo) >> 8);
            ((unsigned char*)plane1)[i] = (unsigned char)lo;
        } else {
            const float a = (float)src[i];
            unsigned hb;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hb) : "f"(a));
            const float hi = __uint_as_float(hb);
            ((float*)plane0)[i] = hi;
            ((float*)plane1)[i] = a - hi;
        }
    }
}

// filters C,R,S,K -> ONE array [ntn][2*bn rows][kp] for the implicit kernel: for every CTA column
// the high bytes of its kt output channels (rows 0..bn-1) and, behind them, the low bytes minus
// 128 as signed bytes (rows bn..2bn-1).  Row kt of either half is the sum column: 0 in the high
// half, +1 in the low half, on every K position the MMAs touch.  The K positions of chunk cc start
// at cc*kc_pad and run over (channel within the chunk, r, s); padding positions and channels
// beyond C hold the filter value 0 (bytes 0 and -128).
template <typename T>
__global__ void __launch_bounds__(256)
filter_planes_kernel(const T* __restrict__ F, int C, int RS, int K, int cu, int cchunks, int kc_pad,
                     int ntn, int bn, int kt, int kp, int bprop, unsigned char* __restrict__ planes) {
    const long long total = (long long)ntn * 2 * bn * kp;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int kc = (int)(i % kp);
        const int r2 = (int)((i / kp) % (2 * bn)), tile = (int)(i / ((long long)kp * 2 * bn));
        const bool low = r2 >= bn;
        const int col = low ? r2 - bn : r2;
        const int cc = kc / kc_pad, within = kc - cc * kc_pad;
        int m = 0;                                           // the filter mantissa at this position
        bool sum_col = false;
        if (col == kt) {
            sum_col = cc < cchunks;
        } else if (col < kt && tile * kt + col < K && cc < cchunks && within < cu * RS) {
            const int cl = within / RS, tap = within - cl * RS;
            const int c = cc * cu + cl;
            // bprop: the filter tensor is that of the FORWARD convolution, [K outputs here = its
            // input channels][R][S][C reduced here = its output channels], read flipped
            if (c < C)
                m = bprop ? (int)F[((long long)(tile * kt + col) * RS + (RS - 1 - tap)) * C + c]
                          : (int)F[((long long)c * RS + tap) * K + tile * kt + col];
        }
        unsigned char v;
        if (sum_col) v = low ? 1 : 0;
        else {
            const int lo = m & 0xff;
            v = low ? (unsigned char)(lo ^ 0x80) : (unsigned char)(((m - lo) >> 8) & 0xff);
        }
        planes[i] = v;
    }
}

// int8 plane in C,H,W,N layout; box = [cu][R][S][128 images]
int make_map_4d(CUtensorMap* map, void* base, const ConvGeom& g, int cu) {
    cuuint64_t dims[4] = {(cuuint64_t)g.N, (cuuint64_t)g.W, (cuuint64_t)g.H, (cuuint64_t)g.C};
    cuuint64_t strides[3] = {(cuuint64_t)g.N, (cuuint64_t)g.W * g.N, (cuuint64_t)g.H * g.W * g.N};
    cuuint32_t box[4] = {(cuuint32_t)kKBytes, (cuuint32_t)g.S, (cuuint32_t)g.R, (cuuint32_t)cu};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, base, dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return b2::fail(B2_ERR_CUDA, "cuTensorMapEncodeTiled (4-d) failed (%d)", (int)r);
    return B2_OK;
}

struct ImplicitShape {
    int ntn, kt, bn, nbuf, tmem_cols, cu, cchunks, kc_pad, npanels, kp, nstages, smem;
    size_t act_plane, filt_bytes, bytes;
};

ImplicitShape implicit_shape(const ConvGeom& g) {
    ImplicitShape s;
    // output channels per CTA column: at most 127, so that with the sum column the two filter
    // planes make one operand of at most 256 rows
    s.ntn = (g.K + 126) / 127;
    s.kt = (g.K + s.ntn - 1) / s.ntn;
    s.bn = round_up(s.kt + 1, 16);
    const int sets = 512 / (3 * s.bn);
    s.nbuf = sets >= 4 ? 4 : sets >= 3 ? 3 : sets >= 2 ? 2 : 1;
    s.tmem_cols = 32;
    while (s.tmem_cols < 3 * s.bn * s.nbuf) s.tmem_cols *= 2;
    const int RS = g.R * g.S;
    // 16 channels per chunk for real windows (a 3x3 chunk is 144 rows = 18 KB per plane); a 1x1
    // filter takes up to 128 channels per chunk
    s.cu = RS > 1 ? 16 : (g.C >= 128 ? 128 : round_up(g.C, 32));
    s.cchunks = (g.C + s.cu - 1) / s.cu;
    s.kc_pad = round_up(s.cu * RS, 32);
    s.kp = round_up(s.cchunks * s.kc_pad, kKBytes);
    s.npanels = s.kp / kKBytes;
    const int filt_smem = s.npanels * 2 * s.bn * kKBytes;
    const int stage = 2 * s.kc_pad * 128;
    int nst = (kConvSmemMax - kConvSmemFixed - filt_smem) / stage;
    if (nst > kConvMaxStages) nst = kConvMaxStages;
    s.nstages = nst;
    s.smem = kConvSmemFixed + filt_smem + (nst > 0 ? nst : 0) * stage;
    s.act_plane = (((size_t)g.C * g.H * g.W * g.N) + 1023) / 1024 * 1024;
    s.filt_bytes = (((size_t)s.ntn * 2 * s.bn * s.kp) + 1023) / 1024 * 1024;
    s.bytes = 2 * s.act_plane + s.filt_bytes;
    return s;
}

// flex16 only: an MN-major tf32 operand needs the 32-byte-atom variant of the 128-byte swizzle
// (both in the tensor map and in the matrix descriptor); with the plain 128-byte swizzle the
// tensor core reads zeros.  fp32 convolutions therefore stay on the gather + K-major path, and so
// do dilated filters and windows too large for two stages of shared memory.
bool implicit_ok(int mode, const ConvGeom& g) {
    if (mode != MODE_FLEX16 || g.N % 128 != 0 || g.dil_h != 1 || g.dil_w != 1) return false;
    if (!flat_depth(g)) return false;
    if (g.R > 256 || g.S > 256 || (long long)g.P * g.Q * (g.N / 128) >= (1LL << 30)) return false;
    // the exact int32 sums: |X| <= 2*128*255 per K row
    if ((long long)g.C * g.R * g.S + 32 > 32768) return false;
    return implicit_shape(g).nstages >= 2;
}

// The input gradient of a convolution is itself a unit-stride convolution: of the error tensor
// (K channels, P x Q), with zeros put between its elements when the forward pass was strided,
// with the filters flipped and transposed, padded by R-1-pad.  The dilated tensor is H+2pad-R+1
// high (for unit stride that is P), so that the result is exactly H high.  Returns false where
// this does not hold or does not pay (filter dilation, padding larger than the window allows,
// strides whose zero-filling would multiply the work by more than four).
bool bprop_as_fprop(const ConvGeom& f, ConvGeom* g) {
    if (f.dil_h != 1 || f.dil_w != 1 || f.str_h * f.str_w > 4 || !flat_depth(f)) return false;
    if (f.pad_h > f.R - 1 || f.pad_w > f.S - 1) return false;
    const int he = f.H + 2 * f.pad_h - f.R + 1, we = f.W + 2 * f.pad_w - f.S + 1;
    if (he < (f.P - 1) * f.str_h + 1 || we < (f.Q - 1) * f.str_w + 1) return false;
    *g = f;
    g->C = f.K; g->H = he; g->W = we; g->K = f.C; g->P = f.H; g->Q = f.W;
    g->pad_h = f.R - 1 - f.pad_h; g->pad_w = f.S - 1 - f.pad_w;
    g->str_h = g->str_w = 1;
    g->up_h = f.str_h; g->up_w = f.str_w; g->src_h = f.P; g->src_w = f.Q;
    return true;
}

// geometry of the implicit kernel for a pass (0 forward, 1 input gradient); false if unsupported
bool pass_geom(const ConvGeom& f, int pass, ConvGeom* g) {
    if (pass == 0) { *g = f; return implicit_ok(MODE_FLEX16, f); }
    return pass == 1 && bprop_as_fprop(f, g) && implicit_ok(MODE_FLEX16, *g);
}

// The three parts of an implicit-GEMM forward convolution: the two operand pre-passes (which a
// caller can skip when it already holds the planes) and the tile kernel.
// int16 tensor [C][src_h][src_w][N] -> the two byte planes of its zero-dilated form
// [C][H][W][N]; eight images per thread (N is a multiple of 128 on this path).
__global__ void __launch_bounds__(256)
dilate_planes_kernel(const short* __restrict__ src, ConvGeom g, long long n8,
                     void* __restrict__ plane0, void* __restrict__ plane1) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    const int nv = g.N / 8;
    for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < n8; v += stride) {
        const int n = (int)(v % nv);
        long long r = v / nv;
        const int w = (int)(r % g.W); r /= g.W;
        const int h = (int)(r % g.H);
        const int c = (int)(r / g.H);
        const int sh = h / g.up_h, sw = w / g.up_w;
        unsigned hi[2] = {0, 0}, lo[2] = {0, 0};
        if (sh * g.up_h == h && sw * g.up_w == w && sh < g.src_h && sw < g.src_w) {
            const long long at = (((long long)c * g.src_h + sh) * g.src_w + sw) * nv + n;
            const int4 q = __ldcs(reinterpret_cast<const int4*>(src) + at);
            const unsigned x[4] = {(unsigned)q.x, (unsigned)q.y, (unsigned)q.z, (unsigned)q.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const unsigned l2 = __byte_perm(x[j], 0, 0x4420);   // low bytes of the two int16
                const unsigned h2 = __byte_perm(x[j], 0, 0x4431);   // high bytes
                lo[j >> 1] |= (l2 & 0xffffu) << (16 * (j & 1));
                hi[j >> 1] |= (h2 & 0xffffu) << (16 * (j & 1));
            }
        }
        reinterpret_cast<uint2*>(plane0)[v] = make_uint2(hi[0], hi[1]);
        reinterpret_cast<uint2*>(plane1)[v] = make_uint2(lo[0], lo[1]);
    }
}

template <typename T, int MODE>
int implicit_split_activations(const T* I, const ConvGeom& g, const ImplicitShape& s, void* planes,
                               cudaStream_t st) {
    const long long n_act = (long long)g.C * g.H * g.W * g.N;
    long long blocks = (n_act / 8 + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (blocks < 1) blocks = 1;
    if (g.up_h != 1 || g.up_w != 1 || g.src_h != g.H || g.src_w != g.W) {
        B2_REQUIRE(MODE == MODE_FLEX16 && g.N % 8 == 0 && ((uintptr_t)I & 15) == 0,
                   "the dilated planes need int16 data, 16-byte aligned, N a multiple of 8");
        dilate_planes_kernel<<<(unsigned)blocks, 256, 0, st>>>(
            (const short*)I, g, n_act / 8, planes, (unsigned char*)planes + s.act_plane);
        B2_CUDA(cudaGetLastError());
        return B2_OK;
    }
    split_same_layout_kernel<T, MODE><<<(unsigned)blocks, 256, 0, st>>>(
        I, n_act, planes, (unsigned char*)planes + s.act_plane);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

template <typename T, int MODE>
int implicit_filter_planes(const T* F, const ConvGeom& g, const ImplicitShape& s, void* planes,
                           cudaStream_t st, int bprop = 0) {
    const long long n_f = (long long)s.ntn * 2 * s.bn * s.kp;
    long long fb = (n_f + 255) / 256;
    if (fb > 148 * 8) fb = 148 * 8;
    filter_planes_kernel<T><<<(unsigned)fb, 256, 0, st>>>(F, g.C, g.R * g.S, g.K, s.cu, s.cchunks,
                                                        s.kc_pad, s.ntn, s.bn, s.kt, s.kp, bprop,
                                                        (unsigned char*)planes);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

int implicit_tiles(const void* act_planes, const void* filt_planes, void* O, const ConvGeom& g,
                   const ImplicitShape& s, const b2_flex_scale* table, int slotI, int slotF,
                   int slotO, int* stats, unsigned long long* probe_out, int* status, int probe,
                   cudaStream_t st, const b2_conv_epilogue* epi = nullptr) {
    int rc = get_encode();
    if (rc) return rc;
    B2_REQUIRE((((uintptr_t)act_planes | (uintptr_t)filt_planes) & 1023) == 0,
               "operand planes must be 1024-byte aligned");
    void* A0 = (void*)act_planes; void* A1 = (unsigned char*)act_planes + s.act_plane;
    CUtensorMap mI0, mI1, mB;
    if ((rc = make_map_4d(&mI0, A0, g, s.cu))) return rc;
    if ((rc = make_map_4d(&mI1, A1, g, s.cu))) return rc;
    if ((rc = make_map(&mB, (void*)filt_planes, s.ntn * 2 * s.bn, s.kp, 1, 2 * s.bn))) return rc;
    ConvTileParams p;
    p.P = g.P; p.Q = g.Q; p.N = g.N; p.K = g.K;
    p.pad_h = g.pad_h; p.pad_w = g.pad_w; p.str_h = g.str_h; p.str_w = g.str_w;
    p.cu = s.cu; p.cchunks = s.cchunks; p.kc_pad = s.kc_pad;
    p.box_bytes = s.cu * g.R * g.S * 128;
    p.npanels = s.npanels; p.nstages = s.nstages;
    p.bn = s.bn; p.kt = s.kt; p.nbuf = s.nbuf; p.tmem_cols = s.tmem_cols;
    p.nblk = g.N / 128;
    p.num_tiles = g.P * g.Q * p.nblk;
    p.ldc = (long long)g.P * g.Q * g.N;
    p.O = O; p.table = table; p.slotA = slotI; p.slotB = slotF; p.slotC = slotO;
    p.stats = stats; p.probe_out = probe_out; p.status = status; p.probe = probe;
    p.fused = 0; p.bias = nullptr; p.residual = nullptr; p.slot_bias = p.slot_res = 0; p.relu = 0;
    p.write_i16 = 1; p.out_planes = nullptr; p.out_plane_bytes = 0;
    if (epi) {
        B2_REQUIRE(!epi->bias || epi->slot_bias >= 0, "bias needs its scale slot");
        B2_REQUIRE(!epi->residual || epi->slot_residual >= 0, "residual needs its scale slot");
        B2_REQUIRE(epi->write_int16 || epi->out_planes, "the fused epilogue stores nothing");
        B2_REQUIRE(!epi->out_planes || ((uintptr_t)epi->out_planes & 15) == 0, "planes alignment");
        p.fused = 1;
        p.bias = epi->bias; p.slot_bias = epi->slot_bias;
        p.residual = epi->residual; p.slot_res = epi->slot_residual;
        p.relu = epi->relu ? 1 : 0;
        p.write_i16 = epi->write_int16 ? 1 : 0;
        p.out_planes = (unsigned char*)epi->out_planes;
        p.out_plane_bytes = (long long)epi->plane_bytes;
    }
    {
        // profiling aid: B2_CONV_DBG=<device address> makes CTA 0 write 8 cycle counters there
        const char* e = getenv("B2_CONV_DBG");
        p.dbg = e ? (long long*)strtoull(e, nullptr, 0) : nullptr;
    }
    static bool attr_set = false;
    if (!attr_set) {
        B2_CUDA(cudaFuncSetAttribute(conv_implicit_kernel,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, kConvSmemMax));
        attr_set = true;
    }
    dim3 grid(p.num_tiles < 148 ? p.num_tiles : 148, s.ntn);
    // a CTA with one or two tiles has no use for more accumulator sets than tiles: with fewer
    // sets, more epilogue warps share the columns of each
    const int per_cta = (p.num_tiles + (int)grid.x - 1) / (int)grid.x;
    if (per_cta < p.nbuf) p.nbuf = per_cta >= 4 ? 4 : per_cta == 3 ? 3 : per_cta == 2 ? 2 : 1;
    p.n_mma = p.nbuf >= 3 ? 3 : p.nbuf;
    if (const char* e = getenv("B2_CONV_ISSUERS")) {      // measurement aid: 1..3
        const int want = atoi(e);
        if (want >= 1 && want < p.n_mma) p.n_mma = want;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(kConvThreads); cfg.dynamicSmemBytes = s.smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = getenv("B2_CONV_NO_PDL") ? 0 : 1;
    B2_CUDA(cudaLaunchKernelEx(&cfg, conv_implicit_kernel, mI0, mI1, mB, p));
    return B2_OK;
}

template <typename T, int MODE>
int run_fprop_implicit(const T* I, const T* F, void* O, const ConvGeom& g,
                       const b2_flex_scale* table, int slotI, int slotF, int slotO, int* stats,
                       void* scratch, size_t scratch_bytes, unsigned long long* probe_out,
                       int* status, int probe, cudaStream_t st) {
    const ImplicitShape s = implicit_shape(g);
    B2_REQUIRE(scratch && scratch_bytes >= s.bytes && ((uintptr_t)scratch & 1023) == 0,
               "convolution needs %zu bytes of 1024-byte aligned scratch, got %zu", s.bytes,
               scratch_bytes);
    unsigned char* base = (unsigned char*)scratch;
    int rc = implicit_split_activations<T, MODE>(I, g, s, base, st);
    if (rc) return rc;
    if ((rc = implicit_filter_planes<T, MODE>(F, g, s, base + 2 * s.act_plane, st))) return rc;
    return implicit_tiles(base, base + 2 * s.act_plane, O, g, s, table, slotI, slotF, slotO, stats,
                          probe_out, status, probe, st);
}

template <typename T, int MODE>
int run_fprop(const T* I, const T* F, void* O, const b2_conv_dims* d, const b2_flex_scale* table,
              int slotI, int slotF, int slotO, int* stats, void* scratch, size_t scratch_bytes,
              unsigned long long* probe_out, int* status, int probe, cudaStream_t st) {
    ConvGeom g;
    int rc = geom_from(d, &g);
    if (rc) return rc;
    B2_REQUIRE(I && F && O, "null tensor");
    if (implicit_ok(MODE, g) && !getenv("B2_CONV_IM2COL"))
        return run_fprop_implicit<T, MODE>(I, F, O, g, table, slotI, slotF, slotO, stats, scratch,
                                           scratch_bytes, probe_out, status, probe, st);
    const long long rows_ll = (long long)g.M * g.P * g.Q * g.N;
    B2_REQUIRE(rows_ll < (1LL << 31) - 256, "too many output positions");
    B2_REQUIRE((long long)g.C * g.T * g.R * g.S < (1LL << 24), "filter window too large");
    const int rows = (int)rows_ll, kg = g.C * g.T * g.R * g.S;
    if (MODE == MODE_FLEX16) B2_REQUIRE(kg <= 32768, "flex16 convolution needs C*T*R*S <= 32768");
    const Shapes s = shapes_for(MODE, rows, g.K, kg);
    B2_REQUIRE(scratch && scratch_bytes >= s.bytes && ((uintptr_t)scratch & 1023) == 0,
               "convolution needs %zu bytes of 1024-byte aligned scratch, got %zu", s.bytes,
               scratch_bytes);
    unsigned char* base = (unsigned char*)scratch;
    const size_t a_plane = (size_t)s.Mp * s.Kp * s.esize, b_plane = (size_t)s.Np * s.Kp * s.esize;
    {
        B2_REQUIRE((long long)g.C * g.D * g.H * g.W * g.N < (1LL << 31), "input tensor too large");
        im2col_planes_kernel<T, MODE, false><<<s.Mp / 32, 256, 0, st>>>(I, g, rows, kg, s.Mp, s.Kp,
                                                                base, base + a_plane);
        // filters: element (n = k_out, k = kidx) = F[kidx * K + k_out]
        B2_CUDA(cudaGetLastError());
        rc = split_operand<T, MODE>(F, 1, g.K, g.K, kg, s.Np, s.Kp, base + 2 * a_plane,
                                    base + 2 * a_plane + b_plane, 0, nullptr, st);
        if (rc) return rc;
    }
    GemmParams p;
    p.M = rows; p.N = g.K; p.num_kb = 0;
    p.ldc = rows; p.C = O; p.table = table; p.slotA = slotI; p.slotB = slotF; p.slotC = slotO;
    p.stats = stats; p.probe_out = probe_out; p.status = status; p.probe = probe;
    p.c_colmajor = 1;
    p.rowsum = nullptr;
    return launch_on_planes<MODE>(base, s, p, st);
}

// ---- training contractions -------------------------------------------------------------------
// filter planes for bprop: row = c, column = (k*R + r_)*S + s_, value F[((c*R + r_)*S + s_)*K + k]
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
filter_bprop_planes_kernel(const T* __restrict__ F, int C, int RS, int K, int rows_p, int kp,
                           void* __restrict__ plane0, void* __restrict__ plane1) {
    const long long total = (long long)rows_p * kp;
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total;
         i += (long long)gridDim.x * 256) {
        const int c = (int)(i / kp), kidx = (int)(i % kp);
        T v = 0;
        if (c < C && kidx < K * RS) {
            const int k = kidx / RS, rs = kidx - k * RS;
            v = F[((long long)c * RS + rs) * K + k];
        }
        if (MODE == MODE_FLEX16) {
            const int m = (int)v, lo = m & 0xff;
            ((signed char*)plane0)[i] = (signed char)((m - lo) >> 8);
            ((unsigned char*)plane1)[i] = (unsigned char)lo;
        } else {
            float hi, lo;
            tf32_split((float)v, hi, lo);
            ((float*)plane0)[i] = hi;
            ((float*)plane1)[i] = lo;
        }
    }
}

// A planes of the update contraction: row = (c*R + r_)*S + s_, column = (p*Q + q)*N + n, value
// I[c, p*str - pad + r_*dil, q*str - pad + s_*dil, n] (zero outside the image).  One thread writes
// 16 (flex16) or 4 (fp32) consecutive columns; they share (p, q) when N is a multiple of that.
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
update_planes_kernel(const T* __restrict__ I, ConvGeom g, int rows, int kg, int rows_p, int kp,
                     void* __restrict__ plane0, void* __restrict__ plane1) {
    constexpr int kPer = MODE == MODE_FLEX16 ? 16 : 4;
    const int upr = kp / kPer;
    const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;
    if (idx >= (long long)rows_p * upr) return;
    const int m = (int)(idx / upr), j0 = (int)(idx % upr) * kPer;
    __align__(16) T v[kPer];
#pragma unroll
    for (int e = 0; e < kPer; ++e) v[e] = 0;
    if (m < rows && j0 < kg) {
        const int RS = g.R * g.S, TRS = g.T * RS;
        const int c = m / TRS, trs = m - c * TRS, ft = trs / RS, rs = trs - ft * RS;
        const int fr = rs / g.S, fs = rs - fr * g.S;
        const T* plane = I + (long long)c * g.D * g.H * g.W * g.N;
        const bool fast = (g.N % kPer == 0) && ((uintptr_t)I & 15) == 0;
        if (fast) {
            const int n0 = j0 % g.N, pq = j0 / g.N, q = pq % g.Q, mp = pq / g.Q, pp = mp % g.P;
            const int dd = (mp / g.P) * g.str_d - g.pad_d + ft * g.dil_d;
            const int h = pp * g.str_h - g.pad_h + fr * g.dil_h;
            const int w = q * g.str_w - g.pad_w + fs * g.dil_w;
            if (h >= 0 && h < g.H && w >= 0 && w < g.W && dd >= 0 && dd < g.D) {
                const T* sp = plane + (((long long)dd * g.H + h) * g.W + w) * g.N + n0;
                if (MODE == MODE_FLEX16) {
                    const int4 a = __ldg((const int4*)sp), b = __ldg((const int4*)sp + 1);
                    *(int4*)&v[0] = a;
                    *(int4*)&v[8 % kPer] = b;
                } else {
                    *(float4*)&v[0] = __ldg((const float4*)sp);
                }
            }
        } else {
#pragma unroll
            for (int e = 0; e < kPer; ++e) {
                const int j = j0 + e;
                if (j >= kg) break;
                const int n = j % g.N, pq = j / g.N, q = pq % g.Q, mp = pq / g.Q, pp = mp % g.P;
                const int dd = (mp / g.P) * g.str_d - g.pad_d + ft * g.dil_d;
                const int h = pp * g.str_h - g.pad_h + fr * g.dil_h;
                const int w = q * g.str_w - g.pad_w + fs * g.dil_w;
                if (h >= 0 && h < g.H && w >= 0 && w < g.W && dd >= 0 && dd < g.D)
                    v[e] = plane[(((long long)dd * g.H + h) * g.W + w) * g.N + n];
            }
        }
    }
    const long long o = (long long)m * kp + j0;
    if (MODE == MODE_FLEX16) {
        unsigned hi[4] = {0, 0, 0, 0}, lo[4] = {0, 0, 0, 0};
#pragma unroll
        for (int e = 0; e < kPer; ++e) {
            const int mm = (int)v[e], l = mm & 0xff;
            hi[e >> 2] |= (unsigned)(((mm - l) >> 8) & 0xff) << (8 * (e & 3));
            lo[e >> 2] |= (unsigned)l << (8 * (e & 3));
        }
        *(uint4*)((unsigned char*)plane0 + o) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *(uint4*)((unsigned char*)plane1 + o) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    } else {
        float hi[4], lo[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) tf32_split((float)v[e % kPer], hi[e], lo[e]);
        *(float4*)((float*)plane0 + o) = make_float4(hi[0], hi[1], hi[2], hi[3]);
        *(float4*)((float*)plane1 + o) = make_float4(lo[0], lo[1], lo[2], lo[3]);
    }
}

inline void fill_params(GemmParams* p, int M, int N, long long ldc, void* C, int colmajor,
                        const b2_flex_scale* table, int slotA, int slotB, int slotC, int* stats,
                        unsigned long long* probe_out, int* status, int probe) {
    p->M = M; p->N = N; p->num_kb = 0; p->ldc = ldc; p->C = C; p->table = table;
    p->slotA = slotA; p->slotB = slotB; p->slotC = slotC; p->stats = stats;
    p->probe_out = probe_out; p->status = status; p->probe = probe; p->c_colmajor = colmajor;
    p->rowsum = nullptr;
}

struct TrainShape { Shapes s; int splits; size_t bytes; };

TrainShape bprop_shape(int mode, const ConvGeom& g) {
    TrainShape t;
    t.s = shapes_for(mode, g.D * g.H * g.W * g.N, g.C, g.K * g.T * g.R * g.S);
    t.splits = pick_splits(mode, t.s, false);
    t.bytes = align1k(t.s.bytes) + splitk_bytes(mode, t.s, t.splits);
    return t;
}

TrainShape update_shape(int mode, const ConvGeom& g) {
    TrainShape t;
    t.s = shapes_for(mode, g.C * g.T * g.R * g.S, g.K, g.M * g.P * g.Q * g.N);
    t.splits = pick_splits(mode, t.s, true);
    t.bytes = align1k(t.s.bytes) + splitk_bytes(mode, t.s, t.splits);
    return t;
}

template <typename T, int MODE>
int run_bprop(const T* E, const T* F, void* GI, const b2_conv_dims* d, const b2_flex_scale* table,
              int slotE, int slotF, int slotG, int* stats, void* scratch, size_t scratch_bytes,
              unsigned long long* probe_out, int* status, int probe, cudaStream_t st) {
    ConvGeom g;
    int rc = geom_from(d, &g);
    if (rc) return rc;
    B2_REQUIRE(E && F && GI, "null tensor");
    ConvGeom gb;
    if (MODE == MODE_FLEX16 && pass_geom(g, 1, &gb) && !getenv("B2_CONV_IM2COL")) {
        const ImplicitShape si = implicit_shape(gb);
        B2_REQUIRE(scratch && scratch_bytes >= si.bytes && ((uintptr_t)scratch & 1023) == 0,
                   "convolution bprop needs %zu bytes of 1024-byte aligned scratch, got %zu",
                   si.bytes, scratch_bytes);
        unsigned char* base = (unsigned char*)scratch;
        if ((rc = implicit_split_activations<T, MODE>(E, gb, si, base, st))) return rc;
        if ((rc = implicit_filter_planes<T, MODE>(F, gb, si, base + 2 * si.act_plane, st, 1))) return rc;
        return implicit_tiles(base, base + 2 * si.act_plane, GI, gb, si, table, slotE, slotF, slotG,
                              stats, probe_out, status, probe, st);
    }
    const long long rows_ll = (long long)g.D * g.H * g.W * g.N;
    B2_REQUIRE(rows_ll < (1LL << 31) - 256 && (long long)g.K * g.M * g.P * g.Q * g.N < (1LL << 31) &&
               (long long)g.K * g.T * g.R * g.S < (1LL << 24), "tensor too large");
    const int rows = (int)rows_ll, kg = g.K * g.T * g.R * g.S;
    const TrainShape t = bprop_shape(MODE, g);
    const Shapes& s = t.s;
    B2_REQUIRE(scratch && scratch_bytes >= t.bytes && ((uintptr_t)scratch & 1023) == 0,
               "convolution bprop needs %zu bytes of 1024-byte aligned scratch, got %zu", t.bytes,
               scratch_bytes);
    unsigned char* base = (unsigned char*)scratch;
    const size_t a_plane = (size_t)s.Mp * s.Kp * s.esize, b_plane = (size_t)s.Np * s.Kp * s.esize;
    im2col_planes_kernel<T, MODE, true><<<s.Mp / 32, 256, 0, st>>>(E, g, rows, kg, s.Mp, s.Kp, base,
                                                                   base + a_plane);
    long long blocks = ((long long)s.Np * s.Kp + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    filter_bprop_planes_kernel<T, MODE><<<(unsigned)blocks, 256, 0, st>>>(
        F, g.C, g.T * g.R * g.S, g.K, s.Np, s.Kp, base + 2 * a_plane, base + 2 * a_plane + b_plane);
    B2_CUDA(cudaGetLastError());
    GemmParams p;
    fill_params(&p, rows, g.C, rows, GI, 1, table, slotE, slotF, slotG, stats, probe_out, status,
                probe);
    return launch_on_planes<MODE>(base, s, p, st, t.splits, base + align1k(s.bytes));
}

// ---- filter gradient on the tile kernel's operands ------------------------------------------------
// U[(c,r,s), k] = sum over (p,q,n) of I[c, p*str-pad+r, q*str-pad+s, n] * E[k, p, q, n].
// One k-block = one output pixel x 128 images.  Its A operand is the very box the forward kernel
// loads (rows (c,r,s) of one channel chunk, 128 images along the row: K-major here), its B operand
// the rows k of the error tensor's planes at that pixel.  A CTA owns a channel chunk, a tile of
// filters and a range of k-blocks; two threads issue the products of alternate k-blocks into
// accumulators of their own ([HH | Ah*El'] and [Al*Eh | LL], El' = El - 128 with the row sums of A
// taken from a constant extra row of B), and the CTA writes its exact int64 sums as one slice of
// partial[slice][C*R*S][K], which splitk_finish_kernel adds up, rescales and stores.
struct UpdTileParams {
    int Q, nblk, nkb;              // k-block kb = (p*Q + q)*nblk + nb
    int pad_h, pad_w, str_h, str_w;
    int cu, rs, C, K;              // channels per chunk, R*S
    int ntn, kt, bn;               // filter tiles: kt filters each, bn = round_up(kt + 1, 16) rows
    int per;                       // k-blocks per slice (grid.x)
    int nstages, tmem_cols;
    unsigned box_a, box_b;         // bytes of one activation box, of one error box
    long long* partial;
    int* status;
};

constexpr int kUpdThreads = 256;
constexpr int kUpdMaxStages = 6;
constexpr int kUpdAPlane = 128 * kKBytes;          // 128 rows of 128 bytes
constexpr int kUpdSmemFixed = 1024 + 512;

__global__ void __launch_bounds__(kUpdThreads, 1)
conv_update_kernel(const __grid_constant__ CUtensorMap mapI0, const __grid_constant__ CUtensorMap mapI1,
                   const __grid_constant__ CUtensorMap mapE0, const __grid_constant__ CUtensorMap mapE1,
                   const UpdTileParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* ring = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int bn = p.bn, kt = p.kt;
    const int b_bytes = 2 * bn * kKBytes;                   // [E_hi rows | E_lo' rows]
    const int stage = 2 * kUpdAPlane + b_bytes;
    unsigned long long* full_bar = (unsigned long long*)(ring + (size_t)p.nstages * stage);   // [2][max]
    unsigned long long* empty_bar = full_bar + 2 * kUpdMaxStages;
    unsigned long long* tmem_full = empty_bar + kUpdMaxStages;                               // [2]
    unsigned* tmem_holder = (unsigned*)(tmem_full + 2);
    int* fail_flag = (int*)(tmem_holder + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int chunk = blockIdx.y / p.ntn, ktile = blockIdx.y - chunk * p.ntn;
    const int kb0 = blockIdx.x * p.per;
    int mine = p.nkb - kb0;
    if (mine > p.per) mine = p.per;

    if (threadIdx.x == 0) {
        prefetch_map(&mapI0); prefetch_map(&mapI1); prefetch_map(&mapE0); prefetch_map(&mapE1);
        for (int s = 0; s < kUpdMaxStages; ++s) {
            mbar_init(&full_bar[s], 1); mbar_init(&full_bar[kUpdMaxStages + s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&tmem_full[0], 1); mbar_init(&tmem_full[1], 1);
        *fail_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_holder, p.tmem_cols);
    {
        // rows kt .. bn-1 of both parts of every stage's B tile are constants the loads never
        // touch: zero, except row kt of the low part, which is all ones (the row-sum column)
        const int rows = bn - kt, units = p.nstages * 2 * rows * 8;        // 16-byte units
        for (int i = threadIdx.x; i < units; i += kUpdThreads) {
            const int u = i & 7, r = (i >> 3) % rows, part = ((i >> 3) / rows) & 1;
            const int st = (i >> 3) / (2 * rows);
            const unsigned v = (part == 1 && r == 0) ? 0x01010101u : 0u;
            uint4* dst = (uint4*)(ring + (size_t)st * stage + 2 * kUpdAPlane +
                                  (size_t)(part * bn + kt + r) * kKBytes) + u;
            *dst = make_uint4(v, v, v, v);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = *tmem_holder;

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            unsigned empty_parity = 1;
            for (int i = 0; i < mine; ++i) {
                const int kb = kb0 + i;
                const int pq = kb / p.nblk, nb = kb - pq * p.nblk;
                const int pp = pq / p.Q, q = pq - pp * p.Q;
                unsigned long long* fb = full_bar + (i & 1) * kUpdMaxStages;
                if (!mbar_wait_relaxed(&empty_bar[s], empty_parity)) { atomicExch(fail_flag, 1); break; }
                unsigned char* sa = ring + (size_t)s * stage;
                mbar_expect_tx(&fb[s], 2 * p.box_a + 2 * p.box_b);
                tma_load_4d(sa, &mapI0, nb * 128, q * p.str_w - p.pad_w, pp * p.str_h - p.pad_h,
                            chunk * p.cu, &fb[s]);
                tma_load_4d(sa + kUpdAPlane, &mapI1, nb * 128, q * p.str_w - p.pad_w,
                            pp * p.str_h - p.pad_h, chunk * p.cu, &fb[s]);
                tma_load_2d(sa + 2 * kUpdAPlane, &mapE0, kb * 128, ktile * kt, &fb[s]);
                tma_load_2d(sa + 2 * kUpdAPlane + bn * kKBytes, &mapE1, kb * 128, ktile * kt, &fb[s]);
                if (++s == p.nstages) { s = 0; empty_parity ^= 1u; }
            }
        }
    } else if (warp == 1 || warp == 2) {
        const int id = warp - 1;
        if (lane == 0) {
            const unsigned id_s = make_idesc_n(2, 1, 1, 2 * bn), id_u = make_idesc_n(2, 0, 1, 2 * bn);
            const unsigned acc = tmem_base + id * 4 * bn;
            unsigned long long* fb = full_bar + id * kUpdMaxStages;
            unsigned phase_bits = 0, accumulate = 0;
            bool ok = true;
            for (int i = id; i < mine && ok; i += 2) {
                const int s = i % p.nstages;
                if (!mbar_wait(&fb[s], (phase_bits >> s) & 1u)) { atomicExch(fail_flag, 1); ok = false; break; }
                phase_bits ^= 1u << s;
                tc_fence_after();
                unsigned char* sa = ring + (size_t)s * stage;
                const unsigned long long dAh = make_smem_desc(sa), dAl = make_smem_desc(sa + kUpdAPlane);
                const unsigned long long dB = make_smem_desc(sa + 2 * kUpdAPlane);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    tc_mma<MODE_FLEX16>(acc, dAh + 2 * k, dB + 2 * k, id_s, accumulate);            // HH | Ah*El'
                    tc_mma<MODE_FLEX16>(acc + 2 * bn, dAl + 2 * k, dB + 2 * k, id_u, accumulate);   // Al*Eh | LL
                    accumulate = 1;
                }
                tc_commit(&empty_bar[s]);
            }
            if (accumulate) tc_commit(&tmem_full[id]);
            else mbar_arrive(&tmem_full[id]);          // no k-block of its own: nothing to wait for
        }
    } else if (warp >= 4) {
        const int quarter = warp - 4;
        const bool two = mine >= 2;                     // the second accumulator set holds sums
        bool ok = mbar_wait_relaxed(&tmem_full[0], 0);
        ok = mbar_wait_relaxed(&tmem_full[1], 0) && ok;
        if (!ok) atomicExch(fail_flag, 1);
        tc_fence_after();
        const int row = quarter * 32 + lane;
        const int cg = chunk * p.cu + row / p.rs;
        const bool valid = ok && row < p.cu * p.rs && cg < p.C;
        const unsigned a0 = tmem_base + ((unsigned)(quarter * 32) << 16), a1 = a0 + 4 * bn;
        // (the loaded registers are only read after the wait)
        const unsigned h0 = tmem_ld1(a0 + bn + kt), l0 = tmem_ld1(a0 + 3 * bn + kt);
        unsigned h1 = 0, l1 = 0;
        if (two) { h1 = tmem_ld1(a1 + bn + kt); l1 = tmem_ld1(a1 + 3 * bn + kt); }
        tmem_ld_wait();
        const long long s_hi = (long long)(int)h0 + (long long)(int)h1;
        const long long s_lo = (long long)(int)l0 + (long long)(int)l1;
        const long long fix = 128LL * (256LL * s_hi + s_lo);
        long long* out = p.partial + ((long long)blockIdx.x * p.C * p.rs + (long long)chunk * p.cu * p.rs + row) * p.K +
                         ktile * kt;
        for (int c0 = 0; c0 < kt; c0 += 8) {
            unsigned hh[8], x1[8], x2[8], ll[8];
            tmem_ld8(a0 + c0, hh); tmem_ld8(a0 + bn + c0, x1);
            tmem_ld8(a0 + 2 * bn + c0, x2); tmem_ld8(a0 + 3 * bn + c0, ll);
            tmem_ld_wait();
            long long v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                v[j] = ((long long)(int)hh[j] << 16) + (((long long)(int)x1[j] + (long long)(int)x2[j]) << 8) +
                       (long long)(int)ll[j];
            if (two) {
                tmem_ld8(a1 + c0, hh); tmem_ld8(a1 + bn + c0, x1);
                tmem_ld8(a1 + 2 * bn + c0, x2); tmem_ld8(a1 + 3 * bn + c0, ll);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    v[j] += ((long long)(int)hh[j] << 16) + (((long long)(int)x1[j] + (long long)(int)x2[j]) << 8) +
                            (long long)(int)ll[j];
            }
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (valid && c0 + j < kt && ktile * kt + c0 + j < p.K) out[c0 + j] = v[j] + fix;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, p.tmem_cols);
    }
    if (threadIdx.x == 0 && *fail_flag && p.status) atomicExch(p.status, 1);
}

struct UpdShape {
    bool ok;
    int cu, cchunks, ntn, kt, bn, tmem_cols, nstages, smem, nkb, per, nsplit;
    size_t act_plane, err_plane, partial_bytes, bytes;
};

UpdShape update_implicit_shape(int mode, const ConvGeom& g) {
    UpdShape u;
    u.ok = false;
    const int rs = g.R * g.S;
    const long long cols = (long long)g.P * g.Q * g.N;
    if (mode != MODE_FLEX16 || g.N % 128 != 0 || g.dil_h != 1 || g.dil_w != 1 || rs > 128 ||
        !flat_depth(g) ||
        g.R > 256 || g.S > 256 || cols >= (1LL << 31) - 256 || getenv("B2_CONV_IM2COL"))
        return u;
    const int cu_max = 128 / rs;
    u.cchunks = (g.C + cu_max - 1) / cu_max;
    u.cu = (g.C + u.cchunks - 1) / u.cchunks;
    u.ntn = (g.K + 62) / 63;                       // two accumulator sets of 4*bn columns in 512
    u.kt = (g.K + u.ntn - 1) / u.ntn;
    u.bn = round_up(u.kt + 1, 16);
    u.tmem_cols = 32;
    while (u.tmem_cols < 8 * u.bn) u.tmem_cols *= 2;
    const int stage = 2 * kUpdAPlane + 2 * u.bn * kKBytes;
    u.nstages = (kConvSmemMax - kUpdSmemFixed) / stage;
    if (u.nstages > kUpdMaxStages) u.nstages = kUpdMaxStages;
    if (u.nstages < 2) return u;
    u.smem = kUpdSmemFixed + u.nstages * stage;
    u.nkb = (int)(cols / 128);
    int slices = 148 / (u.cchunks * u.ntn);
    if (slices < 1) slices = 1;
    u.per = (u.nkb + slices - 1) / slices;
    if (u.per > 256) u.per = 256;                  // the int32 sums stay exact up to 32768 terms
    u.nsplit = (u.nkb + u.per - 1) / u.per;
    u.act_plane = (((size_t)g.C * g.H * g.W * g.N) + 1023) / 1024 * 1024;
    u.err_plane = (((size_t)g.K * cols) + 1023) / 1024 * 1024;
    u.partial_bytes = (size_t)u.nsplit * g.C * rs * g.K * sizeof(long long);
    u.bytes = 2 * u.act_plane + 2 * u.err_plane + align1k(u.partial_bytes);
    u.ok = true;
    return u;
}

template <typename T, int MODE>
int run_update_implicit(const T* I, const T* E, void* U, const ConvGeom& g, const UpdShape& u,
                        const b2_flex_scale* table, int slotI, int slotE, int slotU, int* stats,
                        void* scratch, size_t scratch_bytes, unsigned long long* probe_out,
                        int* status, int probe, cudaStream_t st) {
    int rc = get_encode();
    if (rc) return rc;
    B2_REQUIRE(scratch && scratch_bytes >= u.bytes && ((uintptr_t)scratch & 1023) == 0,
               "convolution update needs %zu bytes of 1024-byte aligned scratch, got %zu", u.bytes,
               scratch_bytes);
    unsigned char* base = (unsigned char*)scratch;
    unsigned char* eplanes = base + 2 * u.act_plane;
    long long* partial = (long long*)(eplanes + 2 * u.err_plane);
    const long long n_act = (long long)g.C * g.H * g.W * g.N, n_err = (long long)g.K * g.P * g.Q * g.N;
    long long blocks = (n_act / 8 + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    split_same_layout_kernel<T, MODE><<<(unsigned)(blocks < 1 ? 1 : blocks), 256, 0, st>>>(
        I, n_act, base, base + u.act_plane, 0u);
    blocks = (n_err / 8 + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    // the error tensor's low plane as signed bytes (low - 128): both of its planes then make one
    // signed operand
    split_same_layout_kernel<T, MODE><<<(unsigned)(blocks < 1 ? 1 : blocks), 256, 0, st>>>(
        E, n_err, eplanes, eplanes + u.err_plane, 0x80808080u);
    B2_CUDA(cudaGetLastError());
    CUtensorMap mI0, mI1, mE0, mE1;
    if ((rc = make_map_4d(&mI0, base, g, u.cu))) return rc;
    if ((rc = make_map_4d(&mI1, base + u.act_plane, g, u.cu))) return rc;
    const int cols = g.P * g.Q * g.N;
    if ((rc = make_map(&mE0, eplanes, g.K, cols, 1, u.kt))) return rc;
    if ((rc = make_map(&mE1, eplanes + u.err_plane, g.K, cols, 1, u.kt))) return rc;
    UpdTileParams p;
    p.Q = g.Q; p.nblk = g.N / 128; p.nkb = u.nkb;
    p.pad_h = g.pad_h; p.pad_w = g.pad_w; p.str_h = g.str_h; p.str_w = g.str_w;
    p.cu = u.cu; p.rs = g.R * g.S; p.C = g.C; p.K = g.K;
    p.ntn = u.ntn; p.kt = u.kt; p.bn = u.bn; p.per = u.per;
    p.nstages = u.nstages; p.tmem_cols = u.tmem_cols;
    p.box_a = (unsigned)(u.cu * g.R * g.S * kKBytes); p.box_b = (unsigned)(u.kt * kKBytes);
    p.partial = partial; p.status = status;
    static bool attr_set = false;
    if (!attr_set) {
        B2_CUDA(cudaFuncSetAttribute(conv_update_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     kConvSmemMax));
        attr_set = true;
    }
    dim3 grid(u.nsplit, u.cchunks * u.ntn);
    conv_update_kernel<<<grid, kUpdThreads, u.smem, st>>>(mI0, mI1, mE0, mE1, p);
    B2_CUDA(cudaGetLastError());
    GemmParams gp;
    const int rows = g.C * g.R * g.S;
    fill_params(&gp, rows, g.K, g.K, U, 0, table, slotI, slotE, slotU, stats, probe_out, status, probe);
    gp.partial = partial; gp.Mp = rows; gp.Np = g.K; gp.kb_per_split = u.per;
    long long fb = ((long long)rows * g.K + 31) / 32;
    if (fb > 148 * 16) fb = 148 * 16;
    splitk_finish_kernel<MODE><<<(unsigned)fb, 256, 0, st>>>(gp, u.nsplit);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

template <typename T, int MODE>
int run_update(const T* I, const T* E, void* U, const b2_conv_dims* d, const b2_flex_scale* table,
               int slotI, int slotE, int slotU, int* stats, void* scratch, size_t scratch_bytes,
               unsigned long long* probe_out, int* status, int probe, cudaStream_t st) {
    ConvGeom g;
    int rc = geom_from(d, &g);
    if (rc) return rc;
    B2_REQUIRE(I && E && U, "null tensor");
    {
        const UpdShape u = update_implicit_shape(MODE, g);
        if (u.ok)
            return run_update_implicit<T, MODE>(I, E, U, g, u, table, slotI, slotE, slotU, stats,
                                                scratch, scratch_bytes, probe_out, status, probe, st);
    }
    const long long kg_ll = (long long)g.M * g.P * g.Q * g.N;
    B2_REQUIRE(kg_ll < (1LL << 31) - 256 && (long long)g.C * g.D * g.H * g.W * g.N < (1LL << 31) &&
               (long long)g.C * g.T * g.R * g.S < (1LL << 24), "tensor too large");
    const int rows = g.C * g.T * g.R * g.S, kg = (int)kg_ll;
    const TrainShape t = update_shape(MODE, g);
    const Shapes& s = t.s;
    B2_REQUIRE(scratch && scratch_bytes >= t.bytes && ((uintptr_t)scratch & 1023) == 0,
               "convolution update needs %zu bytes of 1024-byte aligned scratch, got %zu", t.bytes,
               scratch_bytes);
    unsigned char* base = (unsigned char*)scratch;
    const size_t a_plane = (size_t)s.Mp * s.Kp * s.esize, b_plane = (size_t)s.Np * s.Kp * s.esize;
    const long long units = (long long)s.Mp * (s.Kp / (MODE == MODE_FLEX16 ? 16 : 4));
    update_planes_kernel<T, MODE><<<(unsigned)((units + 255) / 256), 256, 0, st>>>(
        I, g, rows, kg, s.Mp, s.Kp, base, base + a_plane);
    B2_CUDA(cudaGetLastError());
    // E is [K][(p,q,n)]: already the K-major B operand
    rc = split_operand<T, MODE>(E, (long long)kg, 1, g.K, kg, s.Np, s.Kp, base + 2 * a_plane,
                                base + 2 * a_plane + b_plane, 0, nullptr, st);
    if (rc) return rc;
    GemmParams p;
    fill_params(&p, rows, g.K, g.K, U, 0, table, slotI, slotE, slotU, stats, probe_out, status,
                probe);
    return launch_on_planes<MODE>(base, s, p, st, t.splits, base + align1k(s.bytes));
}

// ---- average pooling over H, W windows (C and D windows of 1) ------------------------------------
// out[c,p,q,n] = mean over the part of the window inside the image (the numpy reference takes
// np.mean of the clipped slice, ngraph/transformers/cpu/cpuengine.py:296-305).  flex16: the output
// shares the input's exponent (ngraph/transformers/passes/flexpass.py:40-48), so mantissas are
// averaged and rounded to nearest even.
template <typename T, bool MAX>
__global__ void __launch_bounds__(256)
pool_kernel(const T* __restrict__ I, T* __restrict__ O, int C, int H, int W, int N, int P, int Q,
            int R, int S, int pad_h, int pad_w, int str_h, int str_w, int* stats) {
    // a block takes 32 consecutive results (consecutive images: coalesced); its eight warps each
    // add every eighth element of the window, the eight partial sums are combined in warp order
    __shared__ float part[8][32];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const long long total = (long long)C * P * Q * N;
    const long long units = (total + 31) / 32;
    int stat = 0;
    for (long long u = blockIdx.x; u < units; u += gridDim.x) {
        const long long i = u * 32 + tx;
        const bool live = i < total;
        float acc = MAX ? -INFINITY : 0.0f;
        int cnt = 1;
        if (live) {
            const int n = (int)(i % N);
            long long t = i / N;
            const int q = (int)(t % Q); t /= Q;
            const int p = (int)(t % P);
            const int c = (int)(t / P);
            const int h0 = max(p * str_h - pad_h, 0), h1 = min(p * str_h - pad_h + R, H);
            const int w0 = max(q * str_w - pad_w, 0), w1 = min(q * str_w - pad_w + S, W);
            const int wlen = max(w1 - w0, 0), area = max(h1 - h0, 0) * wlen;
            cnt = max(area, 1);
            for (int e = ty; e < area; e += 8) {
                const int h = h0 + e / wlen, w = w0 + e % wlen;
                const float v = (float)I[(((long long)c * H + h) * W + w) * N + n];
                acc = MAX ? fmaxf(acc, v) : acc + v;
            }
        }
        part[ty][tx] = acc;
        __syncthreads();
        if (ty == 0 && live) {
            float sum = part[0][tx];
#pragma unroll
            for (int k = 1; k < 8; ++k) sum = MAX ? fmaxf(sum, part[k][tx]) : sum + part[k][tx];
            // (a window that lies entirely in the padding has no element: 0, as the mean gives)
            const float mean = MAX ? (sum == -INFINITY ? 0.0f : sum) : sum / (float)cnt;
            if (sizeof(T) == 2) {
                const int m = __float2int_rn(mean);
                stat = max(stat, m < 0 ? -m : m);
                O[i] = (T)m;
            } else {
                O[i] = (T)mean;
            }
        }
        __syncthreads();
    }
    if (sizeof(T) == 2 && stats && ty == 0) {
        for (int o = 16; o > 0; o >>= 1) stat = max(stat, __shfl_xor_sync(0xffffffffu, stat, o));
        if (tx == 0 && stat) atomicMax(stats, stat);
    }
}

}  // namespace

extern "C" int b2_conv_fprop_scratch_bytes(int32_t flex, const b2_conv_dims* d, size_t* bytes) {
    ConvGeom g;
    int rc = geom_from(d, &g);
    if (rc) return rc;
    B2_REQUIRE(bytes, "null argument");
    const int mode = flex ? MODE_FLEX16 : MODE_F32X3;
    size_t need = shapes_for(mode, g.M * g.P * g.Q * g.N, g.K, g.C * g.T * g.R * g.S).bytes;
    if (implicit_ok(mode, g)) {
        const size_t alt = implicit_shape(g).bytes;
        if (alt > need || !getenv("B2_CONV_IM2COL")) need = alt > need ? alt : need;
    }
    *bytes = need;
    return B2_OK;
}

extern "C" int b2_conv_fprop_f32(const float* I, const float* F, float* O, const b2_conv_dims* d,
                                 void* scratch, size_t scratch_bytes, int32_t* status,
                                 void* stream) {
    return run_fprop<float, MODE_F32X3>(I, F, O, d, nullptr, 0, 0, 0, nullptr, scratch,
                                        scratch_bytes, nullptr, status, 0, (cudaStream_t)stream);
}

extern "C" int b2_conv_fprop_flex16(const int16_t* I, const int16_t* F, int16_t* O,
                                    const b2_conv_dims* d, const b2_flex_scale* table,
                                    int32_t slotI, int32_t slotF, int32_t slotO, int32_t* stats,
                                    void* scratch, size_t scratch_bytes, uint64_t* probe_out,
                                    int32_t* status, int32_t probe, void* stream) {
    B2_REQUIRE(table && slotI >= 0 && slotF >= 0 && slotO >= 0, "flex conv needs the scale table");
    B2_REQUIRE(probe ? probe_out != nullptr : stats != nullptr, "missing statistics destination");
    return run_fprop<short, MODE_FLEX16>(I, F, O, d, table, slotI, slotF, slotO, stats, scratch,
                                         scratch_bytes, (unsigned long long*)probe_out, status,
                                         probe ? 1 : 0, (cudaStream_t)stream);
}

extern "C" int b2_conv_planes_info(const b2_conv_dims* d, int32_t pass, int32_t* supported,
                                   size_t* act_plane_bytes, size_t* filter_planes_bytes) {
    ConvGeom f, g;
    int rc = geom_from(d, &f);
    if (rc) return rc;
    B2_REQUIRE(supported && act_plane_bytes && filter_planes_bytes, "null argument");
    *supported = pass_geom(f, pass, &g) ? 1 : 0;
    *act_plane_bytes = 0;
    *filter_planes_bytes = 0;
    if (*supported) {
        const ImplicitShape s = implicit_shape(g);
        *act_plane_bytes = s.act_plane;
        *filter_planes_bytes = s.filt_bytes;
    }
    return B2_OK;
}

extern "C" int b2_conv_split_activations(const int16_t* X, const b2_conv_dims* d, int32_t pass,
                                         void* planes, void* stream) {
    ConvGeom f, g;
    int rc = geom_from(d, &f);
    if (rc) return rc;
    B2_REQUIRE(X && planes && pass_geom(f, pass, &g), "planes are not available for this convolution");
    return implicit_split_activations<short, MODE_FLEX16>(X, g, implicit_shape(g), planes,
                                                          (cudaStream_t)stream);
}

extern "C" int b2_conv_filter_planes(const int16_t* F, const b2_conv_dims* d, int32_t pass,
                                     void* planes, void* stream) {
    ConvGeom f, g;
    int rc = geom_from(d, &f);
    if (rc) return rc;
    B2_REQUIRE(F && planes && pass_geom(f, pass, &g), "planes are not available for this convolution");
    return implicit_filter_planes<short, MODE_FLEX16>(F, g, implicit_shape(g), planes,
                                                      (cudaStream_t)stream, pass);
}

extern "C" int b2_conv_flex16_planes(int32_t pass, const void* act_planes,
                                     const void* filter_planes, int16_t* out,
                                     const b2_conv_dims* d, const b2_flex_scale* table,
                                     int32_t slotX, int32_t slotF, int32_t slotOut, int32_t* stats,
                                     uint64_t* probe_out, int32_t* status, int32_t probe,
                                     void* stream) {
    ConvGeom f, g;
    int rc = geom_from(d, &f);
    if (rc) return rc;
    B2_REQUIRE(act_planes && filter_planes && out && pass_geom(f, pass, &g),
               "planes are not available for this convolution");
    B2_REQUIRE(table && slotX >= 0 && slotF >= 0 && slotOut >= 0, "flex conv needs the scale table");
    B2_REQUIRE(probe ? probe_out != nullptr : stats != nullptr, "missing statistics destination");
    return implicit_tiles(act_planes, filter_planes, out, g, implicit_shape(g), table, slotX, slotF,
                          slotOut, stats, (unsigned long long*)probe_out, status, probe ? 1 : 0,
                          (cudaStream_t)stream);
}

extern "C" int b2_conv_flex16_planes_fused(int32_t pass, const void* act_planes,
                                           const void* filter_planes, int16_t* out,
                                           const b2_conv_dims* d, const b2_flex_scale* table,
                                           int32_t slotX, int32_t slotF, int32_t slotOut,
                                           const b2_conv_epilogue* epilogue, int32_t* stats,
                                           uint64_t* probe_out, int32_t* status, int32_t probe,
                                           void* stream) {
    ConvGeom f, g;
    int rc = geom_from(d, &f);
    if (rc) return rc;
    B2_REQUIRE(act_planes && filter_planes && epilogue && pass_geom(f, pass, &g),
               "planes are not available for this convolution");
    B2_REQUIRE(out || !epilogue->write_int16, "missing output tensor");
    B2_REQUIRE(table && slotX >= 0 && slotF >= 0 && slotOut >= 0, "flex conv needs the scale table");
    B2_REQUIRE(probe ? probe_out != nullptr : stats != nullptr, "missing statistics destination");
    return implicit_tiles(act_planes, filter_planes, out, g, implicit_shape(g), table, slotX, slotF,
                          slotOut, stats, (unsigned long long*)probe_out, status, probe ? 1 : 0,
                          (cudaStream_t)stream, epilogue);
}

extern "C" int b2_conv_bprop_scratch_bytes(int32_t flex, const b2_conv_dims* d, size_t* bytes) {
    ConvGeom g;
    int rc = geom_from(d, &g);
    if (rc) return rc;
    B2_REQUIRE(bytes, "null argument");
    size_t need = bprop_shape(flex ? MODE_FLEX16 : MODE_F32X3, g).bytes;
    ConvGeom gb;
    if (flex && pass_geom(g, 1, &gb)) {
        const size_t alt = implicit_shape(gb).bytes;
        if (alt > need) need = alt;
    }
    *bytes = need;
    return B2_OK;
}

extern "C" int b2_conv_bprop_f32(const float* E, const float* F, float* GI, const b2_conv_dims* d,
                                 void* scratch, size_t scratch_bytes, int32_t* status,
                                 void* stream) {
    return run_bprop<float, MODE_F32X3>(E, F, GI, d, nullptr, 0, 0, 0, nullptr, scratch,
                                        scratch_bytes, nullptr, status, 0, (cudaStream_t)stream);
}

extern "C" int b2_conv_bprop_flex16(const int16_t* E, const int16_t* F, int16_t* GI,
                                    const b2_conv_dims* d, const b2_flex_scale* table,
                                    int32_t slotE, int32_t slotF, int32_t slotGI, int32_t* stats,
                                    void* scratch, size_t scratch_bytes, uint64_t* probe_out,
                                    int32_t* status, int32_t probe, void* stream) {
    B2_REQUIRE(table && slotE >= 0 && slotF >= 0 && slotGI >= 0, "flex conv needs the scale table");
    B2_REQUIRE(probe ? probe_out != nullptr : stats != nullptr, "missing statistics destination");
    return run_bprop<short, MODE_FLEX16>(E, F, GI, d, table, slotE, slotF, slotGI, stats, scratch,
                                         scratch_bytes, (unsigned long long*)probe_out, status,
                                         probe ? 1 : 0, (cudaStream_t)stream);
}

extern "C" int b2_conv_update_scratch_bytes(int32_t flex, const b2_conv_dims* d, size_t* bytes) {
    ConvGeom g;
    int rc = geom_from(d, &g);
    if (rc) return rc;
    B2_REQUIRE(bytes, "null argument");
    const UpdShape u = update_implicit_shape(flex ? MODE_FLEX16 : MODE_F32X3, g);
    *bytes = u.ok ? u.bytes : update_shape(flex ? MODE_FLEX16 : MODE_F32X3, g).bytes;
    return B2_OK;
}

extern "C" int b2_conv_update_f32(const float* I, const float* E, float* U, const b2_conv_dims* d,
                                  void* scratch, size_t scratch_bytes, int32_t* status,
                                  void* stream) {
    return run_update<float, MODE_F32X3>(I, E, U, d, nullptr, 0, 0, 0, nullptr, scratch,
                                         scratch_bytes, nullptr, status, 0, (cudaStream_t)stream);
}

extern "C" int b2_conv_update_flex16(const int16_t* I, const int16_t* E, int16_t* U,
                                     const b2_conv_dims* d, const b2_flex_scale* table,
                                     int32_t slotI, int32_t slotE, int32_t slotU, int32_t* stats,
                                     void* scratch, size_t scratch_bytes, uint64_t* probe_out,
                                     int32_t* status, int32_t probe, void* stream) {
    B2_REQUIRE(table && slotI >= 0 && slotE >= 0 && slotU >= 0, "flex conv needs the scale table");
    B2_REQUIRE(probe ? probe_out != nullptr : stats != nullptr, "missing statistics destination");
    return run_update<short, MODE_FLEX16>(I, E, U, d, table, slotI, slotE, slotU, stats, scratch,
                                          scratch_bytes, (unsigned long long*)probe_out, status,
                                          probe ? 1 : 0, (cudaStream_t)stream);
}

// Gradient of pooling with respect to its input, gathered per input element (consecutive threads =
// consecutive images): the windows (p, q) that contain (h, w) are visited in increasing (p, q) --
// the order in which the reference's loop adds them (ngraph/transformers/cpu/cpuengine.py:316-336).
// avg: E / (elements of the window inside the image); max: E where (h, w) is the FIRST maximum of
// the window in row-major order (np.argmax).  flex16: fp32 arithmetic on scale_E * mantissa, one
// quantisation with the result's exponent; probe: the bit pattern of max |fp32 result|.
template <typename T, bool MAX>
__global__ void __launch_bounds__(256)
pool_bprop_kernel(const T* __restrict__ E, const T* __restrict__ I, T* __restrict__ GI, int C, int H,
                  int W, int N, int P, int Q, int R, int S, int pad_h, int pad_w, int str_h,
                  int str_w, const b2_flex_scale* __restrict__ table, int slotE, int slotG,
                  int* stats, unsigned long long* probe_out, int probe) {
    const long long total = (long long)C * H * W * N;
    const bool flex = sizeof(T) == 2;
    const float sE = flex ? table[slotE].scale : 1.0f;
    const float qG = flex && !probe ? table[slotG].inv_scale : 1.0f;
    float fstat = 0.0f, fmax = 0.0f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int n = (int)(i % N);
        long long t = i / N;
        const int w = (int)(t % W); t /= W;
        const int h = (int)(t % H);
        const int c = (int)(t / H);
        // windows with p*str - pad <= h < p*str - pad + R
        int p0 = h + pad_h - R + 1;
        p0 = p0 <= 0 ? 0 : (p0 + str_h - 1) / str_h;
        int p1 = (h + pad_h) / str_h;
        if (p1 > P - 1) p1 = P - 1;
        int q0 = w + pad_w - S + 1;
        q0 = q0 <= 0 ? 0 : (q0 + str_w - 1) / str_w;
        int q1 = (w + pad_w) / str_w;
        if (q1 > Q - 1) q1 = Q - 1;
        float acc = 0.0f;
        for (int p = p0; p <= p1; ++p)
            for (int q = q0; q <= q1; ++q) {
                const int h0 = max(p * str_h - pad_h, 0), h1 = min(p * str_h - pad_h + R, H);
                const int w0 = max(q * str_w - pad_w, 0), w1 = min(q * str_w - pad_w + S, W);
                const float e = sE * (float)E[(((long long)c * P + p) * Q + q) * N + n];
                if (MAX) {
                    // is (h, w) the first maximum of the window?
                    const T mine = I[i];
                    bool first = true;
                    for (int hh = h0; hh < h1 && first; ++hh)
                        for (int ww = w0; ww < w1; ++ww) {
                            const T v = I[(((long long)c * H + hh) * W + ww) * N + n];
                            const bool before = hh < h || (hh == h && ww < w);
                            if (v > mine || (before && v == mine)) { first = false; break; }
                        }
                    if (first) acc += e;
                } else {
                    const int cnt = (h1 - h0) * (w1 - w0);
                    acc += e * (1.0f / (float)cnt);
                }
            }
        if (!flex) {
            GI[i] = (T)acc;
        } else if (probe) {
            fmax = fmaxf(fmax, fabsf(acc));
        } else {
            float v = acc * qG;
            v = (v != v) ? 0.0f : v;
            v = fminf(fmaxf(v, -32768.0f), 32767.0f);
            fstat = fmaxf(fstat, fabsf(v));
            GI[i] = (T)(__float_as_int(v + 12582912.0f) - 0x4B400000);
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
            if ((threadIdx.x & 31) == 0 && stat) atomicMax(stats + slotG, stat);
        }
    }
}

namespace {
int run_pool(bool is_max, const void* I, void* O, int32_t flex, int32_t C, int32_t H, int32_t W,
             int32_t N, int32_t P, int32_t Q, int32_t R, int32_t S, int32_t pad_h, int32_t pad_w,
             int32_t str_h, int32_t str_w, int32_t* stats_slot, void* stream) {
    B2_REQUIRE(I && O && C > 0 && H > 0 && W > 0 && N > 0 && P > 0 && Q > 0 && R > 0 && S > 0 &&
               str_h > 0 && str_w > 0, "bad pooling argument");
    const long long total = (long long)C * P * Q * N;
    long long blocks = (total + 31) / 32;            // 32 results per block
    if (blocks > 148 * 16) blocks = 148 * 16;
    cudaStream_t st = (cudaStream_t)stream;
#define B2_POOL_LAUNCH(T, MAXV, STATS)                                                            \
    pool_kernel<T, MAXV><<<(unsigned)blocks, 256, 0, st>>>((const T*)I, (T*)O, C, H, W, N, P, Q, R, \
                                                          S, pad_h, pad_w, str_h, str_w, STATS)
    if (flex) {
        if (is_max) B2_POOL_LAUNCH(short, true, stats_slot);
        else B2_POOL_LAUNCH(short, false, stats_slot);
    } else {
        if (is_max) B2_POOL_LAUNCH(float, true, nullptr);
        else B2_POOL_LAUNCH(float, false, nullptr);
    }
#undef B2_POOL_LAUNCH
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}
}  // namespace

extern "C" int b2_pool_avg_fprop(const void* I, void* O, int32_t flex, int32_t C, int32_t H,
                                 int32_t W, int32_t N, int32_t P, int32_t Q, int32_t R, int32_t S,
                                 int32_t pad_h, int32_t pad_w, int32_t str_h, int32_t str_w,
                                 int32_t* stats_slot, void* stream) {
    return run_pool(false, I, O, flex, C, H, W, N, P, Q, R, S, pad_h, pad_w, str_h, str_w,
                    stats_slot, stream);
}

extern "C" int b2_pool_max_fprop(const void* I, void* O, int32_t flex, int32_t C, int32_t H,
                                 int32_t W, int32_t N, int32_t P, int32_t Q, int32_t R, int32_t S,
                                 int32_t pad_h, int32_t pad_w, int32_t str_h, int32_t str_w,
                                 int32_t* stats_slot, void* stream) {
    return run_pool(true, I, O, flex, C, H, W, N, P, Q, R, S, pad_h, pad_w, str_h, str_w,
                    stats_slot, stream);
}

extern "C" int b2_pool_bprop(const void* E, const void* I, void* GI, int32_t flex, int32_t is_max,
                             int32_t C, int32_t H, int32_t W, int32_t N, int32_t P, int32_t Q,
                             int32_t R, int32_t S, int32_t pad_h, int32_t pad_w, int32_t str_h,
                             int32_t str_w, const b2_flex_scale* table, int32_t slotE,
                             int32_t slotGI, int32_t* stats, uint64_t* probe_out, int32_t probe,
                             void* stream) {
    B2_REQUIRE(E && GI && C > 0 && H > 0 && W > 0 && N > 0 && P > 0 && Q > 0 && R > 0 && S > 0 &&
               str_h > 0 && str_w > 0, "bad pooling argument");
    B2_REQUIRE(!is_max || I, "the gradient of max pooling needs the pooled tensor");
    if (flex) {
        B2_REQUIRE(table && slotE >= 0 && slotGI >= 0, "flex pooling gradient needs the scale table");
        B2_REQUIRE(probe ? probe_out != nullptr : stats != nullptr, "missing statistics destination");
    }
    const long long total = (long long)C * H * W * N;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    cudaStream_t st = (cudaStream_t)stream;
    unsigned long long* po = (unsigned long long*)probe_out;
#define B2_PB_LAUNCH(T, MAXV)                                                                       \
    pool_bprop_kernel<T, MAXV><<<(unsigned)blocks, 256, 0, st>>>(                                  \
        (const T*)E, (const T*)I, (T*)GI, C, H, W, N, P, Q, R, S, pad_h, pad_w, str_h, str_w, table, \
        slotE, slotGI, stats, po, probe ? 1 : 0)
    if (flex) {
        if (is_max) B2_PB_LAUNCH(short, true);
        else B2_PB_LAUNCH(short, false);
    } else {
        if (is_max) B2_PB_LAUNCH(float, true);
        else B2_PB_LAUNCH(float, false);
    }
#undef B2_PB_LAUNCH
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

// ---- lookup table (embedding) ----------------------------------------------------------------
namespace {
// index held as fp32, or as a flex16 mantissa with its tensor's scale
template <typename T>
__device__ __forceinline__ int lut_index(const T* idx, int i, float s) {
    return (int)rintf(s * (float)idx[i]);
}

// out = lut.take(idx, axis): lut_axis 0: lut [V][F], out [n][F]; lut_axis 1: lut [F][V], out [F][n]
template <typename T>
__global__ void __launch_bounds__(256)
lut_fprop_kernel(const T* __restrict__ lut, const T* __restrict__ idx, T* __restrict__ out,
                 int lut_axis, int V, int F, int n, const b2_flex_scale* __restrict__ table,
                 int slotI) {
    const float s_idx = table ? table[slotI].scale : 1.0f;
    const long long total = (long long)n * F;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total;
         e += (long long)gridDim.x * blockDim.x) {
        const int i = lut_axis == 0 ? (int)(e / F) : (int)(e % n);
        const int f = lut_axis == 0 ? (int)(e % F) : (int)(e / n);
        const int w = lut_index(idx, i, s_idx);
        T v = (T)0;
        if (w >= 0 && w < V) v = lut_axis == 0 ? lut[(long long)w * F + f] : lut[(long long)f * V + w];
        out[e] = v;
    }
}

// dW[w] = sum of the rows of delta whose index is w, rows added in increasing position (the order
// of np.sum over the group, ngraph/transformers/cpu/cpuengine.py:425-435); pad_idx stays zero.
// One thread per element of dW; the indices are staged through shared memory 256 at a time.
template <typename T>
__global__ void __launch_bounds__(256)
lut_update_kernel(const T* __restrict__ delta, const T* __restrict__ idx, T* __restrict__ dW,
                  int lut_axis, int V, int F, int n, int pad_idx, const b2_flex_scale* table,
                  int slotD, int slotI, int slotW, int* stats, unsigned long long* probe_out,
                  int probe) {
    __shared__ int widx[256];
    const bool flex = sizeof(T) == 2;
    const float sD = flex ? table[slotD].scale : 1.0f;
    const float sI = flex ? table[slotI].scale : 1.0f;
    const float qW = flex && !probe ? table[slotW].inv_scale : 1.0f;
    const long long total = (long long)V * F;
    const long long rounds = (total + (long long)gridDim.x * 256 - 1) / ((long long)gridDim.x * 256);
    float fstat = 0.0f, fmax = 0.0f;
    for (long long r = 0; r < rounds; ++r) {
        const long long e = (r * gridDim.x + blockIdx.x) * 256 + threadIdx.x;
        const bool live = e < total;
        const int w = live ? (lut_axis == 0 ? (int)(e / F) : (int)(e % V)) : -1;
        const int f = live ? (lut_axis == 0 ? (int)(e % F) : (int)(e / V)) : 0;
        float acc = 0.0f;
        for (int base = 0; base < n; base += 256) {
            __syncthreads();
            if (base + (int)threadIdx.x < n) widx[threadIdx.x] = lut_index(idx, base + threadIdx.x, sI);
            __syncthreads();
            const int m = min(256, n - base);
            if (live && w != pad_idx)
                for (int j = 0; j < m; ++j)
                    if (widx[j] == w) {
                        const int i = base + j;
                        acc += sD * (float)(lut_axis == 0 ? delta[(long long)i * F + f]
                                                          : delta[(long long)f * n + i]);
                    }
        }
        if (!live) continue;
        if (!flex) {
            dW[e] = (T)acc;
        } else if (probe) {
            fmax = fmaxf(fmax, fabsf(acc));
        } else {
            float v = acc * qW;
            v = (v != v) ? 0.0f : v;
            v = fminf(fmaxf(v, -32768.0f), 32767.0f);
            fstat = fmaxf(fstat, fabsf(v));
            dW[e] = (T)(__float_as_int(v + 12582912.0f) - 0x4B400000);
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
            if ((threadIdx.x & 31) == 0 && stat) atomicMax(stats + slotW, stat);
        }
    }
}
}  // namespace

extern "C" int b2_lut_fprop(const void* lut, const void* idx, void* out, int32_t flex,
                            int32_t lut_axis, int32_t V, int32_t F, int32_t n_idx,
                            const b2_flex_scale* table, int32_t slot_idx, void* stream) {
    B2_REQUIRE(lut && idx && out && V > 0 && F > 0 && n_idx > 0 && (lut_axis == 0 || lut_axis == 1),
               "bad lookup-table argument");
    B2_REQUIRE(!flex || (table && slot_idx >= 0), "flex lookup needs the scale table");
    long long blocks = ((long long)n_idx * F + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    cudaStream_t st = (cudaStream_t)stream;
    if (flex)
        lut_fprop_kernel<short><<<(unsigned)blocks, 256, 0, st>>>(
            (const short*)lut, (const short*)idx, (short*)out, lut_axis, V, F, n_idx, table, slot_idx);
    else
        lut_fprop_kernel<float><<<(unsigned)blocks, 256, 0, st>>>(
            (const float*)lut, (const float*)idx, (float*)out, lut_axis, V, F, n_idx, nullptr, 0);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}

extern "C" int b2_lut_update(const void* delta, const void* idx, void* dW, int32_t flex,
                             int32_t lut_axis, int32_t V, int32_t F, int32_t n_idx, int32_t pad_idx,
                             const b2_flex_scale* table, int32_t slot_delta, int32_t slot_idx,
                             int32_t slot_dW, int32_t* stats, uint64_t* probe_out, int32_t probe,
                             void* stream) {
    B2_REQUIRE(delta && idx && dW && V > 0 && F > 0 && n_idx > 0 && (lut_axis == 0 || lut_axis == 1),
               "bad lookup-table argument");
    if (flex) {
        B2_REQUIRE(table && slot_delta >= 0 && slot_idx >= 0 && slot_dW >= 0,
                   "flex lookup update needs the scale table");
        B2_REQUIRE(probe ? probe_out != nullptr : stats != nullptr, "missing statistics destination");
    }
    long long blocks = ((long long)V * F + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    cudaStream_t st = (cudaStream_t)stream;
    unsigned long long* po = (unsigned long long*)probe_out;
    if (flex)
        lut_update_kernel<short><<<(unsigned)blocks, 256, 0, st>>>(
            (const short*)delta, (const short*)idx, (short*)dW, lut_axis, V, F, n_idx, pad_idx, table,
            slot_delta, slot_idx, slot_dW, stats, po, probe ? 1 : 0);
    else
        lut_update_kernel<float><<<(unsigned)blocks, 256, 0, st>>>(
            (const float*)delta, (const float*)idx, (float*)dW, lut_axis, V, F, n_idx, pad_idx, nullptr,
            0, 0, 0, nullptr, nullptr, 0);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}
