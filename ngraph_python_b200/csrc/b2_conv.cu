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
#include "b2_gemm_impl.cuh"

namespace {

struct ConvGeom {
    int C, H, W, N, K, R, S, P, Q, pad_h, pad_w, str_h, str_w, dil_h, dil_w;
};

int geom_from(const b2_conv_dims* d, ConvGeom* g) {
    B2_REQUIRE(d, "null dims");
    B2_REQUIRE(d->D == 1 && d->T == 1 && d->M == 1 && d->pad_d == 0 && d->str_d == 1,
               "only 2-d convolutions (D = T = M = 1) are supported");
    B2_REQUIRE(d->C > 0 && d->H > 0 && d->W > 0 && d->N > 0 && d->K > 0 && d->R > 0 && d->S > 0 &&
               d->P > 0 && d->Q > 0 && d->str_h > 0 && d->str_w > 0 && d->dil_h > 0 && d->dil_w > 0,
               "bad convolution dimensions");
    g->C = d->C; g->H = d->H; g->W = d->W; g->N = d->N; g->K = d->K; g->R = d->R; g->S = d->S;
    g->P = d->P; g->Q = d->Q; g->pad_h = d->pad_h; g->pad_w = d->pad_w; g->str_h = d->str_h;
    g->str_w = d->str_w; g->dil_h = d->dil_h; g->dil_w = d->dil_w;
    return B2_OK;
}

// Gather + split.  Rows of the planes: r = (p*Q + q)*N + n ; columns: kidx = (c*R + r_)*S + s_.
// A block owns 32 consecutive rows (32 images of one output pixel when N is a multiple of 32) and
// walks the columns in chunks of 128 bytes of plane row.  Per chunk the tap decomposition of each
// column is computed once into shared memory; loads run along n (contiguous in the input), the
// write phase emits one 16-byte vector per thread and plane (contiguous along the plane row).
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
im2col_planes_kernel(const T* __restrict__ I, ConvGeom g, int rows, int kg, int rows_p, int kp,
                     void* __restrict__ plane0, void* __restrict__ plane1) {
    constexpr int CK = MODE == MODE_FLEX16 ? 128 : 32;
    __shared__ T tile[CK][33];
    __shared__ int tab_c[CK], tab_h[CK], tab_w[CK];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int r0 = blockIdx.x * 32;
    const int r = r0 + tx;
    const bool rvalid = r < rows;
    int n = 0, h0 = 0, w0 = 0;
    if (rvalid) {
        n = r % g.N;
        const int pq = r / g.N;
        const int q = pq % g.Q, pp = pq / g.Q;
        h0 = pp * g.str_h - g.pad_h;
        w0 = q * g.str_w - g.pad_w;
    }
    const int RS = g.R * g.S;
    const int wr = threadIdx.x >> 3, vec = threadIdx.x & 7;
    const int orow = r0 + wr;
    for (int kc = 0; kc < kp; kc += CK) {
        __syncthreads();
        if (threadIdx.x < CK) {
            const int kidx = kc + threadIdx.x;
            if (kidx < kg) {
                const int c = kidx / RS, rs = kidx - c * RS;
                const int fr = rs / g.S, fs = rs - fr * g.S;
                tab_c[threadIdx.x] = c * g.H * g.W * g.N;
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
                const int h = h0 + tab_h[i], w = w0 + tab_w[i];
                if (h >= 0 && h < g.H && w >= 0 && w < g.W)
                    v = I[(long long)tc + ((long long)h * g.W + w) * g.N + n];
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

template <typename T, int MODE>
int run_fprop(const T* I, const T* F, void* O, const b2_conv_dims* d, const b2_flex_scale* table,
              int slotI, int slotF, int slotO, int* stats, void* scratch, size_t scratch_bytes,
              unsigned long long* probe_out, int* status, int probe, cudaStream_t st) {
    ConvGeom g;
    int rc = geom_from(d, &g);
    if (rc) return rc;
    B2_REQUIRE(I && F && O, "null tensor");
    const long long rows_ll = (long long)g.P * g.Q * g.N;
    B2_REQUIRE(rows_ll < (1LL << 31) - 256, "too many output positions");
    const int rows = (int)rows_ll, kg = g.C * g.R * g.S;
    if (MODE == MODE_FLEX16) B2_REQUIRE(kg <= 32768, "flex16 convolution needs C*R*S <= 32768");
    const Shapes s = shapes_for(MODE, rows, g.K, kg);
    B2_REQUIRE(scratch && scratch_bytes >= s.bytes && ((uintptr_t)scratch & 1023) == 0,
               "convolution needs %zu bytes of 1024-byte aligned scratch, got %zu", s.bytes,
               scratch_bytes);
    unsigned char* base = (unsigned char*)scratch;
    const size_t a_plane = (size_t)s.Mp * s.Kp * s.esize, b_plane = (size_t)s.Np * s.Kp * s.esize;
    {
        B2_REQUIRE((long long)g.C * g.H * g.W * g.N < (1LL << 31), "input tensor too large");
        im2col_planes_kernel<T, MODE><<<s.Mp / 32, 256, 0, st>>>(I, g, rows, kg, s.Mp, s.Kp, base,
                                                         base + a_plane);
        // filters: element (n = k_out, k = kidx) = F[kidx * K + k_out]
        dim3 gb((s.Kp + 31) / 32, (s.Np + 31) / 32);
        split_planes_kernel<T, MODE><<<gb, 256, 0, st>>>(F, 1, g.K, g.K, kg, s.Np, s.Kp,
                                                        base + 2 * a_plane,
                                                        base + 2 * a_plane + b_plane);
        B2_CUDA(cudaGetLastError());
    }
    GemmParams p;
    p.M = rows; p.N = g.K; p.num_kb = 0;
    p.ldc = rows; p.C = O; p.table = table; p.slotA = slotI; p.slotB = slotF; p.slotC = slotO;
    p.stats = stats; p.probe_out = probe_out; p.status = status; p.probe = probe;
    p.c_colmajor = 1;
    return launch_on_planes<MODE>(base, s, p, st);
}

// ---- average pooling over H, W windows (C and D windows of 1) ------------------------------------
// out[c,p,q,n] = mean over the part of the window inside the image (the numpy reference takes
// np.mean of the clipped slice, ngraph/transformers/cpu/cpuengine.py:296-305).  flex16: the output
// shares the input's exponent (ngraph/transformers/passes/flexpass.py:40-48), so mantissas are
// averaged and rounded to nearest even.
template <typename T>
__global__ void __launch_bounds__(256)
pool_avg_kernel(const T* __restrict__ I, T* __restrict__ O, int C, int H, int W, int N, int P, int Q,
                int R, int S, int pad_h, int pad_w, int str_h, int str_w, int* stats) {
    const long long total = (long long)C * P * Q * N;
    int stat = 0;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int n = (int)(i % N);
        long long t = i / N;
        const int q = (int)(t % Q); t /= Q;
        const int p = (int)(t % P);
        const int c = (int)(t / P);
        const int h0 = max(p * str_h - pad_h, 0), h1 = min(p * str_h - pad_h + R, H);
        const int w0 = max(q * str_w - pad_w, 0), w1 = min(q * str_w - pad_w + S, W);
        float acc = 0.0f;
        for (int h = h0; h < h1; ++h)
            for (int w = w0; w < w1; ++w)
                acc += (float)I[(((long long)c * H + h) * W + w) * N + n];
        const int cnt = max((h1 - h0) * (w1 - w0), 1);
        const float mean = acc / (float)cnt;
        if (sizeof(T) == 2) {
            const int m = __float2int_rn(mean);
            stat = max(stat, m < 0 ? -m : m);
            O[i] = (T)m;
        } else {
            O[i] = (T)mean;
        }
    }
    if (sizeof(T) == 2 && stats) {
        for (int o = 16; o > 0; o >>= 1) stat = max(stat, __shfl_xor_sync(0xffffffffu, stat, o));
        if ((threadIdx.x & 31) == 0 && stat) atomicMax(stats, stat);
    }
}

}  // namespace

extern "C" int b2_conv_fprop_scratch_bytes(int32_t flex, const b2_conv_dims* d, size_t* bytes) {
    ConvGeom g;
    int rc = geom_from(d, &g);
    if (rc) return rc;
    B2_REQUIRE(bytes, "null argument");
    *bytes = shapes_for(flex ? MODE_FLEX16 : MODE_F32X3, g.P * g.Q * g.N, g.K, g.C * g.R * g.S).bytes;
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

extern "C" int b2_pool_avg_fprop(const void* I, void* O, int32_t flex, int32_t C, int32_t H,
                                 int32_t W, int32_t N, int32_t P, int32_t Q, int32_t R, int32_t S,
                                 int32_t pad_h, int32_t pad_w, int32_t str_h, int32_t str_w,
                                 int32_t* stats_slot, void* stream) {
    B2_REQUIRE(I && O && C > 0 && H > 0 && W > 0 && N > 0 && P > 0 && Q > 0 && R > 0 && S > 0 &&
               str_h > 0 && str_w > 0, "bad pooling argument");
    const long long total = (long long)C * P * Q * N;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    cudaStream_t st = (cudaStream_t)stream;
    if (flex)
        pool_avg_kernel<short><<<(unsigned)blocks, 256, 0, st>>>((const short*)I, (short*)O, C, H, W,
                                                                N, P, Q, R, S, pad_h, pad_w, str_h,
                                                                str_w, stats_slot);
    else
        pool_avg_kernel<float><<<(unsigned)blocks, 256, 0, st>>>((const float*)I, (float*)O, C, H, W,
                                                                N, P, Q, R, S, pad_h, pad_w, str_h,
                                                                str_w, nullptr);
    B2_CUDA(cudaGetLastError());
    return B2_OK;
}
