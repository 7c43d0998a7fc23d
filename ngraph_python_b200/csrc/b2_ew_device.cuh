// Device-side helpers shared by every generated fused elementwise/reduction kernel.
//
// This text is compiled twice: by nvcc as part of the library (so that it is syntax-checked and
// its register use shows up in -Xptxas -v), and at run time by NVRTC, prepended to the kernel
// body that b2_ew_codegen.cu emits for one fused program.  It must therefore not include any
// header: only CUDA built-ins.
//
// The semantics of each helper follow the CUDA-C templates the reference generates
// (ngraph/transformers/gpu/float_ew2.py:31-98, 261-281): fp32 arithmetic, CUDA libm, flex16
// stores through cvt.rni.s16.f32 (round to nearest even, saturating), maxabs of the stored
// mantissas as s32.
#ifndef B2_EW_DEVICE_CUH
#define B2_EW_DEVICE_CUH

#define B2_FLT_MAX 3.402823466e+38f
#ifndef B200NG_H
#define B2_EW_MAX_IN 12
#define B2_EW_MAX_OUT 6
#define B2_EW_MAX_CONST 16
#endif

typedef long long b2_i64;

// One row per flex tensor: what a reader multiplies by and what a writer multiplies by.
// (The library's public header declares the same struct; under NVRTC only this one exists.)
#ifndef B200NG_H
struct b2_flex_scale {
    float scale;      // 2^-dec
    float inv_scale;  // 2^dec
};
#endif

// Launch-time arguments of a generated kernel (passed by value).
struct b2_ew_args {
    b2_i64 A, B, C;                       // iteration space, C innermost
    const void* in[B2_EW_MAX_IN];
    b2_i64 in_sa[B2_EW_MAX_IN], in_sb[B2_EW_MAX_IN], in_sc[B2_EW_MAX_IN];
    int in_slot[B2_EW_MAX_IN];            // row of the flex table, -1 for fp32
    void* out[B2_EW_MAX_OUT];             // elementwise outputs first, then reduction outputs
    b2_i64 out_sa[B2_EW_MAX_OUT], out_sb[B2_EW_MAX_OUT], out_sc[B2_EW_MAX_OUT];
    int out_slot[B2_EW_MAX_OUT];
    b2_i64 out_plane[B2_EW_MAX_OUT];      // byte-plane results: offset of the low plane from the high plane
    float consts[B2_EW_MAX_CONST];
    const b2_flex_scale* flex_table;      // device table, indexed by slot
    int* flex_stats;                      // device s32 per slot: max |mantissa| written
    float* scratch;                       // split reductions: [nsplit][rows][n_red] partials
    int* status;                          // optional: set to 1 if a bounded wait ran out
    int nsplit;
    unsigned fresh_mask;                  // probe launches: results whose exponent is not chosen yet
};

// fp32 -> int16 with the semantics of cvt.rni.s16.f32 (round to nearest even, saturate to
// [-32768, 32767], NaN -> 0), written with full-rate instructions: clamp, then add 1.5 * 2^23 so
// that the FADD itself rounds to an integer held in the low mantissa bits.  (The cvt instruction
// issues at a quarter of the FP32 rate, which makes a flex kernel conversion-bound.)
// `stat` follows max |clamped value|; rounding is monotonic and symmetric, so rounding that
// maximum once at the end gives max |mantissa| (with -32768 counting as 32768).
__device__ __forceinline__ int b2_f32_to_i16(float v, float& stat) {
    v = (v != v) ? 0.0f : v;
    v = fminf(fmaxf(v, -32768.0f), 32767.0f);
    stat = fmaxf(stat, fabsf(v));
    return __float_as_int(v + 12582912.0f) - 0x4B400000;
}
__device__ __forceinline__ int b2_stat_to_int(float stat) { return (int)rintf(stat); }
// the value a flex16 tensor holds after v was stored into it with 1/step q and step s
__device__ __forceinline__ float b2_requant(float v, float q, float s) {
    float unused = 0.0f;
    return (float)b2_f32_to_i16(v * q, unused) * s;
}

// two int16 mantissas packed in one 32-bit word -> two fp32 values times `scale`, exact:
// (m ^ 0x8000) placed under the exponent of 2^23 is the float 2^23 + m + 32768.
__device__ __forceinline__ void b2_i16x2_to_f32(unsigned w, float scale, float bias, float& lo,
                                                float& hi) {
    w ^= 0x80008000u;
    const float flo = __int_as_float(__byte_perm(w, 0x4B000000u, 0x7610));
    const float fhi = __int_as_float(__byte_perm(w, 0x4B000000u, 0x7632));
    lo = __fmaf_rn(flo, scale, bias);   // exact: power-of-two scale, |m| < 2^16
    hi = __fmaf_rn(fhi, scale, bias);
}
__device__ __forceinline__ float b2_i16_bias(float scale) { return -8421376.0f * scale; }

__device__ __forceinline__ int b2_absmax(int cur, int v) {
    int a = v < 0 ? -v : v;
    return a > cur ? a : cur;
}

// |x| as an order-preserving integer, NaN counted as 0 (used when a first call measures the
// unsaturated range of an output before any exponent exists).
__device__ __forceinline__ int b2_absbits(float v) {
    float a = fabsf(v);
    return (a != a) ? 0 : __float_as_int(a);
}

// ---- vector loads: raw registers first, conversion later (so the next step's loads can be in
// flight while this step computes) ---------------------------------------------------------------
struct b2_f8 { float4 a, b; };

__device__ __forceinline__ void b2_ldraw(const float* p, float4& w) {
    w = __ldcs(reinterpret_cast<const float4*>(p));
}
__device__ __forceinline__ void b2_ldraw(const float* p, b2_f8& w) {
    w.a = __ldcs(reinterpret_cast<const float4*>(p));
    w.b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
}
__device__ __forceinline__ void b2_ldraw(const short* p, int4& w) {
    w = __ldcs(reinterpret_cast<const int4*>(p));
}
__device__ __forceinline__ void b2_ldraw(const short* p, int2& w) {
    w = __ldcs(reinterpret_cast<const int2*>(p));
}
__device__ __forceinline__ void b2_cvt(const float4& w, float* v, float) {
    v[0] = w.x; v[1] = w.y; v[2] = w.z; v[3] = w.w;
}
__device__ __forceinline__ void b2_cvt(const b2_f8& w, float* v, float) {
    v[0] = w.a.x; v[1] = w.a.y; v[2] = w.a.z; v[3] = w.a.w;
    v[4] = w.b.x; v[5] = w.b.y; v[6] = w.b.z; v[7] = w.b.w;
}
// eight int16 mantissas from one 128-bit access
__device__ __forceinline__ void b2_cvt(const int4& t, float* v, float scale) {
    const float bias = b2_i16_bias(scale);
    b2_i16x2_to_f32((unsigned)t.x, scale, bias, v[0], v[1]);
    b2_i16x2_to_f32((unsigned)t.y, scale, bias, v[2], v[3]);
    b2_i16x2_to_f32((unsigned)t.z, scale, bias, v[4], v[5]);
    b2_i16x2_to_f32((unsigned)t.w, scale, bias, v[6], v[7]);
}
__device__ __forceinline__ void b2_cvt(const int2& t, float* v, float scale) {
    const float bias = b2_i16_bias(scale);
    b2_i16x2_to_f32((unsigned)t.x, scale, bias, v[0], v[1]);
    b2_i16x2_to_f32((unsigned)t.y, scale, bias, v[2], v[3]);
}
__device__ __forceinline__ void b2_st4_cs(float* p, const float* v) {
    __stcs(reinterpret_cast<float4*>(p), make_float4(v[0], v[1], v[2], v[3]));
}
// element e of a raw vector (e is a compile-time constant once the element loop is unrolled, so
// the selects fold away); conversion happens here, next to the use, to keep few values live
__device__ __forceinline__ float b2_elem(const float4& w, int e, float, float) {
    return e == 0 ? w.x : e == 1 ? w.y : e == 2 ? w.z : w.w;
}
__device__ __forceinline__ float b2_elem(const b2_f8& w, int e, float s, float b) {
    return e < 4 ? b2_elem(w.a, e, s, b) : b2_elem(w.b, e - 4, s, b);
}
__device__ __forceinline__ float b2_elem_i16(unsigned word, int half, float scale, float bias) {
    word ^= 0x80008000u;
    const unsigned bits = half ? __byte_perm(word, 0x4B000000u, 0x7632)
                               : __byte_perm(word, 0x4B000000u, 0x7610);
    return __fmaf_rn(__int_as_float(bits), scale, bias);
}
__device__ __forceinline__ float b2_elem(const int4& w, int e, float scale, float bias) {
    const int word = (e >> 1) == 0 ? w.x : (e >> 1) == 1 ? w.y : (e >> 1) == 2 ? w.z : w.w;
    return b2_elem_i16((unsigned)word, e & 1, scale, bias);
}
__device__ __forceinline__ float b2_elem(const int2& w, int e, float scale, float bias) {
    const int word = (e >> 1) == 0 ? w.x : w.y;
    return b2_elem_i16((unsigned)word, e & 1, scale, bias);
}
__device__ __forceinline__ int b2_pack_i16x2(int lo, int hi) {
    return (int)__byte_perm((unsigned)lo, (unsigned)hi, 0x5410);
}
__device__ __forceinline__ void b2_st8_i16(short* p, const int* m) {
    int4 t;
    t.x = b2_pack_i16x2(m[0], m[1]);
    t.y = b2_pack_i16x2(m[2], m[3]);
    t.z = b2_pack_i16x2(m[4], m[5]);
    t.w = b2_pack_i16x2(m[6], m[7]);
    __stcs(reinterpret_cast<int4*>(p), t);
}
// flex16 results stored as two byte planes (high bytes at p, low bytes `lo` bytes further): the
// operand format of the convolution kernels, so that no separate split pass is needed
__device__ __forceinline__ void b2_st8_planes(unsigned char* p, b2_i64 lo, const int* m) {
    uint2 h, l;
    const unsigned a = (unsigned)b2_pack_i16x2(m[0], m[1]), b = (unsigned)b2_pack_i16x2(m[2], m[3]);
    const unsigned c = (unsigned)b2_pack_i16x2(m[4], m[5]), d = (unsigned)b2_pack_i16x2(m[6], m[7]);
    h.x = __byte_perm(a, b, 0x7531); l.x = __byte_perm(a, b, 0x6420);
    h.y = __byte_perm(c, d, 0x7531); l.y = __byte_perm(c, d, 0x6420);
    __stcs(reinterpret_cast<uint2*>(p), h);
    __stcs(reinterpret_cast<uint2*>(p + lo), l);
}
__device__ __forceinline__ void b2_st4_planes(unsigned char* p, b2_i64 lo, const int* m) {
    const unsigned a = (unsigned)b2_pack_i16x2(m[0], m[1]), b = (unsigned)b2_pack_i16x2(m[2], m[3]);
    __stcs(reinterpret_cast<unsigned*>(p), __byte_perm(a, b, 0x7531));
    __stcs(reinterpret_cast<unsigned*>(p + lo), __byte_perm(a, b, 0x6420));
}
__device__ __forceinline__ void b2_st4_i16(short* p, const int* m) {
    int2 t;
    t.x = b2_pack_i16x2(m[0], m[1]);
    t.y = b2_pack_i16x2(m[2], m[3]);
    __stcs(reinterpret_cast<int2*>(p), t);
}

// ---- reductions across a warp / a CTA ---------------------------------------------------------
#ifndef B200NG_H
#define B2_RED_SUM 0
#define B2_RED_PROD 1
#define B2_RED_MAX 2
#define B2_RED_MIN 3
#define B2_RED_ARGMAX 4
#define B2_RED_ARGMIN 5
#endif

template <int OP> __device__ __forceinline__ float b2_red_init() {
    return OP == B2_RED_SUM ? 0.0f : OP == B2_RED_PROD ? 1.0f
         : (OP == B2_RED_MAX || OP == B2_RED_ARGMAX) ? -B2_FLT_MAX : B2_FLT_MAX;
}
template <int OP> __device__ __forceinline__ float b2_red_comb(float a, float b) {
    return OP == B2_RED_SUM ? a + b : OP == B2_RED_PROD ? a * b
         : OP == B2_RED_MAX ? fmaxf(a, b) : fminf(a, b);
}
// arg reductions carry (value, index); ties keep the smaller index, which is what a sequential
// strict-compare scan returns (float_ew2.py:74-75)
template <int OP> __device__ __forceinline__ void b2_arg_comb(float& v, int& i, float ov, int oi) {
    bool take = (OP == B2_RED_ARGMAX) ? (ov > v || (ov == v && oi < i))
                                      : (ov < v || (ov == v && oi < i));
    if (take) { v = ov; i = oi; }
}

template <int OP> __device__ __forceinline__ float b2_warp_reduce(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = b2_red_comb<OP>(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
template <int OP> __device__ __forceinline__ void b2_warp_reduce_arg(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, v, o);
        int oi = __shfl_xor_sync(0xffffffffu, i, o);
        b2_arg_comb<OP>(v, i, ov, oi);
    }
}
__device__ __forceinline__ int b2_warp_max_i(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        int t = __shfl_xor_sync(0xffffffffu, v, o);
        v = t > v ? t : v;
    }
    return v;
}

// CTA-wide reduce of one float; result valid in thread 0.  smem: 32 floats.
template <int OP> __device__ __forceinline__ float b2_block_reduce(float v, float* smem) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = b2_warp_reduce<OP>(v);
    __syncthreads();                       // smem may still be read from a previous call
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    if (warp == 0) {
        v = lane < nwarp ? smem[lane] : b2_red_init<OP>();
        v = b2_warp_reduce<OP>(v);
    }
    return v;
}
template <int OP>
__device__ __forceinline__ void b2_block_reduce_arg(float& v, int& i, float* smem) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    int* ismem = reinterpret_cast<int*>(smem) + 32;
    b2_warp_reduce_arg<OP>(v, i);
    __syncthreads();
    if (lane == 0) { smem[warp] = v; ismem[warp] = i; }
    __syncthreads();
    if (warp == 0) {
        if (lane < nwarp) { v = smem[lane]; i = ismem[lane]; }
        else { v = b2_red_init<OP>(); i = 0x7fffffff; }
        b2_warp_reduce_arg<OP>(v, i);
    }
}
// CTA-wide integer max followed by ONE global atomic per CTA.
__device__ __forceinline__ void b2_block_stat(int v, int* stat, int* ismem) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = b2_warp_max_i(v);
    __syncthreads();
    if (lane == 0) ismem[warp] = v;
    __syncthreads();
    if (warp == 0) {
        v = lane < nwarp ? ismem[lane] : 0;
        v = b2_warp_max_i(v);
        if (lane == 0 && v > 0) atomicMax(stat, v);
    }
}

// ---- scalar op semantics (one function per template of float_ew2.py:31-68) ----------------------
__device__ __forceinline__ float b2_op_sig(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float b2_op_safelog(float x) { return x > 0.0f ? logf(x) : -50.0f; }
__device__ __forceinline__ float b2_op_sgn(float x) { return x > 0.0f ? 1.0f : (x < 0.0f ? -1.0f : 0.0f); }
__device__ __forceinline__ float b2_op_mod(float x, float y) {
    int yi = (int)y; return yi == 0 ? 0.0f : (float)((int)x % yi);
}
__device__ __forceinline__ float b2_op_int_div(float x, float y) {
    int yi = (int)y; return yi == 0 ? 0.0f : (float)((int)x / yi);
}

// ---- bulk asynchronous copies global -> shared, completion on an mbarrier -------------------------
// The staged kernels keep several 16 KB tiles in flight per CTA without spending registers on
// them: one thread issues cp.async.bulk copies (no multicast), all threads wait on the tile's
// mbarrier.  Every wait is bounded; when it runs out the kernel records it and carries on.
__device__ __forceinline__ unsigned b2_smem_u32(const void* ptr) {
    unsigned long long a;
    asm("cvta.to.shared.u64 %0, %1;" : "=l"(a) : "l"(ptr));
    return (unsigned)a;
}
__device__ __forceinline__ void b2_mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(b2_smem_u32(bar)), "r"(count)
                 : "memory");
}
__device__ __forceinline__ void b2_mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void b2_proxy_fence() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void b2_mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(b2_smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool b2_mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(b2_smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// bounded: ~4M polls (each poll itself waits up to a hardware time limit), then give up
__device__ __forceinline__ bool b2_mbar_wait(unsigned long long* bar, unsigned parity) {
    for (int i = 0; i < (1 << 22); ++i)
        if (b2_mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void b2_bulk_g2s(void* dst_smem, const void* src, unsigned bytes,
                                            unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(b2_smem_u32(dst_smem)), "l"(src), "r"(bytes), "r"(b2_smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void b2_lds_raw(const void* p, float4& w) { w = *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void b2_lds_raw(const void* p, b2_f8& w) {
    w.a = *reinterpret_cast<const float4*>(p);
    w.b = *(reinterpret_cast<const float4*>(p) + 1);
}
__device__ __forceinline__ void b2_lds_raw(const void* p, int4& w) { w = *reinterpret_cast<const int4*>(p); }
__device__ __forceinline__ void b2_lds_raw(const void* p, int2& w) { w = *reinterpret_cast<const int2*>(p); }

// ---- cheaper transcendentals for programs whose results are stored as flex16 ---------------------
// A flex16 store keeps 15 significant bits, so a few fp32 ulps of error in an intermediate move a
// stored mantissa only when the value sits within ~2^-21 of a rounding boundary.  These versions
// use the hardware ex2/rcp approximations (max relative error ~1e-6 over the ranges used) and cost
// a third of the libm calls, which is what lets a flex16 kernel stay bandwidth-bound.
__device__ __forceinline__ float b2_ex2_approx(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float b2_rcp_approx(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float b2_fast_exp(float x) { return b2_ex2_approx(x * 1.4426950408889634f); }
__device__ __forceinline__ float b2_fast_sig(float x) {
    return b2_rcp_approx(1.0f + b2_ex2_approx(x * -1.4426950408889634f));
}
// 1 - 2 / (exp(2|x|) + 1) with the sign of x: absolute error ~1e-7 everywhere (exp overflow gives
// exactly 1), which is far below one flex16 mantissa step of a tensor whose range covers tanh.
__device__ __forceinline__ float b2_fast_tanh(float x) {
    const float e = b2_ex2_approx(fabsf(x) * 2.8853900817779268f);
    const float t = __fmaf_rn(-2.0f, b2_rcp_approx(e + 1.0f), 1.0f);
    return copysignf(t, x);
}

#endif  // B2_EW_DEVICE_CUH
