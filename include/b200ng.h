/*
 * b200ng -- C ABI of the B200 backend for nGraph-Python graphs.
 *
 * Every entry point has C linkage, takes plain pointers and sizes, and returns an int status:
 * 0 on success, a negative B2_ERR_* code on failure (b2_last_error() then returns a
 * description owned by the library, valid until the next failing call on the same thread).
 * Device pointers are raw CUDA device addresses; `stream` is a cudaStream_t passed as void*.
 * Unless stated otherwise an entry point allocates no device memory: the caller owns every
 * buffer, including scratch.
 *
 * The reference drives its GPU through pycuda and has no C ABI of its own; each group below
 * names the reference interface (file:line in NervanaSystems/ngraph-python) whose job it takes
 * over.
 */
#ifndef B200NG_H
#define B200NG_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B2_OK 0
#define B2_ERR_INVALID (-1)     /* bad argument / unsupported program */
#define B2_ERR_CUDA (-2)        /* a CUDA runtime call failed */
#define B2_ERR_COMPILE (-3)     /* run-time kernel compilation failed */
#define B2_ERR_UNAVAILABLE (-4) /* a required system library could not be loaded */
#define B2_ERR_TIMEOUT (-5)     /* a bounded device-side wait ran out */
#define B2_ERR_COMM (-6)        /* NCCL reported an error */

const char* b2_last_error(void);
/* library version: major * 10000 + minor * 100 + patch */
int b2_version(void);
/* number of visible CUDA devices, or a negative error */
int b2_device_count(void);

/* ------------------------------------------------------------------------------------------
 * Fused elementwise + reduction kernels.
 * Replaces: ElementWiseKernel / CudaSourceFile / _get_compound_kernel / _generate_kernel_args
 * (ngraph/transformers/gputransform.py:86-345, ngraph/transformers/gpu/float_ew2.py:553-1653).
 * A program is a straight-line list of fp32 ops over up to 12 input tensors, with elementwise
 * outputs and at most one family of reductions, over an iteration space [A, B, C] (C innermost).
 * ------------------------------------------------------------------------------------------ */
#define B2_EW_MAX_IN 12
#define B2_EW_MAX_OUT 6   /* elementwise + reduction outputs together */
#define B2_EW_MAX_CONST 16
#define B2_EW_MAX_OPS 96

/* B2_FLEX16_PLANES (elementwise results only): the int16 mantissa is stored as two byte planes,
 * high bytes at the destination pointer and low bytes plane_bytes further -- the operand format
 * of the convolution entry points that take planes, so no separate split pass is needed. */
enum b2_dtype { B2_F32 = 0, B2_FLEX16 = 1, B2_FLEX16_PLANES = 2 };

/* op codes: one per template of float_ew2.py:31-68 */
enum b2_ew_opcode {
    B2_OP_ASSIGN = 0, B2_OP_NEG, B2_OP_ABS, B2_OP_SQRT, B2_OP_SQR, B2_OP_EXP, B2_OP_LOG,
    B2_OP_RCP, B2_OP_EXP2, B2_OP_LOG2, B2_OP_SIG, B2_OP_TANH, B2_OP_SAFELOG, B2_OP_SGN,
    B2_OP_SIN, B2_OP_COS,
    B2_OP_ADD = 32, B2_OP_SUB, B2_OP_MUL, B2_OP_DIV, B2_OP_INT_DIV, B2_OP_MOD, B2_OP_EQ,
    B2_OP_NE, B2_OP_LT, B2_OP_LE, B2_OP_GT, B2_OP_GE, B2_OP_POW, B2_OP_MINIMUM, B2_OP_MAXIMUM,
    B2_OP_ONEHOT, /* (index along the reduction-free axis B) == x */
    /* a: register, b: index k of an elementwise flex16 result of the same program.  The value
     * register a has after being stored as result k and read back: mantissa(a) * scale_k.  Lets
     * a kernel go on computing with a tensor it has just written, exactly as a later kernel would
     * see it.  In a probe launch results whose exponent is still to be chosen (bit k of the
     * launch's probe argument, counted from bit 1) pass through unchanged. */
    B2_OP_REQUANT
};

/* reduction codes: float_ew2.py:70-90 */
enum b2_ew_redop {
    B2_RED_SUM = 0, B2_RED_PROD, B2_RED_MAX, B2_RED_MIN, B2_RED_ARGMAX, B2_RED_ARGMIN
};

enum b2_ew_reduce_mode {
    B2_REDUCE_NONE = 0, /* elementwise only */
    B2_REDUCE_C = 1,    /* reduce the innermost axis: results have shape [A, B] */
    B2_REDUCE_B = 2     /* reduce the middle axis: results have shape [A, C] */
};

typedef struct b2_ew_tensor {
    int32_t dtype;       /* enum b2_dtype */
    int32_t flex_slot;   /* row of the flex table / stats array; -1 for fp32 */
    int64_t sa, sb, sc;  /* element strides along A, B, C; 0 broadcasts */
    int64_t plane_bytes; /* B2_FLEX16_PLANES: byte offset of the low plane (multiple of 8) */
} b2_ew_tensor;

/* registers: 0..n_in-1 inputs, n_in..n_in+n_const-1 constants, then one per op in order */
typedef struct b2_ew_op {
    int32_t opcode;
    int32_t a, b;        /* source registers (b ignored by unary ops) */
} b2_ew_op;

typedef struct b2_ew_result {
    int32_t reg;         /* register stored (elementwise) or reduced */
    int32_t redop;       /* enum b2_ew_redop; ignored for elementwise outputs */
    b2_ew_tensor t;      /* strides of the destination; the reduced axis has stride 0 */
} b2_ew_result;

typedef struct b2_ew_program {
    int64_t A, B, C;
    int32_t reduce_mode; /* enum b2_ew_reduce_mode */
    int32_t n_in, n_const, n_ops, n_out, n_red;
    b2_ew_tensor in[B2_EW_MAX_IN];
    b2_ew_op ops[B2_EW_MAX_OPS];
    b2_ew_result out[B2_EW_MAX_OUT]; /* n_out elementwise outputs, then n_red reductions */
} b2_ew_program;

typedef struct b2_flex_scale {
    float scale;      /* 2^-dec : readers multiply mantissas by it */
    float inv_scale;  /* 2^dec  : writers multiply values by it before rounding */
} b2_flex_scale;

typedef struct b2_ew_kernel b2_ew_kernel;

/* Compiles (or fetches from the in-process cache) the kernel for a program.
 * replaces CudaSourceFile.add_kernel + compile (float_ew2.py:1553-1623). */
int b2_ew_compile(const b2_ew_program* prog, b2_ew_kernel** out_kernel);
/* Generates and compiles the program for sm_100a without loading it (needs no GPU): the
 * build-time check of a program.  `vec` asks for the 128-bit variant where the program allows
 * it; the generated source is copied to `source` when given. */
int b2_ew_check(const b2_ew_program* prog, int vec, int probe, char* source, size_t source_cap);
/* Bytes of caller-provided scratch a launch needs (0 for most programs; reductions of a few
 * very long rows are split across CTAs and combined from scratch). */
int b2_ew_scratch_bytes(const b2_ew_kernel* k, size_t* bytes);
/* Launches.  `out` holds the n_out elementwise destinations followed by the n_red reduction
 * destinations.  `probe` != 0 runs the measuring variant used on a tensor's first write: nothing
 * is stored, and flex_stats[slot] receives the bit pattern of the largest |fp32 value| each
 * flex output would have been given (fmaxf order == integer order for non-negative floats).
 * Bits 1.. of `probe` name the results whose exponent is still to be chosen (bit 1 = result 0):
 * a B2_OP_REQUANT op that refers to such a result passes its value through unchanged.
 * `status` (device int32, may be NULL) is set to 1 if a bounded device-side wait ran out, in
 * which case the results of that launch are undefined.
 * replaces ElementWiseKernel.execute / bind_flex_scales (gputransform.py:277-345,
 * flexgputransform.py:56-64). */
int b2_ew_launch(b2_ew_kernel* k, const void* const* in, void* const* out, const float* consts,
                 const b2_flex_scale* flex_table, int32_t* flex_stats, void* scratch,
                 size_t scratch_bytes, int32_t* status, int probe, void* stream);
/* The same launch for callers that cannot allocate (no counterpart in the reference, which
 * always allocates through pycuda).  Meant for hosts that gave the whole device to their own
 * arena at start-up, and for execution loops that must never reach cudaMalloc because it
 * synchronises the device.  Scratch for split reductions comes from an array inside the library
 * (B2_EW_BUILTIN_SCRATCH_BYTES per device, held until the process exits); a launch that needs more
 * fails with B2_ERR_INVALID.  Calls no cudaMalloc/cudaFree and never compiles or loads a kernel:
 * the variant must already exist (b2_ew_compile builds the one for 16-byte-aligned pointers,
 * probe == 0).  The first call on a device resolves the array's address -- make it before any
 * stream capture.  All calls share the array: launches that overlap on the GPU race. */
#define B2_EW_BUILTIN_SCRATCH_BYTES (16 * 1024)
int b2_ew_launch_builtin_scratch(b2_ew_kernel* k, const void* const* in, void* const* out,
                                 const float* consts, const b2_flex_scale* flex_table,
                                 int32_t* flex_stats, int32_t* status, int probe, void* stream);
/* Generated CUDA source of a compiled kernel (for inspection / tests). */
const char* b2_ew_source(const b2_ew_kernel* k);
/* Number of kernel launches one b2_ew_launch issues (1, or 2 for split reductions). */
int b2_ew_launch_count(const b2_ew_kernel* k);
/* Directory searched first for libnvrtc.so.12 (optional; NULL keeps the default search). */
int b2_set_nvrtc_path(const char* path);

/* ------------------------------------------------------------------------------------------
 * Flex16 host<->device conversions, done on the device.
 * Replaces: FlexGPUDeviceTensor.get / __setitem__ (ngraph/transformers/flexgputransform.py:
 * 178-208), which convert on the host with numpy.
 * ------------------------------------------------------------------------------------------ */
/* dst[i] = (int16) trunc(clip(src[i] * table[slot].inv_scale, -32768, 32767));
 * stats[slot] = max(stats[slot], max |dst|). */
int b2_flex_host_quantize(const float* src, int16_t* dst, int64_t n, const b2_flex_scale* table,
                          int32_t slot, int32_t* stats, void* stream);
/* dst[i] = table[slot].scale * (float) src[i] */
int b2_flex_dequantize(const int16_t* src, float* dst, int64_t n, const b2_flex_scale* table,
                       int32_t slot, void* stream);
/* *out = max(*out, bit pattern of max |src[i]|) (NaN counts as 0); used to pick a first exponent
 * for data arriving from the host. */
int b2_absmax_bits_f32(const float* src, int64_t n, int32_t* out, void* stream);
/* End of a call in one launch: host_stats[i] = stats[i], stats[i] = 0 for i < n, and
 * *host_status = *status (both NULL to skip).  host_stats / host_status are pinned host memory
 * that the device can address (cudaHostAlloc memory under unified addressing); the values are
 * there once the stream has been synchronised.  Replaces the per-kernel synchronous statistics
 * read of the reference's flex transformer (manage_after_computation after every kernel,
 * ngraph/transformers/flexgputransform.py:347-371) by one read per call. */
int b2_flex_publish(int32_t* stats, int32_t n, const int32_t* status, int32_t* host_stats,
                    int32_t* host_status, void* stream);

/* ------------------------------------------------------------------------------------------
 * Dense GEMM on tcgen05 tensor cores: C[M,N] = op(A)[M,K] * op(B)[K,N], C row-major (ldc).
 * Replaces: GEMMKernel and the sgemm / fgemm SASS kernels (ngraph/transformers/gpu/gemm.py:26-263,
 * gpu/kernels/sass/fgemm_common_128x128.sass).  op() is given by element strides, as the
 * reference derives nn/nt/tn from strides (gemm.py:95-110): element (m,k) of op(A) is
 * A[m*a_row_stride + k*a_k_stride], element (k,n) of op(B) is B[k*b_k_stride + n*b_col_stride];
 * one stride of each pair must be 1.  `scratch` (1024-byte aligned, b2_gemm_scratch_bytes) holds
 * the K-major operand planes the kernel streams with TMA.
 * ------------------------------------------------------------------------------------------ */
int b2_gemm_scratch_bytes(int32_t flex, int32_t M, int32_t N, int32_t K, size_t* bytes);
/* fp32 via 3xTF32 (relative error ~2^-21). */
int b2_gemm_f32(const float* A, int64_t a_row_stride, int64_t a_k_stride, const float* B,
                int64_t b_k_stride, int64_t b_col_stride, float* C, int64_t ldc, int32_t M,
                int32_t N, int32_t K, void* scratch, size_t scratch_bytes, int32_t* status,
                void* stream);
/* flex16: exact integer products (int8 hi/lo split, int32 accumulation), output rescaled by
 * 2^(decC - decA - decB) with round-to-nearest-even, saturated to int16; stats[slotC] receives
 * max |mantissa| (fgemm epilogue, fgemm_common_128x128.sass:29-97,331-420).  K above 32768 is
 * cut into slices of exact int32 sums that are added in 64-bit.
 * probe != 0: nothing is stored; *probe_out receives max |exact integer sum| (the caller
 * multiplies by 2^-(decA+decB) to get the unsaturated range of the result). */
int b2_gemm_flex16(const int16_t* A, int64_t a_row_stride, int64_t a_k_stride, const int16_t* B,
                   int64_t b_k_stride, int64_t b_col_stride, int16_t* C, int64_t ldc, int32_t M,
                   int32_t N, int32_t K, const b2_flex_scale* table, int32_t slotA, int32_t slotB,
                   int32_t slotC, int32_t* stats, void* scratch, size_t scratch_bytes,
                   uint64_t* probe_out, int32_t* status, int32_t probe, void* stream);

/* ------------------------------------------------------------------------------------------
 * Convolution forward and average pooling on C,D,H,W,N tensors (filters C,T,R,S,K, outputs
 * K,M,P,Q,N), the reference's layouts.
 * Replaces: ConvFpropKernel / FlexConvFpropKernel (ngraph/transformers/gpu/conv.py:24-100,
 * gpu/flex_conv.py:49-200) and PoolFpropKernel avg (gpu/pool.py:27-220).
 * The dims struct has the fields of the reference's conv_params plus the tensor extents
 * (ngraph/op_graph/convolution.py; ngraph/testing/conv_utils.py:ConvParams).
 * ------------------------------------------------------------------------------------------ */
typedef struct b2_conv_dims {
    int32_t C, D, H, W, N;        /* input */
    int32_t K, T, R, S;           /* filter */
    int32_t M, P, Q;              /* output */
    int32_t pad_d, pad_h, pad_w, str_d, str_h, str_w, dil_d, dil_h, dil_w;
} b2_conv_dims;
int b2_conv_fprop_scratch_bytes(int32_t flex, const b2_conv_dims* d, size_t* bytes);
/* fp32 (3xTF32 on the tensor cores). */
int b2_conv_fprop_f32(const float* I, const float* F, float* O, const b2_conv_dims* d,
                      void* scratch, size_t scratch_bytes, int32_t* status, void* stream);
/* flex16: exact integer sums, rescale/saturate/statistic as b2_gemm_flex16; probe as there. */
int b2_conv_fprop_flex16(const int16_t* I, const int16_t* F, int16_t* O, const b2_conv_dims* d,
                         const b2_flex_scale* table, int32_t slotI, int32_t slotF, int32_t slotO,
                         int32_t* stats, void* scratch, size_t scratch_bytes, uint64_t* probe_out,
                         int32_t* status, int32_t probe, void* stream);
/* The flex16 convolution in parts, for callers that keep operand planes around: the tile kernel
 * reads its streamed tensor (pass 0: the activations I; pass 1, the input gradient of a
 * unit-stride convolution: the error tensor E) and the filters as byte planes -- high and low
 * bytes of the int16 mantissas, the streamed tensor in its own C,H,W,N (K,P,Q,N) order with the
 * low plane act_plane_bytes after the high plane, 1024-byte aligned.  A fused elementwise kernel
 * can emit such planes directly (B2_FLEX16_PLANES) and the filter planes of constant weights can
 * be built once, which leaves ONE launch per convolution.  `supported` is 0 where the plane path
 * does not apply (batch not a multiple of 128, dilation, very large windows; pass 1: strides);
 * use b2_conv_fprop_flex16 / b2_conv_bprop_flex16 there.  `d` always describes the FORWARD
 * convolution.  No counterpart in the reference, whose kernels read int16 tensors directly. */
enum b2_conv_pass { B2_CONV_FPROP = 0, B2_CONV_BPROP = 1 };
int b2_conv_planes_info(const b2_conv_dims* d, int32_t pass, int32_t* supported,
                        size_t* act_plane_bytes, size_t* filter_planes_bytes);
int b2_conv_split_activations(const int16_t* X, const b2_conv_dims* d, int32_t pass, void* planes,
                              void* stream);
int b2_conv_filter_planes(const int16_t* F, const b2_conv_dims* d, int32_t pass, void* planes,
                          void* stream);
int b2_conv_flex16_planes(int32_t pass, const void* act_planes, const void* filter_planes,
                          int16_t* out, const b2_conv_dims* d, const b2_flex_scale* table,
                          int32_t slotX, int32_t slotF, int32_t slotOut, int32_t* stats,
                          uint64_t* probe_out, int32_t* status, int32_t probe, void* stream);
/* The same with the elementwise tail of a convolution layer folded into the tile kernel's
 * epilogue: y = relu?(conv + bias[k] + residual) evaluated in fp32 from the exact integer sums,
 * quantised ONCE with the output's exponent (slotOut), stored as int16 (write_int16) and / or as
 * the byte planes the next convolution reads (out_planes, low plane plane_bytes further).  bias:
 * int16 per output channel; residual: int16 tensor in the output's K,P,Q,N layout; NULL = absent.
 * probe != 0 stores nothing and leaves the bit pattern of max |y| (fp32) in *probe_out.
 * Replaces the bias / activation arguments the reference's convolution kernels carry
 * (ConvFpropKernel bsum / relu flags, ngraph/transformers/gpu/conv.py:48-100) and the
 * elementwise kernels it launches after them. */
typedef struct b2_conv_epilogue {
    const int16_t* bias;     int32_t slot_bias;
    const int16_t* residual; int32_t slot_residual;
    int32_t relu;
    int32_t write_int16;
    void* out_planes;        size_t plane_bytes;
} b2_conv_epilogue;
int b2_conv_flex16_planes_fused(int32_t pass, const void* act_planes, const void* filter_planes,
                                int16_t* out, const b2_conv_dims* d, const b2_flex_scale* table,
                                int32_t slotX, int32_t slotF, int32_t slotOut,
                                const b2_conv_epilogue* epilogue, int32_t* stats,
                                uint64_t* probe_out, int32_t* status, int32_t probe, void* stream);
/* The two training contractions of a convolution whose forward pass has the dimensions `d`
 * (d always describes the FORWARD convolution: I is C,D,H,W,N, F is C,T,R,S,K, E is K,M,P,Q,N).
 * Replace ConvBpropKernel / ConvUpdateKernel (ngraph/transformers/gpu/conv.py:121-312) and
 * FlexConvBpropKernel / FlexConvUpdateKernel (gpu/flex_conv.py:203-621); arithmetic as the
 * reference's CPU engine states it (ngraph/transformers/cpu/cpuengine.py:256-271, 395-418).
 *   bprop:  GI[C,D,H,W,N] = sum_{k,r,s} F[c,r,s,k] * E[k,p,q,n],  h = p*str - pad + r*dil
 *   update: U[C,T,R,S,K]  = sum_{p,q,n} I[c,h,w,n] * E[k,p,q,n]   (sums added in a fixed order)
 * flex16 variants: exact integer sums, rescale / saturate / statistic / probe as b2_gemm_flex16
 * with (slot of first operand, slot of second operand, slot of the result). */
int b2_conv_bprop_scratch_bytes(int32_t flex, const b2_conv_dims* d, size_t* bytes);
int b2_conv_bprop_f32(const float* E, const float* F, float* GI, const b2_conv_dims* d,
                      void* scratch, size_t scratch_bytes, int32_t* status, void* stream);
int b2_conv_bprop_flex16(const int16_t* E, const int16_t* F, int16_t* GI, const b2_conv_dims* d,
                         const b2_flex_scale* table, int32_t slotE, int32_t slotF, int32_t slotGI,
                         int32_t* stats, void* scratch, size_t scratch_bytes, uint64_t* probe_out,
                         int32_t* status, int32_t probe, void* stream);
int b2_conv_update_scratch_bytes(int32_t flex, const b2_conv_dims* d, size_t* bytes);
int b2_conv_update_f32(const float* I, const float* E, float* U, const b2_conv_dims* d,
                       void* scratch, size_t scratch_bytes, int32_t* status, void* stream);
int b2_conv_update_flex16(const int16_t* I, const int16_t* E, int16_t* U, const b2_conv_dims* d,
                          const b2_flex_scale* table, int32_t slotI, int32_t slotE, int32_t slotU,
                          int32_t* stats, void* scratch, size_t scratch_bytes, uint64_t* probe_out,
                          int32_t* status, int32_t probe, void* stream);
/* Average pooling over H,W windows.  flex != 0: int16 in and out sharing one exponent
 * (ngraph/transformers/passes/flexpass.py:40-48); *stats_slot = max(*stats_slot, max |out|). */
int b2_pool_avg_fprop(const void* I, void* O, int32_t flex, int32_t C, int32_t H, int32_t W,
                      int32_t N, int32_t P, int32_t Q, int32_t R, int32_t S, int32_t pad_h,
                      int32_t pad_w, int32_t str_h, int32_t str_w, int32_t* stats_slot,
                      void* stream);
/* Max pooling over the part of each window that lies inside the image (np.max of the same
 * slices, ngraph/transformers/cpu/cpuengine.py:297-300); flex as for the average. */
int b2_pool_max_fprop(const void* I, void* O, int32_t flex, int32_t C, int32_t H, int32_t W,
                      int32_t N, int32_t P, int32_t Q, int32_t R, int32_t S, int32_t pad_h,
                      int32_t pad_w, int32_t str_h, int32_t str_w, int32_t* stats_slot,
                      void* stream);
/* Gradient of pooling with respect to its input (BpropPoolOp; arithmetic and summation order of
 * ngraph/transformers/cpu/cpuengine.py:306-336).  avg: every element of a window receives
 * E / (elements of the window inside the image); max: the first maximum of the window (np.argmax
 * order) receives E, found again from the pooled tensor I (unused, may be NULL, for avg).
 * flex16: fp32 arithmetic, one quantisation with slotGI's exponent, statistic or probe (bit
 * pattern of max |fp32 result| into *probe_out) as for the other flex16 entry points. */
int b2_pool_bprop(const void* E, const void* I, void* GI, int32_t flex, int32_t is_max, int32_t C,
                  int32_t H, int32_t W, int32_t N, int32_t P, int32_t Q, int32_t R, int32_t S,
                  int32_t pad_h, int32_t pad_w, int32_t str_h, int32_t str_w,
                  const b2_flex_scale* table, int32_t slotE, int32_t slotGI, int32_t* stats,
                  uint64_t* probe_out, int32_t probe, void* stream);

/* ------------------------------------------------------------------------------------------
 * N-d strided copy / transpose between two tensors of the same extents.
 * Replaces: DimShuffleKernel and the generated copy-transpose kernels (ngraph/transformers/gpu/
 * tensor_ops.py:119-204, gpu/kernels/cuda/copy_transpose.py:78-282), which also implement AssignOp
 * between differently laid-out tensors (gputransform.py:393-395) and non-contiguous host I/O
 * (gputransform.py:873-909).  dst[sum_i idx_i * dst_strides[i]] = src[sum_i idx_i *
 * src_strides[i]] for every index tuple below `shape`; strides are in elements and non-negative
 * (a source stride of 0 broadcasts); the destination must not alias itself.  Where the axis that
 * is contiguous in the source differs from the one contiguous in the destination the copy goes
 * through 32 x 32 shared-memory tiles so that both sides move whole rows.
 * ------------------------------------------------------------------------------------------ */
#define B2_DIMSHUFFLE_MAX_RANK 8
int b2_dimshuffle(const void* src, void* dst, int32_t elem_bytes, int32_t rank,
                  const int64_t* shape, const int64_t* src_strides, const int64_t* dst_strides,
                  void* stream);

/* ------------------------------------------------------------------------------------------
 * Random fill: out[i] ~ U[a, b) (B2_RNG_UNIFORM: a = low, b = high) or N(a, b) (B2_RNG_NORMAL:
 * a = loc, b = scale), n elements, fp32 or flex16 (quantised with slot's exponent; statistic or
 * probe -- bit pattern of max |fp32 value| into *probe_out -- as for b2_pool_bprop).
 * Replaces RngFillKernel / FlexRngFillKernel (ngraph/transformers/gpu/tensor_ops.py:621-661,
 * 713-740).  Counter-based generator (Philox-4x32-10): (seed, offset) determines the tensor.
 * device_counter (may be NULL): a 64-bit device word added to `offset` and advanced by one after
 * a storing launch, so that launches replayed from a CUDA graph still draw fresh numbers.
 * ------------------------------------------------------------------------------------------ */
enum b2_rng_distribution { B2_RNG_UNIFORM = 0, B2_RNG_NORMAL = 1 };
int b2_rng_fill(void* out, int32_t flex, int64_t n, int32_t distribution, float a, float b,
                uint64_t seed, uint64_t offset, uint64_t* device_counter,
                const b2_flex_scale* table, int32_t slot, int32_t* stats, uint64_t* probe_out,
                int32_t probe, void* stream);

/* Lookup table (embedding).  lut_axis 0: lut [V][F], out / delta [n_idx][F], dW [V][F];
 * lut_axis 1: lut [F][V], out / delta [F][n_idx], dW [F][V].  Indices are values of the tensor
 * idx (fp32, or flex16 mantissas with the scale of slot_idx), rounded to the nearest integer.
 *   fprop:  out = lut.take(idx, axis)                (rows outside [0, V) read as zero);
 *           flex16: mantissas are copied, the result carries the table's exponent
 *   update: dW[w] = sum of the rows of delta whose index is w, in increasing position; the row
 *           pad_idx (pass -1 for none) and rows never looked up are zero
 * replaces LUTBpropKernel / fprop_lut / update_lut (ngraph/transformers/gpu/lut.py,
 * ngraph/transformers/cpu/cpuengine.py:421-435).  flex16 update: fp32 sums, one quantisation with
 * slot_dW's exponent, statistic or probe as for b2_pool_bprop. */
int b2_lut_fprop(const void* lut, const void* idx, void* out, int32_t flex, int32_t lut_axis,
                 int32_t V, int32_t F, int32_t n_idx, const b2_flex_scale* table,
                 int32_t slot_idx, void* stream);
int b2_lut_update(const void* delta, const void* idx, void* dW, int32_t flex, int32_t lut_axis,
                  int32_t V, int32_t F, int32_t n_idx, int32_t pad_idx, const b2_flex_scale* table,
                  int32_t slot_delta, int32_t slot_idx, int32_t slot_dW, int32_t* stats,
                  uint64_t* probe_out, int32_t probe, void* stream);

/* ------------------------------------------------------------------------------------------
 * Gradient allreduce over NCCL (NVLink / NVSwitch), one process per GPU.
 * Replaces: CudaAllReduceKernel and its reduction kernel (ngraph/transformers/gpu/tensor_ops.py:
 * 52-116, 416-618), which reduce one gradient tensor at a time with peer-to-peer copies, MPI
 * barriers and host synchronisations.  The caller reduces a whole bucket of fp32 gradients in
 * place, on the stream it names.  NCCL is loaded at run time (the copy already in the process if
 * there is one); without it these entry points return B2_ERR_UNAVAILABLE and the rest of the
 * library is unaffected.
 *   b2_comm_unique_id   one replica makes the 128-byte identifier and hands it to the others
 *                       (any channel: a file, a socket, torch.distributed's store)
 *   b2_comm_init        every replica joins (collective: returns once all have called it)
 *   b2_comm_allreduce_f32  buf[0..count) <- sum over replicas, / nranks when mean != 0; queued on
 *                       `stream`, returns at once
 *   b2_comm_poll_error  B2_OK, or B2_ERR_COMM once NCCL has reported an asynchronous failure (a
 *                       replica that died, a link fault); never blocks
 *   b2_comm_abort       ends the collectives in flight after a failure so that a stream
 *                       synchronisation returns; the handle can then only be destroyed
 * ------------------------------------------------------------------------------------------ */
#define B2_COMM_ID_BYTES 128
typedef struct b2_comm b2_comm;
int b2_set_nccl_path(const char* path);
int b2_comm_version(int32_t* version);
int b2_comm_unique_id(void* id_out);
int b2_comm_init(const void* id, int32_t rank, int32_t nranks, int32_t device, b2_comm** out);
int b2_comm_allreduce_f32(b2_comm* comm, float* buf, int64_t count, int32_t mean, void* stream);
int b2_comm_poll_error(b2_comm* comm);
int b2_comm_abort(b2_comm* comm);
int b2_comm_destroy(b2_comm* comm);

/* ------------------------------------------------------------------------------------------
 * Self-test of the bounded-wait path.  Every device-side wait of the tile kernels gives up after
 * a fixed number of polls, sets the caller's status word to 1 (the launching entry point's
 * `status` argument; the host then reports B2_ERR_TIMEOUT-class failure for that call) and lets
 * the kernel finish normally, tensor memory freed.  This entry point runs that path on purpose: a
 * one-block kernel waits, with the kernels' own wait routine, `poll_limit` polls (1..65536) on a
 * barrier nothing completes, then sets *status = 1, writes the polls it waited to *polls_waited
 * (may be NULL), frees its tensor memory and returns.  Harmless: no fault, no trap, the context
 * stays usable.  No counterpart in the reference (its kernels have no device-side waits).
 * ------------------------------------------------------------------------------------------ */
int b2_selftest_bounded_wait(int32_t poll_limit, int32_t* status, int32_t* polls_waited,
                             void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200NG_H */
