// Fused elementwise + reduction kernels: program -> CUDA source -> NVRTC (sm_100a) -> launch.
//
// Takes the place of the reference's float_ew2 code generator
// (ngraph/transformers/gpu/float_ew2.py:553-1653).  Differences in design:
//   * a program holds MANY ops (the reference emits one kernel per op because its fusion pass
//     was never enabled); intermediate values stay in registers;
//   * loads and stores along the innermost axis are 128-bit; rows are reduced by warp shuffles
//     and one shared-memory exchange;
//   * the flex16 statistic (max |mantissa|) is kept per thread, folded per CTA and sent to
//     global memory with ONE atomicMax per CTA (the reference issues one per thread);
//   * flex scales are read from a device table, so a captured launch can be replayed after the
//     host has changed exponents.
#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <sstream>
#include <unordered_map>
#include <vector>

#include "b2_common.h"

namespace {

// The device helper header as text (generated at build time from b2_ew_device.cuh).
const char* kDeviceHeader =
#include "b2_ew_device_src.inc"
    ;

// ---- host mirror of the launch argument block (layout must match b2_ew_device.cuh) -----------
struct EwArgs {
    long long A, B, C;
    const void* in[B2_EW_MAX_IN];
    long long in_sa[B2_EW_MAX_IN], in_sb[B2_EW_MAX_IN], in_sc[B2_EW_MAX_IN];
    int in_slot[B2_EW_MAX_IN];
    void* out[B2_EW_MAX_OUT];
    long long out_sa[B2_EW_MAX_OUT], out_sb[B2_EW_MAX_OUT], out_sc[B2_EW_MAX_OUT];
    int out_slot[B2_EW_MAX_OUT];
    long long out_plane[B2_EW_MAX_OUT];
    float consts[B2_EW_MAX_CONST];
    const b2_flex_scale* flex_table;
    int* flex_stats;
    float* scratch;
    int* status;
    int nsplit;
    unsigned fresh_mask;
};

// ---- NVRTC through dlopen (no link-time dependency: the library loads on machines without it) --
typedef int nvrtcResult;
typedef struct _nvrtcProgram* nvrtcProgram;
struct Nvrtc {
    void* handle = nullptr;
    nvrtcResult (*CreateProgram)(nvrtcProgram*, const char*, const char*, int, const char* const*,
                                 const char* const*) = nullptr;
    nvrtcResult (*CompileProgram)(nvrtcProgram, int, const char* const*) = nullptr;
    nvrtcResult (*GetCUBINSize)(nvrtcProgram, size_t*) = nullptr;
    nvrtcResult (*GetCUBIN)(nvrtcProgram, char*) = nullptr;
    nvrtcResult (*GetProgramLogSize)(nvrtcProgram, size_t*) = nullptr;
    nvrtcResult (*GetProgramLog)(nvrtcProgram, char*) = nullptr;
    nvrtcResult (*DestroyProgram)(nvrtcProgram*) = nullptr;
    const char* (*GetErrorString)(nvrtcResult) = nullptr;
};
Nvrtc g_nvrtc;
std::string g_nvrtc_dir;
std::mutex g_mutex;

int load_nvrtc() {
    if (g_nvrtc.handle) return B2_OK;
    std::vector<std::string> names;
    if (!g_nvrtc_dir.empty()) names.push_back(g_nvrtc_dir + "/libnvrtc.so.12");
    names.push_back("libnvrtc.so.12");
    names.push_back("/usr/local/cuda/lib64/libnvrtc.so.12");
    names.push_back("libnvrtc.so");
    void* h = nullptr;
    std::string tried;
    for (auto& n : names) {
        h = dlopen(n.c_str(), RTLD_NOW | RTLD_GLOBAL);
        if (h) break;
        tried += n + " ";
    }
    if (!h) return b2::fail(B2_ERR_UNAVAILABLE, "cannot load NVRTC (tried: %s)", tried.c_str());
#define B2_SYM(field, name)                                                        \
    *(void**)(&g_nvrtc.field) = dlsym(h, name);                                    \
    if (!g_nvrtc.field) return b2::fail(B2_ERR_UNAVAILABLE, "NVRTC lacks %s", name);
    B2_SYM(CreateProgram, "nvrtcCreateProgram")
    B2_SYM(CompileProgram, "nvrtcCompileProgram")
    B2_SYM(GetCUBINSize, "nvrtcGetCUBINSize")
    B2_SYM(GetCUBIN, "nvrtcGetCUBIN")
    B2_SYM(GetProgramLogSize, "nvrtcGetProgramLogSize")
    B2_SYM(GetProgramLog, "nvrtcGetProgramLog")
    B2_SYM(DestroyProgram, "nvrtcDestroyProgram")
    B2_SYM(GetErrorString, "nvrtcGetErrorString")
#undef B2_SYM
    g_nvrtc.handle = h;
    return B2_OK;
}

struct Module {
    cudaLibrary_t lib = nullptr;
    cudaKernel_t main = nullptr;
    cudaKernel_t finalize = nullptr;
};
std::unordered_map<std::string, Module*> g_modules;  // keyed by generated source

int nvrtc_compile(const std::string& src, std::vector<char>* cubin) {
    int rc = load_nvrtc();
    if (rc) return rc;
    nvrtcProgram prog;
    nvrtcResult r = g_nvrtc.CreateProgram(&prog, src.c_str(), "b2_ew.cu", 0, nullptr, nullptr);
    if (r) return b2::fail(B2_ERR_COMPILE, "nvrtcCreateProgram: %s", g_nvrtc.GetErrorString(r));
    const char* opts[] = {"--gpu-architecture=sm_100a", "--fmad=false", "--std=c++17",
                          "-lineinfo"};
    r = g_nvrtc.CompileProgram(prog, 4, opts);
    if (r) {
        size_t n = 0;
        g_nvrtc.GetProgramLogSize(prog, &n);
        std::string log(n, '\0');
        if (n) g_nvrtc.GetProgramLog(prog, &log[0]);
        g_nvrtc.DestroyProgram(&prog);
        return b2::fail(B2_ERR_COMPILE, "NVRTC: %s\n%s", g_nvrtc.GetErrorString(r),
                        log.substr(0, 1500).c_str());
    }
    size_t n = 0;
    g_nvrtc.GetCUBINSize(prog, &n);
    cubin->resize(n);
    g_nvrtc.GetCUBIN(prog, cubin->data());
    g_nvrtc.DestroyProgram(&prog);
    return B2_OK;
}

int compile_source(const std::string& src, bool has_finalize, Module** out) {
    std::lock_guard<std::mutex> lock(g_mutex);
    auto it = g_modules.find(src);
    if (it != g_modules.end()) { *out = it->second; return B2_OK; }
    std::vector<char> cubin;
    int rc = nvrtc_compile(src, &cubin);
    if (rc) return rc;
    Module* m = new Module();
    B2_CUDA(cudaLibraryLoadData(&m->lib, cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0));
    B2_CUDA(cudaLibraryGetKernel(&m->main, m->lib, "b2_ew_main"));
    if (has_finalize) B2_CUDA(cudaLibraryGetKernel(&m->finalize, m->lib, "b2_ew_finalize"));
    g_modules[src] = m;
    *out = m;
    return B2_OK;
}

// ---- code generation ------------------------------------------------------------------------
const int kThreads = 256;
const int kSMs = 148;

struct Plan {
    int V = 1;          // elements per thread per step along C
    int group = 256;    // threads cooperating on one row (REDUCE_C)
    int nsplit = 1;     // CTAs sharing one row (REDUCE_C)
    dim3 grid;
    bool vec = false;
    bool prefetch = false;   // load step j+1 into spare registers before computing step j
    int minb = 1;            // __launch_bounds__ second argument (CTAs per SM to fit registers for)
    bool staged = false;     // inputs travel global -> shared by cp.async.bulk, STAGES deep
    int stages = 3;
    int stage_bytes = 0;
};

const char* red_name(int op) {
    static const char* n[] = {"B2_RED_SUM", "B2_RED_PROD", "B2_RED_MAX", "B2_RED_MIN",
                              "B2_RED_ARGMAX", "B2_RED_ARGMIN"};
    return n[op];
}
bool is_arg(int op) { return op == B2_RED_ARGMAX || op == B2_RED_ARGMIN; }

std::string reg(int i) { return "r" + std::to_string(i); }

int emit_op(std::ostringstream& o, const b2_ew_op& op, int dst, bool fast, bool probe) {
    const std::string d = "const float " + reg(dst) + " = ";
    const std::string x = reg(op.a), y = reg(op.b);
    switch (op.opcode) {
        case B2_OP_REQUANT: {
            const std::string k = std::to_string(op.b);
            const std::string rq = "b2_requant(" + x + ", rq" + k + ", rs" + k + ")";
            if (probe) o << d << "((p.fresh_mask >> " << k << ") & 1u) ? " << x << " : " << rq << ";";
            else o << d << rq << ";";
            break;
        }
        case B2_OP_ASSIGN: o << d << x << ";"; break;
        case B2_OP_NEG: o << d << "-" << x << ";"; break;
        case B2_OP_ABS: o << d << "fabsf(" << x << ");"; break;
        case B2_OP_SQRT: o << d << "sqrtf(" << x << ");"; break;
        case B2_OP_SQR: o << d << x << " * " << x << ";"; break;
        case B2_OP_EXP: o << d << (fast ? "b2_fast_exp(" : "expf(") << x << ");"; break;
        case B2_OP_LOG: o << d << "logf(" << x << ");"; break;
        case B2_OP_RCP: o << d << "1.0f / " << x << ";"; break;
        case B2_OP_EXP2: o << d << "exp2f(" << x << ");"; break;
        case B2_OP_LOG2: o << d << "log2f(" << x << ");"; break;
        case B2_OP_SIG: o << d << (fast ? "b2_fast_sig(" : "b2_op_sig(") << x << ");"; break;
        case B2_OP_TANH: o << d << (fast ? "b2_fast_tanh(" : "tanhf(") << x << ");"; break;
        case B2_OP_SAFELOG: o << d << "b2_op_safelog(" << x << ");"; break;
        case B2_OP_SGN: o << d << "b2_op_sgn(" << x << ");"; break;
        case B2_OP_SIN: o << d << "sinf(" << x << ");"; break;
        case B2_OP_COS: o << d << "cosf(" << x << ");"; break;
        case B2_OP_ADD: o << d << x << " + " << y << ";"; break;
        case B2_OP_SUB: o << d << x << " - " << y << ";"; break;
        case B2_OP_MUL: o << d << x << " * " << y << ";"; break;
        case B2_OP_DIV: o << d << x << " / " << y << ";"; break;
        case B2_OP_INT_DIV: o << d << "b2_op_int_div(" << x << ", " << y << ");"; break;
        case B2_OP_MOD: o << d << "b2_op_mod(" << x << ", " << y << ");"; break;
        case B2_OP_EQ: o << d << "(" << x << " == " << y << ") ? 1.0f : 0.0f;"; break;
        case B2_OP_NE: o << d << "(" << x << " != " << y << ") ? 1.0f : 0.0f;"; break;
        case B2_OP_LT: o << d << "(" << x << " < " << y << ") ? 1.0f : 0.0f;"; break;
        case B2_OP_LE: o << d << "(" << x << " <= " << y << ") ? 1.0f : 0.0f;"; break;
        case B2_OP_GT: o << d << "(" << x << " > " << y << ") ? 1.0f : 0.0f;"; break;
        case B2_OP_GE: o << d << "(" << x << " >= " << y << ") ? 1.0f : 0.0f;"; break;
        case B2_OP_POW: o << d << "powf(" << x << ", " << y << ");"; break;
        case B2_OP_MINIMUM: o << d << "fminf(" << x << ", " << y << ");"; break;
        case B2_OP_MAXIMUM: o << d << "fmaxf(" << x << ", " << y << ");"; break;
        case B2_OP_ONEHOT: o << d << "((float)b_idx == " << x << ") ? 1.0f : 0.0f;"; break;
        default: return -1;
    }
    o << "\n";
    return 0;
}

const char* ctype(int dtype) {
    return dtype == B2_FLEX16 ? "short" : dtype == B2_FLEX16_PLANES ? "unsigned char" : "float";
}
// results may be flex16 stored as int16 or as the two byte planes the convolution kernels read
inline bool is_flex(int dtype) { return dtype == B2_FLEX16 || dtype == B2_FLEX16_PLANES; }

// Emits the per-element body: registers for inputs/constants, the op list.
bool uses_flex(const b2_ew_program& p) {
    for (int i = 0; i < p.n_in; ++i) if (p.in[i].dtype == B2_FLEX16) return true;
    for (int k = 0; k < p.n_out + p.n_red; ++k) if (is_flex(p.out[k].t.dtype)) return true;
    return false;
}

int emit_body(std::ostringstream& o, const b2_ew_program& p, const Plan& pl, bool probe) {
    // flex16 programs use the cheaper transcendentals (see b2_ew_device.cuh); fp32 programs
    // keep CUDA libm, as the reference's generated code does.
    const bool fast = uses_flex(p);
    for (int i = 0; i < p.n_in; ++i) {
        o << "            const float " << reg(i) << " = ";
        if (p.in[i].sc == 0) o << "xb" << i << ";\n";
        else if (pl.vec && p.in[i].dtype == B2_FLEX16)
            o << "b2_elem(w" << i << ", e, s" << i << ", bias" << i << ");\n";
        else if (pl.vec) o << "b2_elem(w" << i << ", e, 1.0f, 0.0f);\n";
        else o << "x" << i << "[e];\n";
    }
    for (int i = 0; i < p.n_const; ++i)
        o << "            const float " << reg(p.n_in + i) << " = k" << i << ";\n";
    for (int i = 0; i < p.n_ops; ++i) {
        o << "            ";
        if (emit_op(o, p.ops[i], p.n_in + p.n_const + i, fast, probe)) return -1;
    }
    return 0;
}

// Raw (unconverted) register type of one vector load of an input.
const char* raw_type(int dtype, int V) {
    if (dtype == B2_FLEX16) return V == 8 ? "int4" : "int2";
    return V == 8 ? "b2_f8" : "float4";
}
bool prefetchable(const b2_ew_tensor& t, const Plan& pl) { return pl.vec && t.sc != 0; }

// Issues the raw vector loads of step `jexpr` into registers <prefix><i>.
void emit_raw_loads(std::ostringstream& o, const b2_ew_program& p, const Plan& pl,
                    const std::string& prefix, const std::string& jexpr, const std::string& ind) {
    for (int i = 0; i < p.n_in; ++i)
        if (prefetchable(p.in[i], pl))
            o << ind << "b2_ldraw(in" << i << " + (" << jexpr << ") * V, " << prefix << i << ");\n";
}

// Loads of one step: x<i>[V] for every input.  In the vector variant the raw registers w<i>
// were filled one step earlier (software prefetch) and are only converted here.
void emit_loads(std::ostringstream& o, const b2_ew_program& p, const Plan& pl,
                const std::string& ind) {
    for (int i = 0; i < p.n_in; ++i) {
        const b2_ew_tensor& t = p.in[i];
        const bool flex = t.dtype == B2_FLEX16;
        if (t.sc == 0) {
            // broadcast along C: the scalar xb<i> is used directly
        } else if (pl.vec) {
            // converted lazily, element by element, inside the body (b2_elem)
            if (flex) o << ind << "const float bias" << i << " = b2_i16_bias(s" << i << ");\n";
        } else {
            o << ind << "float x" << i << "[V];\n";
            o << ind << "_Pragma(\"unroll\") for (int e = 0; e < V; ++e) x" << i << "[e] = ";
            if (flex) o << "s" << i << " * (float)";
            o << "in" << i << "[(c + e) * p.in_sc[" << i << "]];\n";
        }
    }
}

// Store of one elementwise output from y<k>[V].
void emit_store(std::ostringstream& o, const b2_ew_program& p, const Plan& pl, int k, bool probe,
                const std::string& ind) {
    const b2_ew_tensor& t = p.out[k].t;
    const bool flex = is_flex(t.dtype);
    const bool planes = t.dtype == B2_FLEX16_PLANES;
    if (probe) {
        if (flex)
            o << ind << "_Pragma(\"unroll\") for (int e = 0; e < V; ++e) stat" << k
              << " = max(stat" << k << ", b2_absbits(y" << k << "[e]));\n";
        return;
    }
    if (!flex) {
        if (pl.vec)
            for (int h = 0; h < pl.V / 4; ++h)
                o << ind << "b2_st4_cs(o" << k << " + c + " << 4 * h << ", y" << k << " + "
                  << 4 * h << ");\n";
        else
            o << ind << "_Pragma(\"unroll\") for (int e = 0; e < V; ++e) o" << k
              << "[(c + e) * p.out_sc[" << k << "]] = y" << k << "[e];\n";
        return;
    }
    o << ind << "{ int m[V];\n"
      << ind << "  _Pragma(\"unroll\") for (int e = 0; e < V; ++e) { m[e] = b2_f32_to_i16(y" << k
      << "[e] * q" << k << ", fstat" << k << "); }\n";
    if (planes && pl.vec)
        o << ind << "  b2_st" << pl.V << "_planes(o" << k << " + c, p.out_plane[" << k << "], m); }\n";
    else if (planes)
        o << ind << "  _Pragma(\"unroll\") for (int e = 0; e < V; ++e) { const b2_i64 at = (c + e) * p.out_sc["
          << k << "]; o" << k << "[at] = (unsigned char)(m[e] >> 8); o" << k << "[p.out_plane[" << k
          << "] + at] = (unsigned char)m[e]; } }\n";
    else if (pl.vec)
        o << ind << "  b2_st" << pl.V << "_i16(o" << k << " + c, m); }\n";
    else
        o << ind << "  _Pragma(\"unroll\") for (int e = 0; e < V; ++e) o" << k
          << "[(c + e) * p.out_sc[" << k << "]] = (short)m[e]; }\n";
}

// Final store of one reduction result `val` (arg reductions: the index as a float).
void emit_red_store(std::ostringstream& o, const b2_ew_program& p, int k, bool probe,
                    const std::string& val, const std::string& addr, const std::string& ind) {
    const b2_ew_tensor& t = p.out[k].t;
    if (is_flex(t.dtype)) {
        if (probe) {
            o << ind << "stat" << k << " = max(stat" << k << ", b2_absbits(" << val << "));\n";
        } else {
            o << ind << "{ const int m = b2_f32_to_i16(" << val << " * q" << k << ", fstat" << k
              << "); ((short*)p.out[" << k << "])[" << addr << "] = (short)m; }\n";
        }
    } else if (!probe) {
        o << ind << "((float*)p.out[" << k << "])[" << addr << "] = " << val << ";\n";
    }
}

void emit_prologue(std::ostringstream& o, const b2_ew_program& p, bool probe) {
    const int nres = p.n_out + p.n_red;
    for (int i = 0; i < p.n_in; ++i)
        if (p.in[i].dtype == B2_FLEX16)
            o << "    const float s" << i << " = p.flex_table[p.in_slot[" << i << "]].scale;\n";
    for (int k = 0; k < nres; ++k)
        if (is_flex(p.out[k].t.dtype)) {
            if (!probe)
                o << "    const float q" << k << " = p.flex_table[p.out_slot[" << k
                  << "]].inv_scale;\n";
            o << "    int stat" << k << " = 0;\n    float fstat" << k << " = 0.0f;\n";
        }
    for (int i = 0; i < p.n_const; ++i)
        o << "    const float k" << i << " = p.consts[" << i << "];\n";
    // 1/step and step of the results that a requant op refers to
    unsigned seen = 0;
    for (int i = 0; i < p.n_ops; ++i)
        if (p.ops[i].opcode == B2_OP_REQUANT && !((seen >> p.ops[i].b) & 1u)) {
            const int k = p.ops[i].b;
            seen |= 1u << k;
            o << "    const float rq" << k << " = p.flex_table[p.out_slot[" << k << "]].inv_scale;\n"
              << "    const float rs" << k << " = p.flex_table[p.out_slot[" << k << "]].scale;\n";
        }
}

void emit_finalize(std::ostringstream& o, const b2_ew_program& p, bool probe) {
    const int nres = p.n_out + p.n_red;
        o << "extern \"C\" __global__ void __launch_bounds__(THREADS) b2_ew_finalize(const b2_ew_args p) {\n";
        o << "    __shared__ float smem[64];\n";
        emit_prologue(o, p, probe);
        o << "    const b2_i64 rows = p.A * p.B;\n"
          << "    const b2_i64 r = (b2_i64)blockIdx.x * THREADS + threadIdx.x;\n"
          << "    if (r < rows) {\n"
          << "        const b2_i64 a_idx = r / p.B, b_idx = r - a_idx * p.B;\n";
        for (int k = p.n_out; k < nres; ++k) {
            const std::string rn = red_name(p.out[k].redop);
            o << "        { float acc = b2_red_init<" << rn << ">();\n"
              << "          for (int s = 0; s < p.nsplit; ++s) acc = b2_red_comb<" << rn
              << ">(acc, p.scratch[((b2_i64)s * rows + r) * NRED + " << (k - p.n_out) << "]);\n";
            const std::string addr = "a_idx * p.out_sa[" + std::to_string(k) +
                                     "] + b_idx * p.out_sb[" + std::to_string(k) + "]";
            emit_red_store(o, p, k, probe, "acc", addr, "          ");
            o << "        }\n";
        }
        o << "    }\n";
        for (int k = p.n_out; k < nres; ++k)
            if (is_flex(p.out[k].t.dtype))
                o << "    b2_block_stat(max(stat" << k << ", b2_stat_to_int(fstat" << k
                  << ")), p.flex_stats + p.out_slot[" << k << "], reinterpret_cast<int*>(smem));\n";
        o << "}\n";
    }

int generate(const b2_ew_program& p, const Plan& pl, bool probe, std::string* out_src,
             bool* has_finalize) {
    std::ostringstream o;
    const int nres = p.n_out + p.n_red;
    const bool split = pl.nsplit > 1;
    *has_finalize = split;
    o << kDeviceHeader << "\n";
    o << "#define V " << pl.V << "\n#define THREADS " << kThreads << "\n#define GROUP "
      << pl.group << "\n#define NRED " << (p.n_red > 0 ? p.n_red : 1) << "\n";
    o << "extern \"C\" __global__ void __launch_bounds__(THREADS, " << pl.minb << ") b2_ew_main(const b2_ew_args p) {\n";
    o << "    __shared__ float smem[64];\n";
    // programmatic dependent launch: nothing above this line touches global memory; the next
    // kernel of the stream may be scheduled while this grid drains
    o << "    asm volatile(\"griddepcontrol.wait;\" ::: \"memory\");\n"
      << "    asm volatile(\"griddepcontrol.launch_dependents;\" ::: \"memory\");\n";
    emit_prologue(o, p, probe);

    if (p.reduce_mode != B2_REDUCE_B) {
        o << "    const b2_i64 rows = p.A * p.B;\n"
          << "    const b2_i64 chunks = p.C / V;\n"
          << "    const int grp = threadIdx.x / GROUP, gl = threadIdx.x % GROUP;\n"
          << "    const int RPC = THREADS / GROUP;\n"
          << "    for (b2_i64 r = (b2_i64)blockIdx.y * RPC + grp; r < rows; r += (b2_i64)gridDim.y * RPC) {\n"
          << "        const b2_i64 a_idx = r / p.B, b_idx = r - a_idx * p.B;\n";
        for (int i = 0; i < p.n_in; ++i) {
            const char* ct = ctype(p.in[i].dtype);
            o << "        const " << ct << "* in" << i << " = (const " << ct << "*)p.in[" << i
              << "] + a_idx * p.in_sa[" << i << "] + b_idx * p.in_sb[" << i << "];\n";
            if (p.in[i].sc == 0) {
                o << "        const float xb" << i << " = ";
                if (p.in[i].dtype == B2_FLEX16) o << "s" << i << " * (float)";
                o << "in" << i << "[0];\n";
            }
        }
        if (!probe)
            for (int k = 0; k < p.n_out; ++k) {
                const char* ct = ctype(p.out[k].t.dtype);
                o << "        " << ct << "* o" << k << " = (" << ct << "*)p.out[" << k
                  << "] + a_idx * p.out_sa[" << k << "] + b_idx * p.out_sb[" << k << "];\n";
            }
        for (int k = p.n_out; k < nres; ++k) {
            o << "        float acc" << k << " = b2_red_init<" << red_name(p.out[k].redop)
              << ">();\n";
            if (is_arg(p.out[k].redop)) o << "        int idx" << k << " = 0x7fffffff;\n";
        }
        o << "        b2_i64 j = (b2_i64)blockIdx.x * GROUP + gl;\n"
          << "        const b2_i64 jstep = (b2_i64)gridDim.x * GROUP;\n";
        for (int i = 0; i < p.n_in; ++i)
            if (prefetchable(p.in[i], pl))
                o << "        " << raw_type(p.in[i].dtype, pl.V) << " w" << i << " = {}, n" << i
                  << " = {};\n";
        if (pl.prefetch) {
            o << "        if (j < chunks) {\n";
            emit_raw_loads(o, p, pl, "w", "j", "            ");
            o << "        }\n";
        }
        o << "        for (; j < chunks; j += jstep) {\n"
          << "            const b2_i64 c = j * V;\n";
        if (pl.prefetch) {
            o << "            if (j + jstep < chunks) {\n";
            emit_raw_loads(o, p, pl, "n", "j + jstep", "                ");
            o << "            }\n";
        } else {
            emit_raw_loads(o, p, pl, "w", "j", "            ");
        }
        emit_loads(o, p, pl, "            ");
        for (int k = 0; k < p.n_out; ++k) o << "            float y" << k << "[V];\n";
        o << "            _Pragma(\"unroll\") for (int e = 0; e < V; ++e) {\n";
        {
            std::ostringstream body;
            if (emit_body(body, p, pl, probe)) return b2::fail(B2_ERR_INVALID, "unknown elementwise opcode");
            o << body.str();
        }
        for (int k = 0; k < p.n_out; ++k)
            o << "            y" << k << "[e] = " << reg(p.out[k].reg) << ";\n";
        for (int k = p.n_out; k < nres; ++k) {
            const int op = p.out[k].redop;
            if (is_arg(op))
                o << "            b2_arg_comb<" << red_name(op) << ">(acc" << k << ", idx" << k
                  << ", " << reg(p.out[k].reg) << ", (int)(c + e));\n";
            else
                o << "            acc" << k << " = b2_red_comb<" << red_name(op) << ">(acc" << k
                  << ", " << reg(p.out[k].reg) << ");\n";
        }
        o << "            }\n";
        for (int k = 0; k < p.n_out; ++k) emit_store(o, p, pl, k, probe, "            ");
        if (pl.prefetch)
            for (int i = 0; i < p.n_in; ++i)
                if (prefetchable(p.in[i], pl)) o << "            w" << i << " = n" << i << ";\n";
        o << "        }\n";
        // row epilogue
        for (int k = p.n_out; k < nres; ++k) {
            const int op = p.out[k].redop;
            const std::string rn = red_name(op);
            if (pl.group == 32) {
                if (is_arg(op))
                    o << "        b2_warp_reduce_arg<" << rn << ">(acc" << k << ", idx" << k << ");\n";
                else
                    o << "        acc" << k << " = b2_warp_reduce<" << rn << ">(acc" << k << ");\n";
            } else {
                if (is_arg(op))
                    o << "        b2_block_reduce_arg<" << rn << ">(acc" << k << ", idx" << k
                      << ", smem);\n";
                else
                    o << "        acc" << k << " = b2_block_reduce<" << rn << ">(acc" << k
                      << ", smem);\n";
            }
        }
        if (p.n_red > 0) {
            o << "        if (gl == 0) {\n";
            for (int k = p.n_out; k < nres; ++k) {
                if (split) {
                    o << "            p.scratch[((b2_i64)blockIdx.x * rows + r) * NRED + "
                      << (k - p.n_out) << "] = acc" << k << ";\n";
                } else {
                    const std::string val = is_arg(p.out[k].redop)
                                                ? "(float)idx" + std::to_string(k)
                                                : "acc" + std::to_string(k);
                    const std::string addr = "a_idx * p.out_sa[" + std::to_string(k) +
                                             "] + b_idx * p.out_sb[" + std::to_string(k) + "]";
                    emit_red_store(o, p, k, probe, val, addr, "            ");
                }
            }
            o << "        }\n";
        }
        o << "    }\n";
    } else {
        // REDUCE_B: threads run along C, every thread walks the B axis.
        o << "    const b2_i64 chunks = p.C / V;\n"
          << "    for (b2_i64 a_idx = blockIdx.y; a_idx < p.A; a_idx += gridDim.y)\n"
          << "    for (b2_i64 j = (b2_i64)blockIdx.x * THREADS + threadIdx.x; j < chunks; "
             "j += (b2_i64)gridDim.x * THREADS) {\n"
          << "        const b2_i64 c = j * V;\n";
        for (int k = p.n_out; k < nres; ++k) {
            o << "        float acc" << k << "[V];\n";
            if (is_arg(p.out[k].redop)) o << "        int idx" << k << "[V];\n";
            o << "        _Pragma(\"unroll\") for (int e = 0; e < V; ++e) { acc" << k
              << "[e] = b2_red_init<" << red_name(p.out[k].redop) << ">();";
            if (is_arg(p.out[k].redop)) o << " idx" << k << "[e] = 0x7fffffff;";
            o << " }\n";
        }
        o << "        for (b2_i64 b_idx = 0; b_idx < p.B; ++b_idx) {\n";
        for (int i = 0; i < p.n_in; ++i) {
            const char* ct = ctype(p.in[i].dtype);
            o << "            const " << ct << "* in" << i << " = (const " << ct << "*)p.in[" << i
              << "] + a_idx * p.in_sa[" << i << "] + b_idx * p.in_sb[" << i << "];\n";
            if (p.in[i].sc == 0) {
                o << "            const float xb" << i << " = ";
                if (p.in[i].dtype == B2_FLEX16) o << "s" << i << " * (float)";
                o << "in" << i << "[0];\n";
            }
        }
        if (!probe)
            for (int k = 0; k < p.n_out; ++k) {
                const char* ct = ctype(p.out[k].t.dtype);
                o << "            " << ct << "* o" << k << " = (" << ct << "*)p.out[" << k
                  << "] + a_idx * p.out_sa[" << k << "] + b_idx * p.out_sb[" << k << "];\n";
            }
        for (int i = 0; i < p.n_in; ++i)
            if (prefetchable(p.in[i], pl))
                o << "            " << raw_type(p.in[i].dtype, pl.V) << " w" << i << ";\n";
        emit_raw_loads(o, p, pl, "w", "j", "            ");
        emit_loads(o, p, pl, "            ");
        for (int k = 0; k < p.n_out; ++k) o << "            float y" << k << "[V];\n";
        o << "            _Pragma(\"unroll\") for (int e = 0; e < V; ++e) {\n";
        {
            std::ostringstream body;
            if (emit_body(body, p, pl, probe)) return b2::fail(B2_ERR_INVALID, "unknown elementwise opcode");
            o << body.str();
        }
        for (int k = 0; k < p.n_out; ++k)
            o << "            y" << k << "[e] = " << reg(p.out[k].reg) << ";\n";
        for (int k = p.n_out; k < nres; ++k) {
            const int op = p.out[k].redop;
            if (is_arg(op))
                o << "            b2_arg_comb<" << red_name(op) << ">(acc" << k << "[e], idx" << k
                  << "[e], " << reg(p.out[k].reg) << ", (int)b_idx);\n";
            else
                o << "            acc" << k << "[e] = b2_red_comb<" << red_name(op) << ">(acc" << k
                  << "[e], " << reg(p.out[k].reg) << ");\n";
        }
        o << "            }\n";
        for (int k = 0; k < p.n_out; ++k) emit_store(o, p, pl, k, probe, "            ");
        o << "        }\n";
        for (int k = p.n_out; k < nres; ++k) {
            o << "        _Pragma(\"unroll\") for (int e = 0; e < V; ++e) {\n";
            const std::string val = is_arg(p.out[k].redop)
                                        ? "(float)idx" + std::to_string(k) + "[e]"
                                        : "acc" + std::to_string(k) + "[e]";
            const std::string addr = "a_idx * p.out_sa[" + std::to_string(k) +
                                     "] + (c + e) * p.out_sc[" + std::to_string(k) + "]";
            emit_red_store(o, p, k, probe, val, addr, "            ");
            o << "        }\n";
        }
        o << "    }\n";
    }
    // flex statistics: one atomic per CTA and output.  In split mode the reduction outputs are
    // produced (and counted) by the finalize kernel.
    {
        const int nstat = split ? p.n_out : nres;
        for (int k = 0; k < nstat; ++k)
            if (is_flex(p.out[k].t.dtype))
                o << "    b2_block_stat(max(stat" << k << ", b2_stat_to_int(fstat" << k
                  << ")), p.flex_stats + p.out_slot[" << k << "], reinterpret_cast<int*>(smem));\n";
    }
    o << "}\n";

    if (split) emit_finalize(o, p, probe);
    *out_src = o.str();
    return B2_OK;
}


// ---- staged variant: REDUCE_NONE / REDUCE_C with one CTA per row segment -----------------------
// Tiles of THREADS*V contiguous elements of every full-size input are copied global -> shared by
// one thread with cp.async.bulk (completion counted on an mbarrier), STAGES tiles ahead of the
// compute, so the bytes in flight per SM do not depend on registers or occupancy.
int generate_staged(const b2_ew_program& p, const Plan& pl, bool probe, std::string* out_src,
                    bool* has_finalize) {
    std::ostringstream o;
    const int nres = p.n_out + p.n_red;
    const bool split = pl.nsplit > 1;
    *has_finalize = split;
    o << kDeviceHeader << "\n";
    o << "#define V " << pl.V << "\n#define THREADS " << kThreads << "\n#define GROUP " << kThreads
      << "\n#define NRED " << (p.n_red > 0 ? p.n_red : 1) << "\n#define STAGES " << pl.stages
      << "\n#define STAGE_BYTES " << pl.stage_bytes << "\n";
    // byte offset of each staged input inside a stage
    std::vector<int> off(p.n_in, -1);
    int cur = 0;
    for (int i = 0; i < p.n_in; ++i)
        if (prefetchable(p.in[i], pl)) {
            off[i] = cur;
            cur += kThreads * pl.V * (p.in[i].dtype == B2_FLEX16 ? 2 : 4);
        }
    o << "extern \"C\" __global__ void __launch_bounds__(THREADS, " << pl.minb << ") b2_ew_main(const b2_ew_args p) {\n"
      << "    __shared__ float smem[64];\n"
      << "    __shared__ unsigned long long full_bar[STAGES];\n"
      << "    extern __shared__ __align__(128) unsigned char stage_mem[];\n";
    // programmatic dependent launch: nothing above this line touches global memory; the next
    // kernel of the stream may be scheduled while this grid drains
    o << "    asm volatile(\"griddepcontrol.wait;\" ::: \"memory\");\n"
      << "    asm volatile(\"griddepcontrol.launch_dependents;\" ::: \"memory\");\n";
    emit_prologue(o, p, probe);
    o << "    const int tid = threadIdx.x;\n"
      << "    const int rows = (int)(p.A * p.B), Bn = (int)p.B;\n"
      << "    const int chunks = (int)(p.C / V);\n"
      << "    const int tpr = (chunks + THREADS - 1) / THREADS;\n"
      << "    const int n_t = tpr > (int)blockIdx.x ? (tpr - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;\n"
      << "    const int n_r = rows > (int)blockIdx.y ? (rows - (int)blockIdx.y + (int)gridDim.y - 1) / (int)gridDim.y : 0;\n"
      << "    const int n_it = n_t * n_r;\n"
      << "    if (tid == 0) {\n"
      << "        for (int s = 0; s < STAGES; ++s) b2_mbar_init(&full_bar[s], 1);\n"
      << "        b2_mbar_init_fence();\n"
      << "    }\n"
      << "    __syncthreads();\n"
      // producer state (thread 0 only): next tile to issue
      << "    int p_it = 0, p_ti = 0, p_r = blockIdx.y;\n"
      << "    auto issue = [&]() {\n"
      << "        const int s = p_it % STAGES;\n"
      << "        const int t = (int)blockIdx.x + p_ti * (int)gridDim.x;\n"
      << "        const int a_i = p_r / Bn, b_i = p_r - a_i * Bn;\n"
      << "        const b2_i64 c0 = (b2_i64)t * (THREADS * V);\n"
      << "        b2_i64 n = p.C - c0; if (n > THREADS * V) n = THREADS * V;\n"
      << "        unsigned char* dst = stage_mem + s * STAGE_BYTES;\n";
    {
        int bytes_per_elem = 0;
        for (int i = 0; i < p.n_in; ++i)
            if (off[i] >= 0) bytes_per_elem += p.in[i].dtype == B2_FLEX16 ? 2 : 4;
        o << "        b2_mbar_expect_tx(&full_bar[s], (unsigned)(n * " << bytes_per_elem << "));\n";
    }
    for (int i = 0; i < p.n_in; ++i)
        if (off[i] >= 0) {
            const char* ct = ctype(p.in[i].dtype);
            o << "        b2_bulk_g2s(dst + " << off[i] << ", (const " << ct << "*)p.in[" << i
              << "] + (b2_i64)a_i * p.in_sa[" << i << "] + (b2_i64)b_i * p.in_sb[" << i
              << "] + c0, (unsigned)(n * sizeof(" << ct << ")), &full_bar[s]);\n";
        }
    o << "        ++p_it;\n"
      << "        if (++p_ti == n_t) { p_ti = 0; p_r += gridDim.y; }\n"
      << "    };\n"
      << "    if (tid == 0) { for (int k = 0; k < STAGES - 1 && k < n_it; ++k) issue(); }\n";
    for (int k = p.n_out; k < nres; ++k) {
        o << "    float acc" << k << " = b2_red_init<" << red_name(p.out[k].redop) << ">();\n";
        if (is_arg(p.out[k].redop)) o << "    int idx" << k << " = 0x7fffffff;\n";
    }
    o << "    int ti = 0, r = blockIdx.y;\n"
      << "    int a_idx = r / Bn, b_idx = r - a_idx * Bn;\n"
      << "    bool timed_out = false;\n"
      << "    for (int it = 0; it < n_it; ++it) {\n"
      << "        const int s = it % STAGES;\n"
      << "        if (tid == 0 && it + STAGES - 1 < n_it) { b2_proxy_fence(); issue(); }\n"
      << "        const int t = (int)blockIdx.x + ti * (int)gridDim.x;\n"
      << "        const b2_i64 c = ((b2_i64)t * THREADS + tid) * V;\n"
      << "        const bool active = c < p.C;\n"
      << "        if (!b2_mbar_wait(&full_bar[s], (unsigned)((it / STAGES) & 1))) timed_out = true;\n"
      << "        const unsigned char* src = stage_mem + s * STAGE_BYTES;\n";
    for (int i = 0; i < p.n_in; ++i)
        if (off[i] >= 0) {
            const int esz = p.in[i].dtype == B2_FLEX16 ? 2 : 4;
            o << "        " << raw_type(p.in[i].dtype, pl.V) << " w" << i << " = {};\n"
              << "        if (active) b2_lds_raw(src + " << off[i] << " + tid * " << pl.V * esz
              << ", w" << i << ");\n";
        }
    o << "        __syncthreads();   // stage s may be refilled from the next iteration on\n"
      << "        if (active) {\n";
    for (int i = 0; i < p.n_in; ++i)
        if (p.in[i].sc == 0) {
            const char* ct = ctype(p.in[i].dtype);
            o << "            const float xb" << i << " = ";
            if (p.in[i].dtype == B2_FLEX16) o << "s" << i << " * (float)";
            o << "((const " << ct << "*)p.in[" << i << "])[(b2_i64)a_idx * p.in_sa[" << i
              << "] + (b2_i64)b_idx * p.in_sb[" << i << "]];\n";
        }
    if (!probe)
        for (int k = 0; k < p.n_out; ++k) {
            const char* ct = ctype(p.out[k].t.dtype);
            o << "            " << ct << "* o" << k << " = (" << ct << "*)p.out[" << k
              << "] + (b2_i64)a_idx * p.out_sa[" << k << "] + (b2_i64)b_idx * p.out_sb[" << k
              << "];\n";
        }
    emit_loads(o, p, pl, "            ");
    for (int k = 0; k < p.n_out; ++k) o << "            float y" << k << "[V];\n";
    o << "            _Pragma(\"unroll\") for (int e = 0; e < V; ++e) {\n";
    {
        std::ostringstream body;
        if (emit_body(body, p, pl, probe)) return b2::fail(B2_ERR_INVALID, "unknown elementwise opcode");
        o << body.str();
    }
    for (int k = 0; k < p.n_out; ++k)
        o << "            y" << k << "[e] = " << reg(p.out[k].reg) << ";\n";
    for (int k = p.n_out; k < nres; ++k) {
        const int op = p.out[k].redop;
        if (is_arg(op))
            o << "            b2_arg_comb<" << red_name(op) << ">(acc" << k << ", idx" << k << ", "
              << reg(p.out[k].reg) << ", (int)(c + e));\n";
        else
            o << "            acc" << k << " = b2_red_comb<" << red_name(op) << ">(acc" << k << ", "
              << reg(p.out[k].reg) << ");\n";
    }
    o << "            }\n";
    for (int k = 0; k < p.n_out; ++k) emit_store(o, p, pl, k, probe, "            ");
    o << "        }\n"
      << "        if (++ti == n_t) {\n";
    // end of this CTA's part of the row: reduce and store
    for (int k = p.n_out; k < nres; ++k) {
        const int op = p.out[k].redop;
        const std::string rn = red_name(op);
        if (is_arg(op))
            o << "            b2_block_reduce_arg<" << rn << ">(acc" << k << ", idx" << k << ", smem);\n";
        else
            o << "            acc" << k << " = b2_block_reduce<" << rn << ">(acc" << k << ", smem);\n";
    }
    if (p.n_red > 0) {
        o << "            if (tid == 0) {\n";
        for (int k = p.n_out; k < nres; ++k) {
            if (split) {
                o << "                p.scratch[((b2_i64)blockIdx.x * rows + r) * NRED + "
                  << (k - p.n_out) << "] = acc" << k << ";\n";
            } else {
                const std::string val = is_arg(p.out[k].redop) ? "(float)idx" + std::to_string(k)
                                                                : "acc" + std::to_string(k);
                const std::string addr = "(b2_i64)a_idx * p.out_sa[" + std::to_string(k) +
                                         "] + (b2_i64)b_idx * p.out_sb[" + std::to_string(k) + "]";
                emit_red_store(o, p, k, probe, val, addr, "                ");
            }
        }
        o << "            }\n";
        for (int k = p.n_out; k < nres; ++k) {
            o << "            acc" << k << " = b2_red_init<" << red_name(p.out[k].redop) << ">();\n";
            if (is_arg(p.out[k].redop)) o << "            idx" << k << " = 0x7fffffff;\n";
        }
    }
    o << "            ti = 0; r += gridDim.y;\n"
      << "            a_idx = r / Bn; b_idx = r - a_idx * Bn;\n"
      << "        }\n"
      << "    }\n"
      << "    if (timed_out && p.status) atomicExch(p.status, 1);\n";
    {
        const int nstat = split ? p.n_out : nres;
        for (int k = 0; k < nstat; ++k)
            if (is_flex(p.out[k].t.dtype))
                o << "    b2_block_stat(max(stat" << k << ", b2_stat_to_int(fstat" << k
                  << ")), p.flex_stats + p.out_slot[" << k << "], reinterpret_cast<int*>(smem));\n";
    }
    o << "}\n";
    if (split) emit_finalize(o, p, probe);
    *out_src = o.str();
    return B2_OK;
}

bool vector_ok(const b2_ew_program& p, int V) {
    if (p.C % V) return false;
    auto ok = [&](const b2_ew_tensor& t) {
        if (t.sc == 0) return true;
        if (t.sc != 1) return false;
        if (p.A > 1 && t.sa % V) return false;
        if (p.B > 1 && t.sb % V) return false;
        return true;
    };
    for (int i = 0; i < p.n_in; ++i) if (!ok(p.in[i])) return false;
    for (int k = 0; k < p.n_out; ++k) {
        if (p.out[k].t.sc != 1) return false;
        if (!ok(p.out[k].t)) return false;
    }
    return true;
}

Plan make_plan(const b2_ew_program& p, bool want_vec) {
    Plan pl;
    bool any16 = false;
    for (int i = 0; i < p.n_in; ++i) any16 |= p.in[i].dtype == B2_FLEX16;
    for (int k = 0; k < p.n_out; ++k) any16 |= is_flex(p.out[k].t.dtype);
    pl.V = 1;
    pl.vec = false;
    if (want_vec) {
        if (any16 && vector_ok(p, 8)) { pl.V = 8; pl.vec = true; }
        else if (vector_ok(p, 4)) { pl.V = 4; pl.vec = true; }
    }
    const long long rows = p.A * p.B;
    const long long chunks = p.C / pl.V;
    const int wave = kSMs * 8;
    if (p.reduce_mode == B2_REDUCE_NONE) {
        long long gx = (chunks + kThreads - 1) / kThreads;
        if (gx < 1) gx = 1;
        if (gx > 64) gx = 64;
        long long gy = rows;
        long long cap = (2LL * wave + gx - 1) / gx;
        if (gy > cap) gy = cap;
        if (rows == 1) { gx = (chunks + kThreads - 1) / kThreads; if (gx > 2 * wave) gx = 2 * wave; if (gx < 1) gx = 1; }
        pl.group = kThreads;
        pl.grid = dim3((unsigned)gx, (unsigned)gy, 1);
    } else if (p.reduce_mode == B2_REDUCE_C) {
        bool has_arg = false;
        for (int k = p.n_out; k < p.n_out + p.n_red; ++k) has_arg |= is_arg(p.out[k].redop);
        if (chunks <= 64) {
            pl.group = 32;
            long long gy = (rows + 7) / 8;
            if (gy > 65535) gy = 65535;
            pl.grid = dim3(1, (unsigned)gy, 1);
        } else {
            pl.group = kThreads;
            long long gy = rows > 65535 ? 65535 : rows;
            pl.nsplit = 1;
            if (!has_arg && rows < 2 * kSMs && chunks >= 8LL * kThreads) {
                long long want = (4LL * kSMs + rows - 1) / rows;
                long long maxs = chunks / (4LL * kThreads);
                long long ns = want < maxs ? want : maxs;
                if (ns > 1024) ns = 1024;
                if (ns > 1) pl.nsplit = (int)ns;
            }
            pl.grid = dim3((unsigned)pl.nsplit, (unsigned)gy, 1);
        }
    } else {
        long long gx = (chunks + kThreads - 1) / kThreads;
        if (gx < 1) gx = 1;
        long long gy = p.A > 65535 ? 65535 : p.A;
        pl.group = kThreads;
        pl.grid = dim3((unsigned)gx, (unsigned)gy, 1);
    }
    {
        const char* pf = getenv("B2_EW_PREFETCH");
        pl.prefetch = pf && pf[0] == '1';
    }
    {
        const char* mb = getenv("B2_EW_MINB");
        pl.minb = mb ? atoi(mb) : 5;
        if (pl.minb < 1) pl.minb = 1;
        if (pl.minb > 8) pl.minb = 8;
    }
    // staged variant: full-size inputs go global -> shared by bulk async copies
    const char* env = getenv("B2_EW_STAGED");
    const bool allow = env && env[0] == '1';   // off by default: measured slower than plain loads
    if (allow && pl.vec && p.reduce_mode != B2_REDUCE_B && pl.group == kThreads &&
        rows < (1LL << 30) && chunks < (1LL << 30)) {
        int bytes = 0;
        for (int i = 0; i < p.n_in; ++i)
            if (prefetchable(p.in[i], pl)) bytes += kThreads * pl.V * (p.in[i].dtype == B2_FLEX16 ? 2 : 4);
        const long long tpr = (chunks + kThreads - 1) / kThreads;
        if (bytes > 0 && rows * tpr >= 4) {
            pl.staged = true;
            pl.stage_bytes = bytes;
            pl.stages = bytes * 4 <= 64 * 1024 ? 4 : 3;
            if (bytes * pl.stages > 200 * 1024) pl.staged = false;
        }
        if (pl.staged) {
            // CTAs resident per SM by shared memory; a few waves of persistent CTAs
            int per_sm = (200 * 1024) / (bytes * pl.stages);
            if (per_sm > 6) per_sm = 6;
            if (per_sm < 1) per_sm = 1;
            const long long want = 4LL * kSMs * per_sm;
            if (p.reduce_mode == B2_REDUCE_C) {
                long long gy = rows < want ? rows : want;
                pl.grid = dim3((unsigned)pl.nsplit, (unsigned)gy, 1);
            } else {
                long long gx = tpr < 64 ? tpr : 64;
                if (rows == 1) gx = tpr < want ? tpr : want;
                long long gy = (want + gx - 1) / gx;
                if (gy > rows) gy = rows;
                pl.grid = dim3((unsigned)gx, (unsigned)gy, 1);
            }
        }
    }
    return pl;
}

}  // namespace

struct b2_ew_kernel {
    b2_ew_program prog;
    // [vec?][probe?]
    Module* mod[2][2] = {{nullptr, nullptr}, {nullptr, nullptr}};
    Plan plan[2];
    std::string src[2][2];
    bool can_vec = false;
};

namespace {

int validate(const b2_ew_program& p) {
    B2_REQUIRE(p.A >= 1 && p.B >= 1 && p.C >= 1, "iteration space must be at least 1x1x1");
    B2_REQUIRE(p.n_in >= 0 && p.n_in <= B2_EW_MAX_IN, "too many inputs (%d)", p.n_in);
    B2_REQUIRE(p.n_const >= 0 && p.n_const <= B2_EW_MAX_CONST, "too many constants");
    B2_REQUIRE(p.n_ops >= 0 && p.n_ops <= B2_EW_MAX_OPS, "too many ops (%d)", p.n_ops);
    B2_REQUIRE(p.n_out >= 0 && p.n_red >= 0 && p.n_out + p.n_red >= 1 &&
               p.n_out + p.n_red <= B2_EW_MAX_OUT, "bad number of results");
    B2_REQUIRE(p.reduce_mode >= B2_REDUCE_NONE && p.reduce_mode <= B2_REDUCE_B, "bad reduce mode");
    B2_REQUIRE((p.n_red > 0) == (p.reduce_mode != B2_REDUCE_NONE),
               "reductions and reduce_mode disagree");
    const int nreg = p.n_in + p.n_const + p.n_ops;
    for (int i = 0; i < p.n_ops; ++i) {
        const int lim = p.n_in + p.n_const + i;
        B2_REQUIRE(p.ops[i].a >= 0 && p.ops[i].a < lim, "op %d reads an undefined register", i);
        if (p.ops[i].opcode == B2_OP_REQUANT)
            B2_REQUIRE(p.ops[i].b >= 0 && p.ops[i].b < p.n_out && is_flex(p.out[p.ops[i].b].t.dtype),
                       "op %d: requant needs an elementwise flex16 result of this program", i);
        else if (p.ops[i].opcode >= B2_OP_ADD && p.ops[i].opcode != B2_OP_ONEHOT)
            B2_REQUIRE(p.ops[i].b >= 0 && p.ops[i].b < lim, "op %d reads an undefined register", i);
    }
    for (int k = 0; k < p.n_out + p.n_red; ++k) {
        B2_REQUIRE(p.out[k].reg >= 0 && p.out[k].reg < nreg, "result %d reads an undefined register", k);
        B2_REQUIRE(p.out[k].t.dtype == B2_F32 || is_flex(p.out[k].t.dtype), "bad result dtype");
        B2_REQUIRE(p.out[k].t.dtype != B2_FLEX16_PLANES || k < p.n_out,
                   "byte planes are for elementwise results only");
        if (is_flex(p.out[k].t.dtype))
            B2_REQUIRE(p.out[k].t.flex_slot >= 0, "flex result %d has no slot", k);
        if (k >= p.n_out)
            B2_REQUIRE(p.out[k].redop >= B2_RED_SUM && p.out[k].redop <= B2_RED_ARGMIN, "bad redop");
    }
    for (int i = 0; i < p.n_in; ++i) {
        B2_REQUIRE(p.in[i].dtype == B2_F32 || p.in[i].dtype == B2_FLEX16, "bad input dtype");
        if (p.in[i].dtype == B2_FLEX16)
            B2_REQUIRE(p.in[i].flex_slot >= 0, "flex input %d has no slot", i);
    }
    return B2_OK;
}

int ensure_variant(b2_ew_kernel* k, int vec, int probe) {
    if (k->mod[vec][probe]) return B2_OK;
    bool has_final = false;
    std::string src;
    const Plan& pl = k->plan[vec];
    int rc = pl.staged ? generate_staged(k->prog, pl, probe != 0, &src, &has_final)
                       : generate(k->prog, pl, probe != 0, &src, &has_final);
    if (rc) return rc;
    rc = compile_source(src, has_final, &k->mod[vec][probe]);
    if (rc) return rc;
    if (pl.staged) {
        const int dyn = pl.stages * pl.stage_bytes;
        if (dyn > 40 * 1024)
            B2_CUDA(cudaFuncSetAttribute((const void*)k->mod[vec][probe]->main,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, dyn));
    }
    k->src[vec][probe] = src;
    return B2_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

extern "C" int b2_set_nvrtc_path(const char* path) {
    std::lock_guard<std::mutex> lock(g_mutex);
    g_nvrtc_dir = path ? path : "";
    return B2_OK;
}

extern "C" int b2_ew_check(const b2_ew_program* prog, int vec, int probe, char* source,
                           size_t source_cap) {
    B2_REQUIRE(prog, "null argument");
    int rc = validate(*prog);
    if (rc) return rc;
    Plan pl = make_plan(*prog, vec != 0);
    std::string src;
    bool has_final = false;
    rc = pl.staged ? generate_staged(*prog, pl, probe != 0, &src, &has_final)
                   : generate(*prog, pl, probe != 0, &src, &has_final);
    if (rc) return rc;
    if (source && source_cap) {
        strncpy(source, src.c_str(), source_cap - 1);
        source[source_cap - 1] = '\0';
    }
    std::vector<char> cubin;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        rc = nvrtc_compile(src, &cubin);
    }
    return rc;
}

extern "C" int b2_ew_compile(const b2_ew_program* prog, b2_ew_kernel** out_kernel) {
    B2_REQUIRE(prog && out_kernel, "null argument");
    int rc = validate(*prog);
    if (rc) return rc;
    b2_ew_kernel* k = new b2_ew_kernel();
    k->prog = *prog;
    k->plan[0] = make_plan(*prog, false);
    k->plan[1] = make_plan(*prog, true);
    k->can_vec = k->plan[1].vec;
    rc = ensure_variant(k, k->can_vec ? 1 : 0, 0);
    if (rc) { delete k; return rc; }
    *out_kernel = k;
    return B2_OK;
}

extern "C" int b2_ew_scratch_bytes(const b2_ew_kernel* k, size_t* bytes) {
    B2_REQUIRE(k && bytes, "null argument");
    size_t need = 0;
    for (int v = 0; v < 2; ++v) {
        const Plan& pl = k->plan[v];
        if (pl.nsplit > 1) {
            size_t n = (size_t)pl.nsplit * (size_t)(k->prog.A * k->prog.B) * (size_t)k->prog.n_red *
                       sizeof(float);
            if (n > need) need = n;
        }
    }
    *bytes = need;
    return B2_OK;
}

extern "C" const char* b2_ew_source(const b2_ew_kernel* k) {
    if (!k) return "";
    for (int v = 1; v >= 0; --v)
        if (!k->src[v][0].empty()) return k->src[v][0].c_str();
    return "";
}

extern "C" int b2_ew_launch_count(const b2_ew_kernel* k) {
    if (!k) return 0;
    return k->plan[k->can_vec ? 1 : 0].nsplit > 1 ? 2 : 1;
}

namespace {
// The main kernel waits for the stream's earlier work itself (griddepcontrol.wait, its first
// statement), so it may be scheduled while the kernel before it drains.
cudaError_t launch_main(const void* func, dim3 grid, void** params, size_t dyn, cudaStream_t st) {
    static const bool plain = getenv("B2_EW_NO_PDL") != nullptr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = dyn; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = plain ? 0 : 1;
    return cudaLaunchKernelExC(&cfg, func, params);
}
}  // namespace

// What both launch entry points share: argument checks and the choice between the vector and the
// scalar variant (decided by the pointers' alignment), then the argument block and the launches.
namespace {
int check_launch(const b2_ew_kernel* k, const void* const* in, void* const* out,
                 const float* consts, const b2_flex_scale* flex_table, const int32_t* flex_stats,
                 int* vec_out) {
    B2_REQUIRE(k && (in || k->prog.n_in == 0) && out, "null argument");
    const b2_ew_program& p = k->prog;
    const int nres = p.n_out + p.n_red;
    bool any_flex = false;
    int vec = k->can_vec ? 1 : 0;
    for (int i = 0; i < p.n_in; ++i) {
        B2_REQUIRE(in[i], "input %d is null", i);
        any_flex |= p.in[i].dtype == B2_FLEX16;
        if (vec && p.in[i].sc == 1 && !aligned16(in[i])) vec = 0;
    }
    for (int q = 0; q < nres; ++q) {
        B2_REQUIRE(out[q], "result %d is null", q);
        any_flex |= is_flex(p.out[q].t.dtype);
        if (vec && q < p.n_out && !aligned16(out[q])) vec = 0;
    }
    if (any_flex) B2_REQUIRE(flex_table && flex_stats, "flex tensors need a scale table and stats");
    B2_REQUIRE(p.n_const == 0 || consts, "constants missing");
    *vec_out = vec;
    return B2_OK;
}

size_t scratch_need(const b2_ew_kernel* k, int vec) {
    const Plan& pl = k->plan[vec];
    const b2_ew_program& p = k->prog;
    return pl.nsplit > 1
        ? (size_t)pl.nsplit * (size_t)(p.A * p.B) * (size_t)p.n_red * sizeof(float) : 0;
}

int launch_variant(const b2_ew_kernel* k, int vec, const Module* m, const void* const* in,
                   void* const* out, const float* consts, const b2_flex_scale* flex_table,
                   int32_t* flex_stats, void* scratch, int32_t* status, unsigned fresh_mask,
                   void* stream) {
    const b2_ew_program& p = k->prog;
    const Plan& pl = k->plan[vec];
    const int nres = p.n_out + p.n_red;
    EwArgs a;
    memset(&a, 0, sizeof(a));
    a.A = p.A; a.B = p.B; a.C = p.C;
    for (int i = 0; i < p.n_in; ++i) {
        a.in[i] = in[i];
        a.in_sa[i] = p.in[i].sa; a.in_sb[i] = p.in[i].sb; a.in_sc[i] = p.in[i].sc;
        a.in_slot[i] = p.in[i].flex_slot;
    }
    for (int q = 0; q < nres; ++q) {
        a.out[q] = out[q];
        a.out_sa[q] = p.out[q].t.sa; a.out_sb[q] = p.out[q].t.sb; a.out_sc[q] = p.out[q].t.sc;
        a.out_slot[q] = p.out[q].t.flex_slot;
        a.out_plane[q] = p.out[q].t.plane_bytes;
    }
    for (int i = 0; i < p.n_const; ++i) a.consts[i] = consts[i];
    a.flex_table = flex_table;
    a.flex_stats = flex_stats;
    a.scratch = static_cast<float*>(scratch);
    a.status = status;
    a.nsplit = pl.nsplit;
    a.fresh_mask = fresh_mask;
    void* params[] = {&a};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t dyn = pl.staged ? (size_t)pl.stages * pl.stage_bytes : 0;
    B2_CUDA(launch_main((const void*)m->main, pl.grid, params, dyn, st));
    if (pl.nsplit > 1) {
        const long long rows = p.A * p.B;
        dim3 g((unsigned)((rows + kThreads - 1) / kThreads));
        B2_CUDA(cudaLaunchKernel((const void*)m->finalize, g, dim3(kThreads), params, 0, st));
    }
    return B2_OK;
}
}  // namespace

extern "C" int b2_ew_launch(b2_ew_kernel* k, const void* const* in, void* const* out,
                            const float* consts, const b2_flex_scale* flex_table,
                            int32_t* flex_stats, void* scratch, size_t scratch_bytes,
                            int32_t* status, int probe, void* stream) {
    int vec = 0;
    int rc = check_launch(k, in, out, consts, flex_table, flex_stats, &vec);
    if (rc) return rc;
    const unsigned fresh_mask = probe > 0 ? (unsigned)probe >> 1 : 0u;
    probe = probe ? 1 : 0;
    rc = ensure_variant(k, vec, probe);
    if (rc) return rc;
    const size_t need = scratch_need(k, vec);
    B2_REQUIRE(need == 0 || (scratch && scratch_bytes >= need),
               "split reduction needs %zu bytes of scratch, got %zu", need, scratch_bytes);
    return launch_variant(k, vec, k->mod[vec][probe], in, out, consts, flex_table, flex_stats,
                          scratch, status, fresh_mask, stream);
}

// ------------------------------------------------------------------------------------------------
// Launch with the library's own scratch: an entry point that allocates nothing.
//
// Who needs it: a host that cannot (or must not) call cudaMalloc when it discovers that a kernel
// wants scratch.  Two such hosts exist for this library: an embedding runtime that took the whole
// device for its own arena when it started, so that a later cudaMalloc fails or has to wait for
// that arena to give memory back; and a steady-state execution loop that was promised "no
// allocator calls", because cudaMalloc/cudaFree synchronise the device and would stall every
// stream in flight.  The only kernels here that use scratch are the split row reductions (a few
// very long rows shared by many CTAs, fp32 partials combined by b2_ew_finalize); this variant
// gives them a fixed array that lives in the library's device image instead of a caller buffer.
//
// Limits and rules:
//   * the array is B2_EW_BUILTIN_SCRATCH_BYTES (16 KiB) per device, held by every GPU that loads
//     the library until the process exits; a launch that needs more is refused with an error;
//   * the first call on a device looks the array's device address up (cudaGetSymbolAddress, with
//     that device current) and remembers it; make that first call outside any stream capture;
//   * all calls share the array and it keeps whatever the previous call left.  The split
//     reduction writes every partial before b2_ew_finalize reads it, so nothing has to be cleared
//     first -- but two such launches that overlap on the GPU (different streams) would overwrite
//     each other's partials: run them on one stream, or serialise them;
//   * no kernel is compiled or loaded here: the variant (aligned / unaligned pointers, probe) must
//     already exist, which b2_ew_compile guarantees for aligned pointers and probe == 0.
// ------------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_builtin_scratch[B2_EW_BUILTIN_SCRATCH_BYTES];

namespace {
const int kMaxDevices = 64;
void* g_builtin_scratch_ptr[kMaxDevices] = {nullptr};
std::mutex g_builtin_mutex;

// In host code `g_builtin_scratch` is only a handle for the symbol, not a device address: the
// address a kernel can use has to be asked for, per device.
int builtin_scratch_for_current_device(void** out) {
    int dev = -1;
    B2_CUDA(cudaGetDevice(&dev));
    B2_REQUIRE(dev >= 0 && dev < kMaxDevices, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_builtin_mutex);
    if (!g_builtin_scratch_ptr[dev]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_builtin_scratch);
        if (e != cudaSuccess || !p)
            return b2::fail(B2_ERR_CUDA, "cudaGetSymbolAddress(built-in scratch) failed: %s",
                            cudaGetErrorString(e));
        g_builtin_scratch_ptr[dev] = p;
    }
    *out = g_builtin_scratch_ptr[dev];
    return B2_OK;
}
}  // namespace

extern "C" int b2_ew_launch_builtin_scratch(b2_ew_kernel* k, const void* const* in,
                                            void* const* out, const float* consts,
                                            const b2_flex_scale* flex_table, int32_t* flex_stats,
                                            int32_t* status, int probe, void* stream) {
    int vec = 0;
    int rc = check_launch(k, in, out, consts, flex_table, flex_stats, &vec);
    if (rc) return rc;
    const unsigned fresh_mask = probe > 0 ? (unsigned)probe >> 1 : 0u;
    probe = probe ? 1 : 0;
    const Module* m = k->mod[vec][probe];
    B2_REQUIRE(m != nullptr,
               "this kernel variant (vector=%d, probe=%d) has not been compiled yet; the "
               "no-allocation launch never compiles or loads code -- run b2_ew_launch once with "
               "the same kind of pointers first", vec, probe);
    const size_t need = scratch_need(k, vec);
    B2_REQUIRE(need <= (size_t)B2_EW_BUILTIN_SCRATCH_BYTES,
               "this launch needs %zu bytes of scratch but the built-in scratch holds %zu; use "
               "b2_ew_launch with a caller buffer", need, (size_t)B2_EW_BUILTIN_SCRATCH_BYTES);
    void* scratch = nullptr;
    rc = builtin_scratch_for_current_device(&scratch);
    if (rc) return rc;
    return launch_variant(k, vec, m, in, out, consts, flex_table, flex_stats, scratch, status,
                          fresh_mask, stream);
}
