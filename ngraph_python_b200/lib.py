"""ctypes binding of libb200ng.so (the C ABI declared in include/b200ng.h).

There is no fallback: if the shared library is missing, import fails with instructions to build
it; if a call fails, `B200Error` carries the library's message.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libb200ng.so")

EW_MAX_IN, EW_MAX_OUT, EW_MAX_CONST, EW_MAX_OPS = 12, 6, 16, 96
F32, FLEX16, FLEX16_PLANES = 0, 1, 2
REDUCE_NONE, REDUCE_C, REDUCE_B = 0, 1, 2

OPCODES = {
    "assign": 0, "neg": 1, "abs": 2, "sqrt": 3, "sqr": 4, "exp": 5, "log": 6, "rcp": 7,
    "exp2": 8, "log2": 9, "sig": 10, "tanh": 11, "safelog": 12, "sgn": 13, "sin": 14, "cos": 15,
    "add": 32, "sub": 33, "mul": 34, "div": 35, "int_div": 36, "mod": 37, "eq": 38, "ne": 39,
    "lt": 40, "le": 41, "gt": 42, "ge": 43, "pow": 44, "minimum": 45, "maximum": 46, "onehot": 47,
    "requant": 48,      # (register, index of a flex16 result): the value as stored and read back
}
UNARY_OPS = frozenset(k for k, v in OPCODES.items() if v < 32) | {"onehot"}
REDOPS = {"sum": 0, "prod": 1, "max": 2, "min": 3, "argmax": 4, "argmin": 5}


class B200Error(RuntimeError):
    pass


class EwTensor(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("flex_slot", C.c_int32),
                ("sa", C.c_int64), ("sb", C.c_int64), ("sc", C.c_int64),
                ("plane_bytes", C.c_int64)]


class EwOp(C.Structure):
    _fields_ = [("opcode", C.c_int32), ("a", C.c_int32), ("b", C.c_int32)]


class EwResult(C.Structure):
    _fields_ = [("reg", C.c_int32), ("redop", C.c_int32), ("t", EwTensor)]


class ConvEpilogue(C.Structure):
    _fields_ = [("bias", C.c_void_p), ("slot_bias", C.c_int32),
                ("residual", C.c_void_p), ("slot_residual", C.c_int32),
                ("relu", C.c_int32), ("write_int16", C.c_int32),
                ("out_planes", C.c_void_p), ("plane_bytes", C.c_size_t)]


class EwProgram(C.Structure):
    _fields_ = [("A", C.c_int64), ("B", C.c_int64), ("C", C.c_int64),
                ("reduce_mode", C.c_int32),
                ("n_in", C.c_int32), ("n_const", C.c_int32), ("n_ops", C.c_int32),
                ("n_out", C.c_int32), ("n_red", C.c_int32),
                ("inp", EwTensor * EW_MAX_IN),
                ("ops", EwOp * EW_MAX_OPS),
                ("out", EwResult * EW_MAX_OUT)]


class ConvDims(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("C", "D", "H", "W", "N", "K", "T", "R", "S", "M", "P", "Q", "pad_d", "pad_h",
                 "pad_w", "str_d", "str_h", "str_w", "dil_d", "dil_h", "dil_w")]


class FlexScale(C.Structure):
    _fields_ = [("scale", C.c_float), ("inv_scale", C.c_float)]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "%s is missing: build it with `python ngraph_python_b200/build.py` "
            "(needs nvcc; there is no CPU fallback)" % LIB_PATH)
    lib = C.CDLL(LIB_PATH)
    vp, i32, i64, sz = C.c_void_p, C.c_int32, C.c_int64, C.c_size_t
    sigs = {
        "b2_last_error": (C.c_char_p, []),
        "b2_version": (C.c_int, []),
        "b2_device_count": (C.c_int, []),
        "b2_set_nvrtc_path": (C.c_int, [C.c_char_p]),
        "b2_ew_check": (C.c_int, [C.POINTER(EwProgram), C.c_int, C.c_int, C.c_char_p, sz]),
        "b2_ew_compile": (C.c_int, [C.POINTER(EwProgram), C.POINTER(vp)]),
        "b2_ew_scratch_bytes": (C.c_int, [vp, C.POINTER(sz)]),
        "b2_ew_launch": (C.c_int, [vp, C.POINTER(vp), C.POINTER(vp), C.POINTER(C.c_float), vp, vp,
                                   vp, sz, vp, C.c_int, vp]),
        "b2_ew_launch_builtin_scratch": (C.c_int, [vp, C.POINTER(vp), C.POINTER(vp),
                                                   C.POINTER(C.c_float), vp, vp, vp, C.c_int, vp]),
        "b2_ew_source": (C.c_char_p, [vp]),
        "b2_ew_launch_count": (C.c_int, [vp]),
        "b2_gemm_scratch_bytes": (C.c_int, [i32, i32, i32, i32, C.POINTER(sz)]),
        "b2_gemm_f32": (C.c_int, [vp, i64, i64, vp, i64, i64, vp, i64, i32, i32, i32, vp, sz, vp,
                                  vp]),
        "b2_gemm_flex16": (C.c_int, [vp, i64, i64, vp, i64, i64, vp, i64, i32, i32, i32, vp, i32,
                                     i32, i32, vp, vp, sz, vp, vp, i32, vp]),
        "b2_conv_fprop_scratch_bytes": (C.c_int, [i32, C.POINTER(ConvDims), C.POINTER(sz)]),
        "b2_conv_fprop_f32": (C.c_int, [vp, vp, vp, C.POINTER(ConvDims), vp, sz, vp, vp]),
        "b2_conv_fprop_flex16": (C.c_int, [vp, vp, vp, C.POINTER(ConvDims), vp, i32, i32, i32, vp,
                                           vp, sz, vp, vp, i32, vp]),
        "b2_conv_planes_info": (C.c_int, [C.POINTER(ConvDims), i32, C.POINTER(i32), C.POINTER(sz),
                                          C.POINTER(sz)]),
        "b2_conv_split_activations": (C.c_int, [vp, C.POINTER(ConvDims), i32, vp, vp]),
        "b2_conv_filter_planes": (C.c_int, [vp, C.POINTER(ConvDims), i32, vp, vp]),
        "b2_conv_flex16_planes": (C.c_int, [i32, vp, vp, vp, C.POINTER(ConvDims), vp, i32, i32,
                                            i32, vp, vp, vp, i32, vp]),
        "b2_conv_flex16_planes_fused": (C.c_int, [i32, vp, vp, vp, C.POINTER(ConvDims), vp, i32, i32,
                                                  i32, C.POINTER(ConvEpilogue), vp, vp, vp, i32, vp]),
        "b2_conv_bprop_scratch_bytes": (C.c_int, [i32, C.POINTER(ConvDims), C.POINTER(sz)]),
        "b2_conv_bprop_f32": (C.c_int, [vp, vp, vp, C.POINTER(ConvDims), vp, sz, vp, vp]),
        "b2_conv_bprop_flex16": (C.c_int, [vp, vp, vp, C.POINTER(ConvDims), vp, i32, i32, i32, vp,
                                           vp, sz, vp, vp, i32, vp]),
        "b2_conv_update_scratch_bytes": (C.c_int, [i32, C.POINTER(ConvDims), C.POINTER(sz)]),
        "b2_conv_update_f32": (C.c_int, [vp, vp, vp, C.POINTER(ConvDims), vp, sz, vp, vp]),
        "b2_conv_update_flex16": (C.c_int, [vp, vp, vp, C.POINTER(ConvDims), vp, i32, i32, i32, vp,
                                            vp, sz, vp, vp, i32, vp]),
        "b2_pool_avg_fprop": (C.c_int, [vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32,
                                        i32, i32, i32, vp, vp]),
        "b2_pool_max_fprop": (C.c_int, [vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32,
                                        i32, i32, i32, vp, vp]),
        "b2_pool_bprop": (C.c_int, [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32,
                                    i32, i32, i32, i32, vp, i32, i32, vp, vp, i32, vp]),
        "b2_lut_fprop": (C.c_int, [vp, vp, vp, i32, i32, i32, i32, i32, vp, i32, vp]),
        "b2_lut_update": (C.c_int, [vp, vp, vp, i32, i32, i32, i32, i32, i32, vp, i32, i32, i32,
                                    vp, vp, i32, vp]),
        "b2_dimshuffle": (C.c_int, [vp, vp, i32, i32, C.POINTER(i64), C.POINTER(i64),
                                    C.POINTER(i64), vp]),
        "b2_rng_fill": (C.c_int, [vp, i32, i64, i32, C.c_float, C.c_float, C.c_uint64, C.c_uint64,
                                  vp, vp, i32, vp, vp, i32, vp]),
        "b2_selftest_bounded_wait": (C.c_int, [i32, vp, vp, vp]),
        "b2_set_nccl_path": (C.c_int, [C.c_char_p]),
        "b2_comm_version": (C.c_int, [C.POINTER(i32)]),
        "b2_comm_unique_id": (C.c_int, [vp]),
        "b2_comm_init": (C.c_int, [vp, i32, i32, i32, C.POINTER(vp)]),
        "b2_comm_allreduce_f32": (C.c_int, [vp, vp, i64, i32, vp]),
        "b2_comm_poll_error": (C.c_int, [vp]),
        "b2_comm_abort": (C.c_int, [vp]),
        "b2_comm_destroy": (C.c_int, [vp]),
        "b2_flex_host_quantize": (C.c_int, [vp, vp, i64, vp, i32, vp, vp]),
        "b2_flex_dequantize": (C.c_int, [vp, vp, i64, vp, i32, vp]),
        "b2_absmax_bits_f32": (C.c_int, [vp, i64, vp, vp]),
        "b2_flex_publish": (C.c_int, [vp, i32, vp, vp, vp, vp]),
    }
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib, sigs


_lib, SIGNATURES = _load()


def check(rc):
    if rc < 0:
        raise B200Error("b200ng error %d: %s" % (rc, _lib.b2_last_error().decode(errors="replace")))
    return rc


def raw():
    return _lib


def _find_nvrtc_dir():
    try:
        import nvidia.cuda_nvrtc as m  # wheel bundled with torch
        d = os.path.join(os.path.dirname(m.__file__), "lib")
        if os.path.exists(os.path.join(d, "libnvrtc.so.12")):
            return d
    except Exception:
        pass
    return None


if not os.path.exists("/usr/local/cuda/lib64/libnvrtc.so.12"):
    _d = _find_nvrtc_dir()
    if _d:
        _lib.b2_set_nvrtc_path(_d.encode())


def _find_nccl_dir():
    try:
        import nvidia.nccl as m  # wheel bundled with torch
        d = os.path.join(list(m.__path__)[0], "lib")
        if os.path.exists(os.path.join(d, "libnccl.so.2")):
            return d
    except Exception:
        pass
    return None


_d = _find_nccl_dir()
if _d:
    _lib.b2_set_nccl_path(_d.encode())


def make_program(dims, inputs, consts, ops, outs, reds, reduce_mode):
    """dims=(A,B,C); inputs/outs/reds entries are dicts with dtype, slot, strides (sa,sb,sc);
    ops are (name, a, b); outs carry 'reg'; reds carry 'reg' and 'redop'."""
    p = EwProgram()
    p.A, p.B, p.C = [int(d) for d in dims]
    p.reduce_mode = reduce_mode
    if len(inputs) > EW_MAX_IN or len(ops) > EW_MAX_OPS or len(outs) + len(reds) > EW_MAX_OUT \
            or len(consts) > EW_MAX_CONST:
        raise B200Error("fused program exceeds the kernel limits")
    p.n_in, p.n_const, p.n_ops = len(inputs), len(consts), len(ops)
    p.n_out, p.n_red = len(outs), len(reds)

    def fill(t, d):
        t.dtype = d["dtype"]
        t.flex_slot = d.get("slot", -1)
        t.sa, t.sb, t.sc = [int(s) for s in d["strides"]]
        t.plane_bytes = int(d.get("plane_bytes", 0))
    for i, d in enumerate(inputs):
        fill(p.inp[i], d)
    for i, (name, a, b) in enumerate(ops):
        p.ops[i].opcode = OPCODES[name]
        p.ops[i].a = a
        p.ops[i].b = b if b is not None else 0
    for k, d in enumerate(list(outs) + list(reds)):
        p.out[k].reg = d["reg"]
        p.out[k].redop = REDOPS[d["redop"]] if "redop" in d else 0
        fill(p.out[k].t, d)
    return p


def ew_check(prog, vec=True, probe=False, want_source=False):
    buf = C.create_string_buffer(1 << 18) if want_source else None
    check(_lib.b2_ew_check(C.byref(prog), int(vec), int(probe), buf, len(buf) if buf else 0))
    return buf.value.decode() if buf else None


class EwKernel(object):
    """A compiled fused kernel."""

    def __init__(self, prog):
        self.prog = prog
        h = C.c_void_p()
        check(_lib.b2_ew_compile(C.byref(prog), C.byref(h)))
        self.handle = h
        n = C.c_size_t()
        check(_lib.b2_ew_scratch_bytes(h, C.byref(n)))
        self.scratch_bytes = n.value
        self.launches = _lib.b2_ew_launch_count(h)
        self._consts = (C.c_float * EW_MAX_CONST)()

    def source(self):
        return _lib.b2_ew_source(self.handle).decode()

    def launch(self, in_ptrs, out_ptrs, consts=(), flex_table=0, flex_stats=0, scratch=0,
               scratch_bytes=0, status=0, probe=False, stream=0):
        ins = (C.c_void_p * max(1, len(in_ptrs)))(*in_ptrs)
        outs = (C.c_void_p * max(1, len(out_ptrs)))(*out_ptrs)
        for i, c in enumerate(consts):
            self._consts[i] = c
        check(_lib.b2_ew_launch(self.handle, ins, outs, self._consts, flex_table, flex_stats,
                                scratch, scratch_bytes, status, int(probe), stream))

    def launch_builtin_scratch(self, in_ptrs, out_ptrs, consts=(), flex_table=0, flex_stats=0,
                               status=0, probe=False, stream=0):
        """Same launch through the entry point that allocates nothing: split reductions use the
        16 KiB scratch array that lives inside the library instead of a caller buffer."""
        ins = (C.c_void_p * max(1, len(in_ptrs)))(*in_ptrs)
        outs = (C.c_void_p * max(1, len(out_ptrs)))(*out_ptrs)
        for i, c in enumerate(consts):
            self._consts[i] = c
        check(_lib.b2_ew_launch_builtin_scratch(self.handle, ins, outs, self._consts, flex_table,
                                                flex_stats, status, int(probe), stream))


class PlannedKernel(object):
    """Generated and compiled for sm_100a, but not loaded (no device needed)."""

    def __init__(self, prog, flex=False):
        self.prog = prog
        self._source = ew_check(prog, vec=True, probe=False, want_source=True)
        if flex:
            ew_check(prog, vec=True, probe=True)
        self.scratch_bytes = 0
        self.launches = 2 if "b2_ew_finalize" in self._source else 1

    def source(self):
        return self._source


def gemm_scratch_bytes(flex, M, N, K):
    n = C.c_size_t()
    check(_lib.b2_gemm_scratch_bytes(int(bool(flex)), M, N, K, C.byref(n)))
    return n.value


def conv_fprop_scratch_bytes(flex, dims):
    n = C.c_size_t()
    check(_lib.b2_conv_fprop_scratch_bytes(int(bool(flex)), C.byref(dims), C.byref(n)))
    return n.value


CONV_FPROP, CONV_BPROP = 0, 1
RNG_UNIFORM, RNG_NORMAL = 0, 1


def conv_planes_info(dims, conv_pass=CONV_FPROP):
    """(supported, bytes of one plane of the streamed tensor, bytes of the filter planes)."""
    ok, a, f = C.c_int32(), C.c_size_t(), C.c_size_t()
    check(_lib.b2_conv_planes_info(C.byref(dims), conv_pass, C.byref(ok), C.byref(a), C.byref(f)))
    return bool(ok.value), a.value, f.value


def conv_bprop_scratch_bytes(flex, dims):
    n = C.c_size_t()
    check(_lib.b2_conv_bprop_scratch_bytes(int(bool(flex)), C.byref(dims), C.byref(n)))
    return n.value


def conv_update_scratch_bytes(flex, dims):
    n = C.c_size_t()
    check(_lib.b2_conv_update_scratch_bytes(int(bool(flex)), C.byref(dims), C.byref(n)))
    return n.value


def dimshuffle(src_ptr, dst_ptr, elem_bytes, shape, src_strides, dst_strides, stream=0):
    """N-d strided copy (strides in elements)."""
    n = len(shape)
    arr = C.c_int64 * max(n, 1)
    check(_lib.b2_dimshuffle(src_ptr, dst_ptr, elem_bytes, n, arr(*shape), arr(*src_strides),
                             arr(*dst_strides), stream))
