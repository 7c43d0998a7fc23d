"""Executor steps for the dense contractions and pooling: each wraps one C-ABI entry point.

Takes the place of the reference's per-op kernel objects GEMMKernel (ngraph/transformers/gpu/
gemm.py:26-263), ConvFpropKernel / FlexConvFpropKernel (gpu/conv.py:24-100, gpu/flex_conv.py:
49-200) and PoolFpropKernel / FlexPoolFpropKernel (gpu/pool.py:27-220, gpu/flex_pool.py): bind
buffers once, then launch per call; in flex mode the first write of an output runs the measuring
("probe") variant so that the exponent fits the true range of the result.
"""
import ctypes as C

import numpy as np

from . import lib


def _merge(view, axes):
    """(extent, element stride) of `axes` walked as one dimension of `view`, or None."""
    axes = [a for a in axes if a.length != 1]
    if not axes:
        return 1, 0
    size, stride = 1, None
    for a in reversed(list(axes)):
        s = view.stride_of(a)
        if stride is None:
            stride = s
        elif s != stride * size:
            return None
        size *= a.length
    return size, stride


class _Step(object):
    launches = 0
    scratch_bytes = 0

    def __init__(self, index, op):
        self.index = index
        self.op = op
        self.out_views = []
        self.in_views = []

    def output_buffers(self):
        return [v.buffer for v in self.out_views]

    def _ptr(self, v):
        return v.buffer.ptr() + v.offset * (2 if v.buffer.flex else 4)

    # flex first-write protocol shared by GEMM and conv -------------------------------------------
    def _flex_probe_then(self, t, out_buf, in_bufs, call):
        """call(probe) launches; on the first write of out_buf a probe launch measures the exact
        integer maximum, from which the output exponent is chosen."""
        e = out_buf.entry
        if not e.initialized:
            t._probe64.zero_()
            call(1)
            t.kernel_launches += self.launches
            imax = int(t._probe64.item())
            if getattr(self, "probe_is_float", False):
                # fused epilogue: the kernel leaves the bit pattern of max |fp32 result|
                real = float(np.array([imax & 0xffffffff], dtype=np.uint32).view(np.float32)[0])
            else:
                real = float(imax) * in_bufs[0].entry.scale * in_bufs[1].entry.scale
            dec = e.initialize_from_range(real)
            t._set_table_row(out_buf.slot_write, dec)
            t._stats[out_buf.slot_write:out_buf.slot_write + 1].zero_()
        call(0)
        t.kernel_launches += self.launches


class _PlaneUser(object):
    """flex16 convolution steps that can run on the implicit-GEMM tile kernel: the streamed
    tensor (activations for the forward pass, the error tensor for the input gradient) is read as
    two byte planes which its producer writes directly, and the filter planes are kept for as long
    as the filters do not change -- one launch per convolution."""
    use_planes = False
    filter_planes = None
    filter_version = None

    def _setup_planes(self, t, conv_pass, stream_arg, filter_arg):
        if not self.flex:
            return
        ok, act_bytes, filt_bytes = lib.conv_planes_info(self.dims, conv_pass)
        if not ok:
            return
        self.use_planes = True
        self.conv_pass = conv_pass
        self.plane_arg = stream_arg          # index of the streamed tensor in op.args / in_views
        self.filter_arg = filter_arg
        self.filter_bytes = filt_bytes
        # the input gradient of a strided convolution streams the error tensor with zeros between
        # its elements: planes of its own, written by one extra launch of this step
        self.own_plane_bytes = 0
        if conv_pass == lib.CONV_BPROP and (self.dims.str_h > 1 or self.dims.str_w > 1):
            self.own_plane_bytes = act_bytes
            self.launches = 2
            return
        buf = self.in_views[stream_arg].buffer
        buf.plane_bytes = act_bytes
        buf.plane_steps = getattr(buf, "plane_steps", []) + [self]
        self.launches = 1

    def allocate(self, t):
        if self.use_planes and self.filter_planes is None and not t.plan_only:
            self.filter_planes = t.torch.zeros((self.filter_bytes + 1024,), dtype=t.torch.uint8,
                                               device=t.device)
            self.filter_ptr = self.filter_planes.data_ptr() + (-self.filter_planes.data_ptr()) % 1024
            if self.own_plane_bytes:
                self.own_planes = t.torch.zeros((2 * self.own_plane_bytes + 1024,),
                                                dtype=t.torch.uint8, device=t.device)
                self.own_planes_ptr = self.own_planes.data_ptr() + (-self.own_planes.data_ptr()) % 1024

    def _build_filter_planes(self, t):
        fv = self.in_views[self.filter_arg]
        lib.check(lib.raw().b2_conv_filter_planes(self._ptr(fv), C.byref(self.dims), self.conv_pass,
                                                  self.filter_ptr, t.stream.cuda_stream))
        t.kernel_launches += 1
        self.filter_version = fv.buffer.version

    def refresh(self, t):
        """Rebuilds the cached filter planes when the filters have changed since they were built
        (called before every launch, and before every replay of a captured step list)."""
        if not self.use_planes:
            return
        fbuf = self.in_views[self.filter_arg].buffer
        if fbuf.last_write_step < 0 and self.filter_version != fbuf.version:
            self._build_filter_planes(t)

    def _launch_planes(self, t):
        xv, fv = self.in_views[self.plane_arg], self.in_views[self.filter_arg]
        ov = self.out_views[0]
        raw = lib.raw()
        st = t.stream.cuda_stream
        xbuf, fbuf = xv.buffer, fv.buffer
        planes_ptr = self.own_planes_ptr if self.own_plane_bytes else xbuf.planes_ptr
        if self.own_plane_bytes or not xbuf.planes_by_producer:
            lib.check(raw.b2_conv_split_activations(self._ptr(xv), C.byref(self.dims),
                                                    self.conv_pass, planes_ptr, st))
            t.kernel_launches += 1
        if fbuf.last_write_step >= 0:
            self._build_filter_planes(t)     # filters written inside this computation
        else:
            self.refresh(t)
        slots = (t._slot_for_read(xbuf, self), t._slot_for_read(fbuf, self), ov.buffer.slot_write)
        epi = getattr(self, "epi", None)
        if epi is None:
            def call(probe):
                lib.check(raw.b2_conv_flex16_planes(
                    self.conv_pass, planes_ptr, self.filter_ptr, self._ptr(ov),
                    C.byref(self.dims), t._table.data_ptr(), slots[0], slots[1], slots[2],
                    t._stats.data_ptr(), t._probe64.data_ptr(), t._status.data_ptr(), probe, st))
            self._flex_probe_then(t, ov.buffer, [xbuf, fbuf], call)
            return
        ce = lib.ConvEpilogue()
        extra = self.in_views[2:]
        k = 0
        ce.bias, ce.slot_bias, ce.residual, ce.slot_residual = None, -1, None, -1
        if epi.get("bias") is not None:
            ce.bias, ce.slot_bias = self._ptr(extra[k]), t._slot_for_read(extra[k].buffer, self)
            k += 1
        if epi.get("residual") is not None:
            ce.residual = self._ptr(extra[k])
            ce.slot_residual = t._slot_for_read(extra[k].buffer, self)
        ce.relu = int(bool(epi.get("relu")))
        obuf = ov.buffer
        ce.write_int16 = int(self.write_int16 or obuf.plane_bytes == 0)
        ce.out_planes, ce.plane_bytes = (obuf.planes_ptr, obuf.plane_bytes) if obuf.plane_bytes else (None, 0)

        def call(probe):
            lib.check(raw.b2_conv_flex16_planes_fused(
                self.conv_pass, planes_ptr, self.filter_ptr, self._ptr(ov),
                C.byref(self.dims), t._table.data_ptr(), slots[0], slots[1], slots[2],
                C.byref(ce), t._stats.data_ptr(), t._probe64.data_ptr(), t._status.data_ptr(),
                probe, st))
        self._flex_probe_then(t, obuf, [xbuf, fbuf], call)


class GemmStep(_Step):
    """C[M,N] = op(A)[M,K] * op(B)[K,N] for a DotOp."""
    kind = "gemm"
    launches = 3          # two operand-plane kernels + the tensor-core kernel

    def __init__(self, index, op, t):
        super(GemmStep, self).__init__(index, op)
        x, y = op.args
        xv, yv = t._view_of(x), t._view_of(y)
        red = [a for a in xv.axes if a in op.reduction_axes]
        am, ak = _merge(xv, op.x_out_axes), _merge(xv, red)
        bk, bn = _merge(yv, red), _merge(yv, op.y_out_axes)
        if None in (am, ak, bk, bn):
            raise ValueError("Unhandled op: dot operands must be 2-d collapsible: {}".format(op))
        self.M, self.K, self.N = am[0], ak[0], bn[0]
        if t.flex and self.M * self.N <= 8192 and self.K <= 1024:
            self.launches = 1         # the library's one-launch form for very small products
        if bk[0] != self.K:
            raise ValueError("Unhandled op: reduction axes of the dot operands disagree")
        # extents of 1 carry no stride of their own: describe them as row-major
        a_cs = ak[1] if self.K > 1 else 1
        a_rs = am[1] if self.M > 1 else (self.K if a_cs == 1 else 1)
        b_ns = bn[1] if self.N > 1 else 1
        b_ks = bk[1] if self.K > 1 else (self.N if b_ns == 1 else 1)
        self.a_str = (a_rs, a_cs)
        self.b_str = (b_ks, b_ns)
        if 1 not in self.a_str or 1 not in self.b_str:
            raise ValueError("Unhandled op: dot operand is not contiguous along M/K or K/N")
        self.in_views = [xv, yv]
        self.out_views = [t._view_of(op)]
        self.flex = t.flex
        self.scratch_bytes = lib.gemm_scratch_bytes(self.flex, self.M, self.N, self.K) + 1024

    def launch(self, t):
        xv, yv = self.in_views
        ov = self.out_views[0]
        raw = lib.raw()
        sp, sb = t._scratch_aligned()
        st = t.stream.cuda_stream
        if not self.flex:
            lib.check(raw.b2_gemm_f32(self._ptr(xv), self.a_str[0], self.a_str[1], self._ptr(yv),
                                      self.b_str[0], self.b_str[1], self._ptr(ov), self.N, self.M,
                                      self.N, self.K, sp, sb, t._status.data_ptr(), st))
            t.kernel_launches += self.launches
            return
        slots = (t._slot_for_read(xv.buffer, self), t._slot_for_read(yv.buffer, self),
                 ov.buffer.slot_write)

        def call(probe):
            lib.check(raw.b2_gemm_flex16(
                self._ptr(xv), self.a_str[0], self.a_str[1], self._ptr(yv), self.b_str[0],
                self.b_str[1], self._ptr(ov), self.N, self.M, self.N, self.K, t._table.data_ptr(),
                slots[0], slots[1], slots[2], t._stats.data_ptr(), sp, sb, t._probe64.data_ptr(),
                t._status.data_ptr(), probe, st))
        self._flex_probe_then(t, ov.buffer, [xv.buffer, yv.buffer], call)


class ConvStep(_PlaneUser, _Step):
    """Convolution forward on C,D,H,W,N / C,T,R,S,K / K,M,P,Q,N tensors."""
    kind = "conv"
    launches = 3

    def __init__(self, index, op, t, epilogue=None):
        """epilogue (flex16 implicit-GEMM path only): dict(out=<op whose tensor the step writes>,
        bias=<op or None>, residual=<op or None>, relu=bool) -- the elementwise tail of the layer,
        evaluated in the tile kernel's epilogue."""
        super(ConvStep, self).__init__(index, op)
        inputs, filters = op.args
        self.epi = epilogue
        out_op = epilogue["out"] if epilogue else op
        iv, fv, ov = t._view_of(inputs), t._view_of(filters), t._view_of(out_op)
        if epilogue and not ov.is_dense():
            raise ValueError("fused convolution output must be a dense tensor")
        for v, what in ((iv, "input"), (fv, "filter")):
            if not v.is_dense():
                raise ValueError("Unhandled op: convolution %s must be a dense tensor" % what)
        cp = op.conv_params
        Cc, D, H, W, N = iv.axes.lengths
        C2, T, R, S, K = fv.axes.lengths
        K2, M, P, Q, N2 = op.axes.lengths          # (the tail's tensor may lack the unit axes)
        if K2 != K or N2 != N or ov.buffer.size != K2 * M * P * Q * N2:
            raise ValueError("convolution output axes do not match filter/input axes")
        d = lib.ConvDims()
        d.C, d.D, d.H, d.W, d.N = Cc, D, H, W, N
        d.K, d.T, d.R, d.S = K, T, R, S
        d.M, d.P, d.Q = M, P, Q
        for k in ("pad_d", "pad_h", "pad_w"):
            setattr(d, k, int(cp.get(k, 0)))
        for k in ("str_d", "str_h", "str_w", "dil_d", "dil_h", "dil_w"):
            setattr(d, k, int(cp.get(k, 1)))
        # the output extents must be what the parameters imply (reference: output_dim,
        # ngraph/frontends/neon/utils.py / conv_utils.py)
        for (x, f, pad, st, dil, o, nm) in ((D, T, d.pad_d, d.str_d, d.dil_d, M, "D"),
                                            (H, R, d.pad_h, d.str_h, d.dil_h, P, "H"),
                                            (W, S, d.pad_w, d.str_w, d.dil_w, Q, "W")):
            expect = (x + 2 * pad - dil * (f - 1) - 1) // st + 1
            if expect != o:
                raise ValueError("convolution output extent along %s is %d, parameters imply %d"
                                 % (nm, o, expect))
        self.dims = d
        self.in_views = [iv, fv]
        self.out_views = [ov]
        self.flex = t.flex
        self.scratch_bytes = lib.conv_fprop_scratch_bytes(self.flex, d) + 1024
        self._setup_planes(t, lib.CONV_FPROP, 0, 1)
        if epilogue:
            if not self.use_planes:
                raise ValueError("a fused convolution epilogue needs the implicit-GEMM path")
            self.probe_is_float = True
            self.write_int16 = True          # the planner clears it when only planes are read
            for key in ("bias", "residual"):
                if epilogue.get(key) is not None:
                    v = t._view_of(epilogue[key])
                    if not v.is_dense():
                        raise ValueError("fused convolution %s must be a dense tensor" % key)
                    self.in_views.append(v)

    def launch(self, t):
        if self.use_planes:
            return self._launch_planes(t)
        iv, fv = self.in_views
        ov = self.out_views[0]
        raw = lib.raw()
        sp, sb = t._scratch_aligned()
        st = t.stream.cuda_stream
        if not self.flex:
            lib.check(raw.b2_conv_fprop_f32(self._ptr(iv), self._ptr(fv), self._ptr(ov),
                                            C.byref(self.dims), sp, sb, t._status.data_ptr(), st))
            t.kernel_launches += self.launches
            return
        slots = (t._slot_for_read(iv.buffer, self), t._slot_for_read(fv.buffer, self),
                 ov.buffer.slot_write)

        def call(probe):
            lib.check(raw.b2_conv_fprop_flex16(
                self._ptr(iv), self._ptr(fv), self._ptr(ov), C.byref(self.dims),
                t._table.data_ptr(), slots[0], slots[1], slots[2], t._stats.data_ptr(), sp, sb,
                t._probe64.data_ptr(), t._status.data_ptr(), probe, st))
        self._flex_probe_then(t, ov.buffer, [iv.buffer, fv.buffer], call)


def _conv_dims_of(fprop, t):
    """ConvDims of a forward ConvolutionOp (axes C,D,H,W,N / C,T,R,S,K / K,M,P,Q,N)."""
    cp = fprop.conv_params
    Cc, D, H, W, N = fprop.args[0].axes.lengths
    C2, T, R, S, K = fprop.args[1].axes.lengths
    K2, M, P, Q, N2 = fprop.axes.lengths
    d = lib.ConvDims()
    d.C, d.D, d.H, d.W, d.N = Cc, D, H, W, N
    d.K, d.T, d.R, d.S = K, T, R, S
    d.M, d.P, d.Q = M, P, Q
    for k in ("pad_d", "pad_h", "pad_w"):
        setattr(d, k, int(cp.get(k, 0)))
    for k in ("str_d", "str_h", "str_w", "dil_d", "dil_h", "dil_w"):
        setattr(d, k, int(cp.get(k, 1)))
    return d


class _ConvGradStep(_PlaneUser, _Step):
    """Shared part of the two convolution gradients: two dense operands, one dense result, the
    forward convolution's dimensions."""
    launches = 3
    what = None                     # "bprop" | "update"

    def __init__(self, index, op, t):
        super(_ConvGradStep, self).__init__(index, op)
        av, bv, ov = t._view_of(op.args[0]), t._view_of(op.args[1]), t._view_of(op)
        for v in (av, bv):
            if not v.is_dense():
                raise ValueError("Unhandled op: convolution %s operands must be dense tensors"
                                 % self.what)
        self.dims = _conv_dims_of(op.fprop, t)
        d = self.dims
        expect = {"bprop": ((d.K, d.M, d.P, d.Q, d.N), (d.C, d.T, d.R, d.S, d.K),
                            (d.C, d.D, d.H, d.W, d.N)),
                  "update": ((d.K, d.M, d.P, d.Q, d.N), (d.C, d.D, d.H, d.W, d.N),
                             (d.C, d.T, d.R, d.S, d.K))}[self.what]
        for v, shape in zip((av, bv, ov), expect):
            if tuple(v.axes.lengths) != shape:
                raise ValueError("convolution %s: tensor of shape %s where %s is expected"
                                 % (self.what, tuple(v.axes.lengths), shape))
        self.in_views = [av, bv]
        self.out_views = [ov]
        self.flex = t.flex
        sizer = lib.conv_bprop_scratch_bytes if self.what == "bprop" else \
            lib.conv_update_scratch_bytes
        self.scratch_bytes = sizer(self.flex, d) + 1024
        if self.what == "bprop":
            self._setup_planes(t, lib.CONV_BPROP, 0, 1)      # streamed: delta; filters: args[1]

    def launch(self, t):
        if self.use_planes:
            return self._launch_planes(t)
        av, bv = self.in_views           # (delta, filters) or (delta, inputs)
        ov = self.out_views[0]
        raw = lib.raw()
        sp, sb = t._scratch_aligned()
        st = t.stream.cuda_stream
        if self.what == "bprop":
            first, second = av, bv       # E, F
            f32, f16 = raw.b2_conv_bprop_f32, raw.b2_conv_bprop_flex16
        else:
            first, second = bv, av       # I, E
            f32, f16 = raw.b2_conv_update_f32, raw.b2_conv_update_flex16
        if not self.flex:
            lib.check(f32(self._ptr(first), self._ptr(second), self._ptr(ov), C.byref(self.dims),
                          sp, sb, t._status.data_ptr(), st))
            t.kernel_launches += self.launches
            return
        slots = (t._slot_for_read(first.buffer, self), t._slot_for_read(second.buffer, self),
                 ov.buffer.slot_write)

        def call(probe):
            lib.check(f16(self._ptr(first), self._ptr(second), self._ptr(ov), C.byref(self.dims),
                          t._table.data_ptr(), slots[0], slots[1], slots[2], t._stats.data_ptr(),
                          sp, sb, t._probe64.data_ptr(), t._status.data_ptr(), probe, st))
        self._flex_probe_then(t, ov.buffer, [first.buffer, second.buffer], call)


class ConvBpropStep(_ConvGradStep):
    """Input gradient of a convolution: args (delta K,M,P,Q,N ; filters C,T,R,S,K)."""
    kind = "conv_bprop"
    what = "bprop"


class ConvUpdateStep(_ConvGradStep):
    """Filter gradient of a convolution: args (delta K,M,P,Q,N ; inputs C,D,H,W,N)."""
    kind = "conv_update"
    what = "update"
    launches = 4                    # two operand kernels, the tile kernel, the slice sum


class PoolStep(_Step):
    """Average or max pooling forward; a flex output keeps its input's exponent
    (ngraph/transformers/passes/flexpass.py:40-48)."""
    kind = "pool"
    launches = 1

    def __init__(self, index, op, t):
        super(PoolStep, self).__init__(index, op)
        pp = op.pool_params
        if pp["op"] not in ("avg", "max"):
            raise ValueError("Unhandled op: only average and max pooling are implemented: {}"
                             .format(op))
        self.pool_op = pp["op"]
        iv = t._view_of(op.args[0])
        if not iv.is_dense():
            raise ValueError("Unhandled op: pooling input must be a dense tensor")
        if int(pp.get("J", 1)) != 1 or int(pp.get("T", 1)) != 1:
            raise ValueError("Unhandled op: pooling over channels or depth")
        ov = t._view_of(op)
        if t.flex:
            t._share_entry(ov.buffer, iv.buffer)
        Cc, D, H, W, N = iv.axes.lengths
        K, M, P, Q, N2 = ov.axes.lengths
        self.args = (Cc, H, W, N, P, Q, int(pp["R"]), int(pp["S"]), int(pp.get("pad_h", 0)),
                     int(pp.get("pad_w", 0)), int(pp.get("str_h", 1)), int(pp.get("str_w", 1)))
        self.in_views = [iv]
        self.out_views = [ov]
        self.flex = t.flex

    def output_buffers(self):
        return []          # no exponent of its own to manage

    def launch(self, t):
        iv, ov = self.in_views[0], self.out_views[0]
        stats = 0
        if self.flex:
            stats = t._stats.data_ptr() + 4 * (t._stats.numel() - 2)    # discarded
        fn = lib.raw().b2_pool_max_fprop if self.pool_op == "max" else lib.raw().b2_pool_avg_fprop
        lib.check(fn(self._ptr(iv), self._ptr(ov), int(self.flex),
                     *(self.args + (stats, t.stream.cuda_stream))))
        t.kernel_launches += 1


class PoolBpropStep(_Step):
    """Gradient of average or max pooling with respect to the pooled tensor."""
    kind = "pool_bprop"
    launches = 1
    probe_is_float = True

    def __init__(self, index, op, t):
        super(PoolBpropStep, self).__init__(index, op)
        pp = op.pool_params
        if pp["op"] not in ("avg", "max"):
            raise ValueError("Unhandled op: only average and max pooling are implemented: {}"
                             .format(op))
        if int(pp.get("J", 1)) != 1 or int(pp.get("T", 1)) != 1:
            raise ValueError("Unhandled op: pooling over channels or depth")
        ev, iv, ov = t._view_of(op.args[0]), t._view_of(op.args[1]), t._view_of(op)
        for v in (ev, iv):
            if not v.is_dense():
                raise ValueError("Unhandled op: pooling gradient operands must be dense tensors")
        Cc, D, H, W, N = iv.axes.lengths
        K, M, P, Q, N2 = ev.axes.lengths
        self.is_max = int(pp["op"] == "max")
        self.args = (Cc, H, W, N, P, Q, int(pp["R"]), int(pp["S"]), int(pp.get("pad_h", 0)),
                     int(pp.get("pad_w", 0)), int(pp.get("str_h", 1)), int(pp.get("str_w", 1)))
        self.in_views = [ev, iv]
        self.out_views = [ov]
        self.flex = t.flex

    def launch(self, t):
        ev, iv = self.in_views
        ov = self.out_views[0]
        raw = lib.raw()
        st = t.stream.cuda_stream
        if not self.flex:
            lib.check(raw.b2_pool_bprop(self._ptr(ev), self._ptr(iv), self._ptr(ov), 0, self.is_max,
                                        *(self.args + (None, -1, -1, None, None, 0, st))))
            t.kernel_launches += 1
            return
        t._slot_for_read(iv.buffer, self)
        slots = (t._slot_for_read(ev.buffer, self), ov.buffer.slot_write)

        def call(probe):
            lib.check(raw.b2_pool_bprop(self._ptr(ev), self._ptr(iv), self._ptr(ov), 1, self.is_max,
                                        *(self.args + (t._table.data_ptr(), slots[0], slots[1],
                                                       t._stats.data_ptr(), t._probe64.data_ptr(),
                                                       probe, st))))
        self._flex_probe_then(t, ov.buffer, [ev.buffer, iv.buffer], call)


class LutStep(_Step):
    """Embedding lookup; a flex output keeps the table's exponent (its mantissas are copied)."""
    kind = "lut"
    launches = 1

    def __init__(self, index, op, t):
        super(LutStep, self).__init__(index, op)
        lv, xv, ov = t._view_of(op.args[0]), t._view_of(op.args[1]), t._view_of(op)
        for v in (lv, xv):
            if not v.is_dense():
                raise ValueError("Unhandled op: lookup operands must be dense tensors")
        self.lut_axis = op.lut_axis
        self.V = lv.axes.lengths[op.lut_axis]
        self.F = lv.axes.lengths[1 - op.lut_axis]
        self.n = xv.axes.lengths[0]
        if t.flex:
            t._share_entry(ov.buffer, lv.buffer)
        self.in_views = [lv, xv]
        self.out_views = [ov]
        self.flex = t.flex

    def output_buffers(self):
        return []          # no exponent of its own to manage

    def launch(self, t):
        lv, xv = self.in_views
        ov = self.out_views[0]
        table, slot = (t._table.data_ptr(), t._slot_for_read(xv.buffer, self)) if self.flex else (None, -1)
        lib.check(lib.raw().b2_lut_fprop(self._ptr(lv), self._ptr(xv), self._ptr(ov), int(self.flex),
                                         self.lut_axis, self.V, self.F, self.n, table, slot,
                                         t.stream.cuda_stream))
        t.kernel_launches += 1


class LutUpdateStep(_Step):
    """Gradient of an embedding table: rows of delta added up per looked-up index."""
    kind = "lut_update"
    launches = 1
    probe_is_float = True

    def __init__(self, index, op, t):
        super(LutUpdateStep, self).__init__(index, op)
        dv, xv, ov = t._view_of(op.args[0]), t._view_of(op.args[1]), t._view_of(op)
        for v in (dv, xv):
            if not v.is_dense():
                raise ValueError("Unhandled op: lookup update operands must be dense tensors")
        self.lut_axis = op.lut_axis
        self.V = ov.axes.lengths[op.lut_axis]
        self.F = ov.axes.lengths[1 - op.lut_axis]
        self.n = xv.axes.lengths[0]
        self.pad_idx = -1 if op.pad_idx is None else int(op.pad_idx)
        self.in_views = [dv, xv]
        self.out_views = [ov]
        self.flex = t.flex

    def launch(self, t):
        dv, xv = self.in_views
        ov = self.out_views[0]
        raw = lib.raw()
        st = t.stream.cuda_stream
        head = (self._ptr(dv), self._ptr(xv), self._ptr(ov))
        dims = (self.lut_axis, self.V, self.F, self.n, self.pad_idx)
        if not self.flex:
            lib.check(raw.b2_lut_update(*(head + (0,) + dims + (None, -1, -1, -1, None, None, 0, st))))
            t.kernel_launches += 1
            return
        slots = (t._slot_for_read(dv.buffer, self), t._slot_for_read(xv.buffer, self),
                 ov.buffer.slot_write)

        def call(probe):
            lib.check(raw.b2_lut_update(*(head + (1,) + dims + (
                t._table.data_ptr(), slots[0], slots[1], slots[2], t._stats.data_ptr(),
                t._probe64.data_ptr(), probe, st))))
        self._flex_probe_then(t, ov.buffer, [dv.buffer, xv.buffer], call)


class RngStep(_Step):
    """Random fill (RngFillKernel / FlexRngFillKernel, ngraph/transformers/gpu/tensor_ops.py:
    621-661, 713-740).  The stream of numbers is fixed by the transformer's seed and the position
    of the op in its graph; a device-side counter moves it on after every execution, also under
    CUDA-graph replay."""
    kind = "rng"
    launches = 2           # the fill and the advance of its counter
    probe_is_float = True

    def __init__(self, index, op, t):
        super(RngStep, self).__init__(index, op)
        ov = t._view_of(op)
        self.out_views = [ov]
        self.in_views = []
        self.flex = t.flex
        p = op.params
        if op.distribution == "uniform":
            self.dist, self.a, self.b = lib.RNG_UNIFORM, float(p["low"]), float(p["high"])
        else:
            self.dist, self.a, self.b = lib.RNG_NORMAL, float(p["loc"]), float(p["scale"])
        self.seed = int(t.rng_seed)
        self.stream_id = t._next_rng_stream()
        self.counter = None

    def allocate(self, t):
        if self.counter is None and not t.plan_only:
            self.counter = t.torch.zeros((1,), dtype=t.torch.int64, device=t.device)

    def launch(self, t):
        ov = self.out_views[0]
        raw = lib.raw()
        st = t.stream.cuda_stream
        offset = self.stream_id << 40           # streams of different ops never meet
        head = (self._ptr(ov), int(self.flex), ov.buffer.size, self.dist, self.a, self.b, self.seed,
                offset, self.counter.data_ptr())
        if not self.flex:
            lib.check(raw.b2_rng_fill(*(head + (None, -1, None, None, 0, st))))
            t.kernel_launches += self.launches
            return
        slot = ov.buffer.slot_write

        def call(probe):
            lib.check(raw.b2_rng_fill(*(head + (t._table.data_ptr(), slot, t._stats.data_ptr(),
                                                t._probe64.data_ptr(), probe, st))))
        self._flex_probe_then(t, ov.buffer, [], call)


class DimshuffleStep(_Step):
    """A strided copy between two views with the same axes (DimShuffleKernel of the reference,
    ngraph/transformers/gpu/tensor_ops.py:119-204; it also carries AssignOp between differently
    laid-out tensors, gputransform.py:393-395).  A flex16 copy moves mantissas, so the destination
    shares the source's exponent (the reference propagates the FlexEntry through a dimshuffle the
    same way, ngraph/transformers/passes/flexpass.py:32-48)."""
    kind = "dimshuffle"
    launches = 1

    def __init__(self, index, op, t, src_view, dst_view, axes):
        super(DimshuffleStep, self).__init__(index, op)
        self.in_views = [src_view]
        self.out_views = [dst_view]
        self.lengths = [a.length for a in axes]
        self.src_strides = [src_view.stride_of(a) for a in axes]
        self.dst_strides = [dst_view.stride_of(a) for a in axes]
        if len(self.lengths) > 8:
            raise ValueError("Unhandled op: dimshuffle of more than 8 axes")
        if src_view.buffer.flex != dst_view.buffer.flex:
            raise ValueError("dimshuffle between tensors of different storage types")
        self.elem_bytes = 2 if src_view.buffer.flex else 4
        self.owns_version = True

    def output_buffers(self):
        return []          # no exponent of its own to manage

    def launch(self, t):
        sv, dv = self.in_views[0], self.out_views[0]
        lib.dimshuffle(self._ptr(sv), self._ptr(dv), self.elem_bytes, self.lengths,
                       self.src_strides, self.dst_strides, t.stream.cuda_stream)
        t.kernel_launches += 1


class CommStep(_Step):
    """One tensor's share of a bucketed allreduce (see comm.py).  The tensor lives inside the
    flat fp32 arena; when this step is the last of its bucket the collective for the whole bucket
    is started.  In flex mode the int16 gradient is first de-quantised into the arena."""
    kind = "comm"
    launches = 0

    def __init__(self, index, op, t, src_view, arena_buffer):
        super(CommStep, self).__init__(index, op)
        self.key = id(arena_buffer)
        self.src_view = src_view            # flex: the int16 tensor to de-quantise; else None
        self.arena_buffer = arena_buffer    # fp32 Buffer placed in the arena
        self.in_views = [src_view] if src_view is not None else []
        self.out_views = []
        self.closes_bucket = None           # set when the bucket plan is known
        self.launches = 1 if src_view is not None else 0

    def output_buffers(self):
        return []

    def launch(self, t):
        if self.src_view is not None:
            v = self.src_view
            lib.check(lib.raw().b2_flex_dequantize(
                self._ptr(v), self.arena_buffer.ptr(), v.buffer.size, t._table.data_ptr(),
                t._slot_for_read(v.buffer, self), t.stream.cuda_stream))
            t.kernel_launches += 1
        if t._recording:
            return          # a graph is being recorded: the exchange is issued between replays
        t._allreduce.produced(self.key)
        if self.closes_bucket is not None:
            t._allreduce.bucket_ready(self.closes_bucket)
