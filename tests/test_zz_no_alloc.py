"""The launch that allocates nothing (b2_ew_launch_builtin_scratch), through the C ABI.

Some hosts of this library cannot call cudaMalloc when a kernel turns out to need scratch: a
runtime that handed the whole device to its own arena at start-up, or a steady-state loop that
must not hit cudaMalloc's device-wide synchronisation.  For them the split row reduction can take
its partial-sum scratch from a 16 KiB array inside the library.  This test runs the same compiled
kernel through the ordinary entry point (caller-provided scratch) and through the no-allocation
one, twice in a row with different data, and expects identical results: both run the same code,
only the scratch pointer differs.  It is collected last so that a failure here cannot hide another
test's result, and it does not depend on any state left by the tests before it.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
BUILTIN_BYTES = 16 * 1024        # B2_EW_BUILTIN_SCRATCH_BYTES of include/b200ng.h


def _split_program(lib, rows, cols):
    """sum and max|.| over very long rows: few rows, so each row is shared by many CTAs."""
    ins = [dict(dtype=lib.F32, strides=(0, cols, 1)), dict(dtype=lib.F32, strides=(0, cols, 1))]
    ops = [("mul", 0, 1), ("abs", 2, None)]
    reds = [dict(dtype=lib.F32, strides=(0, 1, 0), reg=2, redop="sum"),
            dict(dtype=lib.F32, strides=(0, 1, 0), reg=3, redop="max")]
    return lib.make_program((1, rows, cols), ins, [], ops, [], reds, lib.REDUCE_C)


def test_builtin_scratch_matches_caller_scratch_twice():
    import torch
    from ngraph_python_b200 import lib
    rows, cols = 3, 1 << 20
    k = lib.EwKernel(_split_program(lib, rows, cols))
    assert k.launches == 2 and k.scratch_bytes > 0, "the program must be a split reduction"
    assert k.scratch_bytes <= BUILTIN_BYTES
    scratch = torch.empty((k.scratch_bytes,), dtype=torch.uint8, device="cuda")
    rng = np.random.RandomState(11)
    for call in range(2):
        a = torch.from_numpy(rng.standard_normal((rows, cols)).astype(np.float32)).cuda()
        b = torch.from_numpy(rng.standard_normal((rows, cols)).astype(np.float32)).cuda()
        ref = [torch.full((rows,), -1.0, device="cuda") for _ in range(2)]
        new = [torch.full((rows,), -2.0, device="cuda") for _ in range(2)]
        ins = [a.data_ptr(), b.data_ptr()]
        # ordinary entry point first: it also makes sure the kernel variant is compiled
        k.launch(ins, [r.data_ptr() for r in ref], scratch=scratch.data_ptr(),
                 scratch_bytes=k.scratch_bytes)
        k.launch_builtin_scratch(ins, [r.data_ptr() for r in new])
        torch.cuda.synchronize()
        for r, n in zip(ref, new):
            assert torch.equal(r, n), "call %d: results differ" % call
        # and both agree with numpy (fp32 bar: rtol 1e-4)
        prod = a.cpu().numpy().astype(np.float64) * b.cpu().numpy()
        np.testing.assert_allclose(new[0].cpu().numpy(), prod.sum(axis=1), rtol=1e-4, atol=0.05)
        np.testing.assert_allclose(new[1].cpu().numpy(), np.abs(prod).max(axis=1), rtol=1e-4)


def test_builtin_scratch_rejects_oversized_and_uncompiled():
    import torch
    from ngraph_python_b200 import lib
    # 290 rows shared by 3 CTAs each x 6 reductions: 20 880 bytes of partials, more than the array
    rows, cols = 290, 1 << 16
    ins = [dict(dtype=lib.F32, strides=(0, cols, 1))]
    reds = [dict(dtype=lib.F32, strides=(0, 1, 0), reg=0, redop=r)
            for r in ("sum", "max", "min", "prod", "sum", "max")]
    k = lib.EwKernel(lib.make_program((1, rows, cols), ins, [], [], [], reds, lib.REDUCE_C))
    x = torch.zeros((rows, cols), device="cuda")
    outs = [torch.zeros((rows,), device="cuda") for _ in reds]
    assert k.launches == 2 and k.scratch_bytes > BUILTIN_BYTES, \
        "the program must need more scratch than the library holds"
    with pytest.raises(lib.B200Error, match="built-in scratch holds"):
        k.launch_builtin_scratch([x.data_ptr()], [o.data_ptr() for o in outs])
    # the ordinary entry point takes the same launch with a caller buffer
    scratch = torch.empty((k.scratch_bytes,), dtype=torch.uint8, device="cuda")
    k.launch([x.data_ptr()], [o.data_ptr() for o in outs], scratch=scratch.data_ptr(),
             scratch_bytes=k.scratch_bytes)
    torch.cuda.synchronize()
    # an unaligned pointer needs the scalar variant, which nothing has compiled yet
    k2 = lib.EwKernel(_split_program(lib, 2, 1 << 20))
    a = torch.zeros((2 * (1 << 20) + 1,), device="cuda")
    o = [torch.zeros((2,), device="cuda") for _ in range(2)]
    with pytest.raises(lib.B200Error, match="has not been compiled"):
        k2.launch_builtin_scratch([a.data_ptr() + 4, a.data_ptr() + 4], [t.data_ptr() for t in o])
