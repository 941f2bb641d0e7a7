"""The allocation-free dot product (fb_dot_product_noalloc_f32) against the regular entry point.

Some callers of the library cannot allocate device memory or pass scratch buffers (a plugin inside
a fixed memory plan, code that must not trigger a synchronising allocation); for them the operand
ranges live in a fixed array inside the library.  This test calls both entry points through the
C ABI on the same inputs, twice in a row with different inputs (the shared array keeps the first
call's contents, which must not leak into the second result), and checks the size limit.

The file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import pytest
import torch

import cases

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _call(fn_name, x, y, shape, layout, scratch):
    from faith_b200 import _lib, ops
    lib = _lib.load()
    B, Lx, Ly, Di, K = shape
    zshape = (B, Lx, Di, Ly) if layout == _lib.FB_NATIVE else (B, Lx, Ly, Di)
    z = [torch.full(zshape, float("nan"), device=DEV), torch.full(zshape, float("nan"), device=DEV),
         torch.full((B, Lx, Ly), float("nan"), device=DEV), torch.full((B, Lx, Ly), float("nan"), device=DEV)]
    ptrs = [t.data_ptr() for t in (x[0], x[2], x[1], x[3], y[0], y[2], y[1], y[3])] + [t.data_ptr() for t in z]
    tail = (B, Lx, Ly, Di, K, 1, _lib.FB_P2, 0.5, 0.25, layout, torch.cuda.current_stream().cuda_stream)
    if scratch is not None:
        ptrs += [t.data_ptr() for t in scratch]
    _lib.check(getattr(lib, fn_name)(*ptrs, *tail), fn_name)
    torch.cuda.synchronize()
    return z


@pytest.mark.parametrize("transposed", [False, True])
def test_noalloc_matches_regular_entry_point_twice(transposed):
    from faith_b200 import _lib
    layout = _lib.FB_TRANSPOSED if transposed else _lib.FB_NATIVE
    for seed, shape in ((1, (4, 32, 32, 128, 32)), (2, (2, 9, 5, 24, 12))):   # two calls in a row
        B, Lx, Ly, Di, K = shape
        x = [t.to(DEV) for t in cases.rand_bounds(900 + seed, B, Lx, Di, K, -0.5, 1.0)]   # lw, lb, uw, ub
        y = [t.to(DEV) for t in cases.rand_bounds(950 + seed, B, Ly, Di, K, -0.5, 1.0)]
        if transposed:
            for t in (x, y):
                t[0] = t[0].transpose(2, 3).contiguous()
                t[2] = t[2].transpose(2, 3).contiguous()
        scratch = [torch.empty(B, Lx, K, device=DEV), torch.empty(B, Lx, K, device=DEV),
                   torch.empty(B, Ly, K, device=DEV), torch.empty(B, Ly, K, device=DEV)]
        ref = _call("fb_dot_product_f32", x, y, shape, layout, scratch)
        got = _call("fb_dot_product_noalloc_f32", x, y, shape, layout, None)
        for a, b, name in zip(got, ref, ("z_lw", "z_uw", "z_lb", "z_ub")):
            assert bool(torch.isfinite(a).all()), name
            # same kernels on the same inputs: the results must agree to the last bit, which is
            # well inside the per-operator bar (rel 1e-5 / abs 1e-6) of the other tests
            assert torch.equal(a, b), "%s differs between the two entry points" % name


def test_noalloc_rejects_sizes_beyond_the_fixed_array():
    from faith_b200 import _lib
    lib = _lib.load()
    cap = lib.fb_dot_product_noalloc_max_floats()
    assert cap == 4 * 1024 * 1024
    B, L, K = 2048, 32, 32     # 2*B*L*K*2 floats = 8 Mi > 4 Mi
    assert 4 * B * L * K > cap
    one = torch.zeros(1, device=DEV)
    ptrs = [one.data_ptr()] * 12
    rc = lib.fb_dot_product_noalloc_f32(*ptrs, B, L, L, 128, K, 1, _lib.FB_P2, 0.5, 1.0, _lib.FB_NATIVE, None)
    assert rc == 5  # FB_ERR_WORKSPACE, nothing launched
    torch.cuda.synchronize()
    # sizes whose product wraps around 64 bits must be refused too (2^31 - 1 cubed), not slip under the limit
    big = 2 ** 31 - 1
    rc = lib.fb_dot_product_noalloc_f32(*ptrs, big, big, big, 128, big, 1, _lib.FB_P2, 0.5, 1.0, _lib.FB_NATIVE, None)
    assert rc == 5
    torch.cuda.synchronize()
