"""Parity of the CUDA operators (through the C ABI) with the CPU oracle and the golden vectors."""
import math

import pytest
import torch

import cases
import helpers
from oracle import bounds_oracle as O

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def gpu_bounds(c, t):
    import faith_b200
    return faith_b200.BoundsLite(c["p"], c["eps"], t[0].to(DEV), t[1].to(DEV), t[2].to(DEV), t[3].to(DEV), c["words"],
                                 ibp=c.get("ibp", False))


def run_gpu_op(c):
    import types
    x_t, ex = cases.case_inputs(c)
    x = gpu_bounds(c, x_t)
    op = c["op"]
    if op == "concretize":
        l, u = x.concretize()
        return {"l": l, "u": u}
    if op in ("relu", "tanh", "exp", "reciprocal", "softmax", "sqr", "sqrt"):
        r = getattr(x, op)()
    elif op == "matmul":
        r = x.matmul(ex["W"].to(DEV))
    elif op == "dense":
        r = x.dense(types.SimpleNamespace(weight=ex["W"].to(DEV), bias=ex["bias"].to(DEV)))
    elif op == "dot":
        r = x.dot_product(gpu_bounds(c, ex["y"]))
    elif op == "context":
        r = x.context(gpu_bounds(c, ex["y"]))
    elif op == "mul_bounds":
        r = x.multiply(gpu_bounds(c, ex["y"]))
    elif op == "layer_norm":
        r = x.layer_norm(types.SimpleNamespace(weight=ex["W"].to(DEV), bias=ex["bias"].to(DEV)), "no_var")
    elif op == "layer_norm_std":
        r = x.layer_norm(types.SimpleNamespace(weight=ex["W"].to(DEV), bias=ex["bias"].to(DEV)), "standard")
    elif op == "mul_tensor":
        r = x.multiply(ex["W"].to(DEV))
    elif op == "scale":
        r = x.multiply(c["c"])
    elif op == "add":
        r = x.add(gpu_bounds(c, ex["y"]))
    else:
        raise KeyError(op)
    return {"lw": r.lw, "lb": r.lb, "uw": r.uw, "ub": r.ub}


@pytest.fixture(scope="module")
def golden_ops():
    return helpers.load_golden("ops.npz")


@pytest.mark.parametrize("name", sorted(cases.OP_CASES))
def test_op_matches_oracle_and_golden(name, golden_ops):
    c = cases.OP_CASES[name]
    got = run_gpu_op(c)
    ref = helpers.run_oracle_op(c)
    for k in ref:
        helpers.assert_close(got[k], ref[k], "%s/%s vs oracle" % (name, k))
        if c.get("golden", True):
            helpers.assert_close(got[k], golden_ops["%s/%s" % (name, k)], "%s/%s vs golden" % (name, k))


def _pair(seed, B, L, Di, Do, p, eps, words, shift=-0.7, wscale=0.2):
    import faith_b200
    t = cases.rand_bounds(seed, B, L, Di, Do, shift, wscale)
    return (O.OBounds(p, eps, *t, words=words),
            faith_b200.BoundsLite(p, eps, *[v.to(DEV) for v in t], perturbed_words=words))


def _cmp(g, o, what, **kw):
    for k in ("lw", "uw", "lb", "ub"):
        helpers.assert_close(getattr(g, k), getattr(o, k), "%s %s" % (what, k), **kw)


# shapes of the reference's own sweep (transformer_forward_test_bound.py:725-737), a ragged one,
# and shapes whose tile does / does not fit in shared memory
RELAX_SHAPES = [(1, 2, 64, 64), (1, 16, 128, 256), (2, 5, 256, 512), (1, 3, 24, 20), (1, 2, 7, 5),
                (1, 2, 1024, 96), (3, 1, 64, 1)]


@pytest.mark.parametrize("op", ["relu", "tanh", "exp"])
@pytest.mark.parametrize("shape", RELAX_SHAPES)
@pytest.mark.parametrize("p,words", [(2.0, 1), (float("inf"), 1), (1.0, 1)])
def test_relax_shapes(op, shape, p, words):
    o, g = _pair(101, *shape, p, 0.5, words)
    _cmp(getattr(g, op)(), getattr(o, op)(), "%s %s p=%s" % (op, shape, p))


def test_relax_words_blocks():
    for words in (2, 4):
        o, g = _pair(102, 2, 3, 64, 40, 2.0, 0.3, words)
        _cmp(g.relu(), o.relu(), "relu words=%d" % words)
        _cmp(g.tanh(), o.tanh(), "tanh words=%d" % words)


def test_reciprocal_and_violation_flag():
    o, g = _pair(103, 2, 4, 64, 48, 2.0, 0.05, 1, shift=1.0)
    _cmp(g.reciprocal(), o.reciprocal(), "reciprocal")
    o2, g2 = _pair(103, 2, 4, 64, 48, 2.0, 0.5, 1, shift=-0.5)  # ranges that reach below zero
    with pytest.raises(AssertionError):
        o2.reciprocal()
    with pytest.raises(AssertionError):
        g2.reciprocal()


def test_relu_all_three_column_kinds_present():
    o, g = _pair(104, 1, 4, 64, 128, 2.0, 0.5, 1)
    l, u = o.concretize()
    assert bool((l > 0).any()) and bool((u < 0).any()) and bool(((l <= 0) & (u >= 0)).any())
    gl, gu = g.concretize()
    helpers.assert_close(gl, l, "concretize l")
    helpers.assert_close(gu, u, "concretize u")


def test_empty_batch_is_a_no_op():
    import faith_b200
    z4 = torch.zeros(0, 3, 8, 8, device=DEV)
    z3 = torch.zeros(0, 3, 8, device=DEV)
    r = faith_b200.BoundsLite(2, 0.1, z4, z3, z4.clone(), z3.clone()).relu()
    assert r.lw.shape == (0, 3, 8, 8)


def test_unwritten_outputs_are_detected():
    """Outputs pre-filled with NaN must be fully overwritten (catches unwritten tails)."""
    from faith_b200 import ops
    from faith_b200._lib import FB_RELU
    t = [v.to(DEV) for v in cases.rand_bounds(105, 2, 3, 24, 20, -0.7, 0.2)]
    out = tuple(torch.full_like(v, float("nan")) for v in (t[0], t[2], t[1], t[3]))
    ops.relax(FB_RELU, t[0], t[2], t[1], t[3], 2.0, 0.5, out=out)
    for v in out:
        assert bool(torch.isfinite(v).all())


def test_dot_product_tensor_core_shapes_match_fp64_and_repeat():
    """Attention shapes (K = 32, Ly = 32, Lx a multiple of 32, Di a multiple of 4) take the tcgen05
    kernel.  The weight part is checked against an fp64 evaluation of the centre/radius formula
    (tolerance: the per-operator bar with the absolute part scaled to the size of the summed terms)
    and repeated launches must agree bit for bit."""
    from faith_b200 import ops
    for B, Lx, Di in ((8, 32, 128), (4, 64, 64), (3, 32, 12)):
        g0 = torch.Generator().manual_seed(17 + B)
        def mk(L):
            lw = torch.randn(B, L, Di, 32, generator=g0) * 0.3
            uw = lw + torch.rand(B, L, Di, 32, generator=g0) * 0.1
            lb = torch.randn(B, L, 32, generator=g0)
            ub = lb + torch.rand(B, L, 32, generator=g0) * 0.1
            return [t.to(DEV) for t in (lw, uw, lb, ub)]
        x, y = mk(Lx), mk(32)
        first = ops.dot_product(x, y, float("inf"), 0.01, 1, 0.25)
        for _ in range(5):
            again = ops.dot_product(x, y, float("inf"), 0.01, 1, 0.25)
            for a, b in zip(first, again):
                assert torch.equal(a, b)
        X = [t.double() for t in x]
        Y = [t.double() for t in y]
        xl = X[2] - 0.01 * X[0].abs().sum(2)
        yl = Y[2] - 0.01 * Y[0].abs().sum(2)
        yu = Y[3] + 0.01 * Y[1].abs().sum(2)
        xc, xr, yc, yr = (X[0] + X[1]) / 2, (X[1] - X[0]) / 2, (Y[0] + Y[1]) / 2, (Y[1] - Y[0]) / 2
        P = torch.einsum("bjmk,bik->bimj", yc, xl)
        Q = torch.einsum("bjmk,bik->bimj", yr, xl.abs())
        zl = torch.einsum("bimk,bjk->bimj", xc, yl) - torch.einsum("bimk,bjk->bimj", xr, yl.abs()) + P - Q
        zu = torch.einsum("bimk,bjk->bimj", xc, yu) + torch.einsum("bimk,bjk->bimj", xr, yu.abs()) + P + Q
        # the same formula evaluated in fp32 by the oracle's dot product gives the noise the fp64 value is the arbiter of
        o32 = O.OBounds(float("inf"), 0.01, x[0].cpu(), x[2].cpu(), x[1].cpu(), x[3].cpu()).dot_product(
            O.OBounds(float("inf"), 0.01, y[0].cpu(), y[2].cpu(), y[1].cpu(), y[3].cpu()))
        helpers.assert_arbitrated(first[0], o32.lw * 0.25, zl * 0.25, "tcgen05 dot product lw")
        helpers.assert_arbitrated(first[1], o32.uw * 0.25, zu * 0.25, "tcgen05 dot product uw")


def test_context_with_values_in_projection_layout_matches_transposed_path():
    """fb_context_heads_f32 (values as [B, K, Di, Ly]) against fb_dot_product with the transposed copy
    of the same values, with and without the head merge; shapes outside the kernel are refused."""
    from faith_b200 import ops, _lib
    B, L, Di, d, H = 8, 32, 64, 32, 4
    g0 = torch.Generator().manual_seed(23)
    def mk(shape_w, shape_b, s):
        lw = torch.randn(*shape_w, generator=g0) * s
        uw = lw + torch.rand(*shape_w, generator=g0) * 0.05
        lb = torch.rand(*shape_b, generator=g0)
        ub = lb + torch.rand(*shape_b, generator=g0) * 0.05
        return [t.to(DEV) for t in (lw, uw, lb, ub)]
    x = mk((B, L, Di, L), (B, L, L), 0.05)          # probabilities [B, Lx, Di, K]
    v = mk((B, L, Di, d), (B, L, d), 0.3)           # values [B, K, Di, Ly]
    vt = [v[0].permute(0, 3, 2, 1).contiguous(), v[1].permute(0, 3, 2, 1).contiguous(),
          v[2].permute(0, 2, 1).contiguous(), v[3].permute(0, 2, 1).contiguous()]
    ref = ops.dot_product(x, vt, 2.0, 0.02, 2, 1.0)
    got = ops.context_kmajor(x, v, 2.0, 0.02, 2, 1.0, 1)
    for a, b, name in zip(got, ref, ("lw", "uw", "lb", "ub")):
        helpers.assert_close(a, b.cpu(), "context " + name, rtol=1e-6, atol=1e-7)
    merged = ops.context_kmajor(x, v, 2.0, 0.02, 2, 1.0, H)
    m_ref = ops.merge_heads(ref, H)
    for a, b, name in zip(merged, m_ref, ("lw", "uw", "lb", "ub")):
        helpers.assert_close(a, b.cpu(), "merged context " + name, rtol=1e-6, atol=1e-7)
    x48 = mk((B, 48, Di, L), (B, 48, L), 0.05)
    with pytest.raises(_lib.FaithError):
        ops.context_kmajor(x48, v, 2.0, 0.02, 2, 1.0, 1)


# ------------------------------------------------------------------ matmul
@pytest.mark.parametrize("shape,Dy", [((1, 2, 64, 64), 64), ((1, 16, 64, 64), 128), ((2, 8, 128, 256), 512),
                                      ((1, 3, 24, 20), 7), ((1, 5, 33, 130), 129), ((1, 4, 64, 128), 2),
                                      ((1, 1, 128, 512), 128),
                                      # narrow output, long contraction (the head of the CNN): many rows through the
                                      # chunked kernel (K a multiple of its 512-chunk, and not), one row (the bias
                                      # part of every call here) through the block-per-row kernel
                                      ((1, 1, 96, 4096), 10), ((1, 2, 40, 2308), 16), ((1, 1, 3, 8192), 10)])
def test_matmul_shapes(shape, Dy):
    import types
    B, L, Di, Do = shape
    g0 = torch.Generator().manual_seed(7)
    t = cases.rand_bounds(201, B, L, Di, Do, 0.0, 1.0)
    # weights with the spread of a trained layer: variance 1/fan_in
    W = torch.randn(Dy, Do, generator=g0) / math.sqrt(Do)
    bias = torch.randn(Dy, generator=g0) * 0.1
    import faith_b200
    o = O.OBounds(2.0, 0.5, *t).dense(W, bias)
    g = faith_b200.BoundsLite(2.0, 0.5, *[v.to(DEV) for v in t]).dense(
        types.SimpleNamespace(weight=W.to(DEV), bias=bias.to(DEV)))
    # fp32 GEMMs with different summation order: judged against the fp64 run of the same algorithm
    o64 = O.OBounds(2.0, 0.5, *[v.double() for v in t]).dense(W.double(), bias.double())
    helpers.assert_bounds_arbitrated(g, o, o64, "dense %s->%d" % (shape, Dy))


def test_matmul_tensor_core_stage_reuse_is_race_free():
    """Every k-block contributes a distinct power of two, so the exact result tells which k-block's
    data each product saw; repeated launches must agree bit for bit.  K = 512 walks each
    shared-memory / tensor-memory stage eight times (a release of a raw stage ahead of the
    completion of the loads from it showed up here as rows that carried the data of k-block it+2)."""
    from faith_b200 import ops
    rows, Di, Do, Dy = 16, 128, 512, 512
    kb = torch.arange(Do, device=DEV) // 32
    x = (2.0 ** kb.float()).expand(1, rows, Di, Do).contiguous()
    zb = torch.zeros(1, rows, Do, device=DEV)
    W = torch.ones(Dy, Do, device=DEV)
    expect = 32.0 * (2 ** (Do // 32) - 1)
    for _ in range(10):
        y_lw, y_uw, y_lb, y_ub = ops.matmul(x, x, zb, zb, W, None)
        assert bool((y_lw == expect).all()) and bool((y_uw == expect).all())
    g0 = torch.Generator().manual_seed(11)
    lw = torch.randn(1, rows, Di, Do, generator=g0).to(DEV)
    uw = lw + torch.rand(1, rows, Di, Do, generator=g0).to(DEV)
    Wr = (torch.randn(Dy, Do, generator=g0) / math.sqrt(Do)).to(DEV)
    first = ops.matmul(lw, uw, zb, zb, Wr, None)
    for _ in range(10):
        again = ops.matmul(lw, uw, zb, zb, Wr, None)
        for a, b in zip(first, again):
            assert torch.equal(a, b)


@pytest.mark.parametrize("op_name", ["relu", "tanh"])
@pytest.mark.parametrize("p,words,Di", [(float("inf"), 1, 128), (2.0, 2, 256)])
def test_relaxation_applied_by_the_following_product(op_name, p, words, Di):
    """fb_relax_coef_f32 + fb_matmul_coef_f32 (slopes applied while the product reads its operands) must
    reproduce fb_relax_f32 followed by fb_matmul_f32 bit for bit; shapes outside the kernel are refused."""
    from faith_b200 import ops, _lib
    op = {"relu": _lib.FB_RELU, "tanh": _lib.FB_TANH}[op_name]
    B, L, Do, Dy = 2, 5, 96, 72
    t = cases.rand_bounds(91, B, L, Di, Do, -0.4, 0.6)
    g0 = torch.Generator().manual_seed(6)
    W = (torch.randn(Dy, Do, generator=g0) / math.sqrt(Do)).to(DEV)
    bias = (torch.randn(Dy, generator=g0) * 0.1).to(DEV)
    lw, lb, uw, ub = [v.to(DEV) for v in t]
    eps = 0.05
    r = ops.relax(op, lw, uw, lb, ub, p, eps, words)
    ref = ops.matmul(r[0], r[1], r[2], r[3], W, bias)
    c_l, c_u, nlb, nub = ops.relax_coef(op, lw, uw, lb, ub, p, eps, words)
    assert torch.equal(nlb, r[2]) and torch.equal(nub, r[3])
    got = ops.matmul_coef(lw, uw, nlb, nub, c_l, c_u, W, bias)
    for a, b, name in zip(got, ref, ("lw", "uw", "lb", "ub")):
        assert torch.equal(a, b), name
    with pytest.raises(_lib.FaithError):   # dim_in not a multiple of 128
        ops.matmul_coef(lw[:, :, :64].contiguous(), uw[:, :, :64].contiguous(), nlb, nub, c_l, c_u, W, bias)


def test_matmul_identity_input():
    """First-layer case: lw = uw = one-hot rows, so every output is a single product 1 * w.  The
    CUDA-core kernel reproduces the reference bit for bit; the tensor-core kernel carries the
    weight as two TF32 parts (22 mantissa bits), i.e. within 2^-21 relative."""
    import faith_b200
    D = 64
    lw = torch.zeros(1, 4, D, D)
    lw[0, 1] = torch.eye(D)
    emb = torch.randn(1, 4, D, generator=torch.Generator().manual_seed(3))
    W = torch.randn(128, D, generator=torch.Generator().manual_seed(4)) / 8
    o = O.OBounds(2.0, 0.1, lw, emb, lw.clone(), emb.clone()).matmul(W)
    g = faith_b200.BoundsLite(2.0, 0.1, lw.to(DEV), emb.to(DEV), lw.to(DEV), emb.to(DEV)).matmul(W.to(DEV))
    helpers.assert_close(g.lw, o.lw, "lw", rtol=2.0 ** -21, atol=0.0)
    helpers.assert_close(g.uw, o.uw, "uw", rtol=2.0 ** -21, atol=0.0)
    assert torch.equal(g.lw, g.uw)          # radius is exactly zero when lw == uw
    helpers.assert_close(g.lb, o.lb, "lb")  # the 4-row bias GEMM runs on the CUDA cores


def test_tensor_core_gemm_never_raised_its_error_flag():
    import ctypes
    import faith_b200
    flag = ctypes.c_int(-1)
    assert faith_b200.load().fb_tc_error_flag(ctypes.byref(flag)) == 0
    assert flag.value == 0


# ------------------------------------------------------------- dot product
@pytest.mark.parametrize("B,Lx,Ly,Di,K", [(1, 2, 2, 64, 16), (4, 32, 32, 128, 32), (2, 8, 8, 64, 64),
                                          (1, 5, 7, 24, 10), (2, 33, 9, 36, 130), (1, 16, 16, 256, 512),
                                          # a few query rows: the thread-per-output kernel
                                          (8, 1, 32, 128, 32), (3, 4, 9, 20, 33), (2, 3, 40, 64, 7)])
@pytest.mark.parametrize("p", [2.0, float("inf")])
def test_dot_product_shapes(B, Lx, Ly, Di, K, p):
    import faith_b200
    tx = cases.rand_bounds(301, B, Lx, Di, K, -0.5, 1.0)
    ty = cases.rand_bounds(302, B, Ly, Di, K, -0.5, 1.0)
    o = O.OBounds(p, 0.5, *tx).dot_product(O.OBounds(p, 0.5, *ty))
    g = faith_b200.BoundsLite(p, 0.5, *[v.to(DEV) for v in tx]).dot_product(
        faith_b200.BoundsLite(p, 0.5, *[v.to(DEV) for v in ty]))
    # The K-term sums reach 1e2..1e4 (operand ranges of a few units times K terms) and cancel, so two
    # fp32 evaluation orders (the reference's four separate GEMMs, the kernel's fused centre/radius
    # accumulation) differ by more than the per-operator bar near zeros of the result.  The result is
    # therefore judged, element by element, against the fp64 run of the same algorithm: within 4x the fp32 noise
    # of the reference itself on top of the per-operator bar.
    d = torch.float64
    o64 = O.OBounds(p, 0.5, *[v.to(d) for v in tx]).dot_product(O.OBounds(p, 0.5, *[v.to(d) for v in ty]))
    helpers.assert_bounds_arbitrated(g, o, o64, "dot K=%d" % K)


def test_context_matches_oracle():
    import faith_b200
    B, L, Di, d = 4, 32, 128, 32
    tp = cases.rand_bounds(303, B, L, Di, L, 0.0, 0.2)
    tv = cases.rand_bounds(304, B, L, Di, d, -0.5, 1.0)
    o = O.OBounds(2.0, 0.1, *tp).context(O.OBounds(2.0, 0.1, *tv))
    g = faith_b200.BoundsLite(2.0, 0.1, *[v.to(DEV) for v in tp]).context(
        faith_b200.BoundsLite(2.0, 0.1, *[v.to(DEV) for v in tv]))
    o64 = O.OBounds(2.0, 0.1, *[v.double() for v in tp]).context(O.OBounds(2.0, 0.1, *[v.double() for v in tv]))
    helpers.assert_bounds_arbitrated(g, o, o64, "context")


def test_split_merge_heads_round_trip():
    from faith_b200 import ops
    B, L, Di, H, d = 2, 5, 12, 4, 8
    t = [v.to(DEV) for v in cases.rand_bounds(305, B, L, Di, H * d)]
    x = (t[0], t[2], t[1], t[3])
    o = O.split_heads(O.OBounds(2.0, 0.1, *[v.cpu() for v in (t[0], t[1], t[2], t[3])]), H)
    s = ops.split_heads(x, H)
    assert torch.equal(s[0].cpu(), o.lw) and torch.equal(s[3].cpu(), o.ub)
    st = ops.split_heads(x, H, transpose_ld=True)
    assert torch.equal(st[0].cpu(), o.lw.transpose(1, 3).contiguous())
    assert torch.equal(st[2].cpu(), o.lb.transpose(1, 2).contiguous())
    m = ops.merge_heads(s, H)
    for a, b in zip(m, x):
        assert torch.equal(a, b)


# ------------------------------------------------- reference pybind surface
def test_c_bound_relu_tanh_transposed_layout():
    from faith_b200 import c_bound
    for fn, name in ((c_bound.c_relu_verification, "relu"), (c_bound.c_tanh_verification, "tanh")):
        for (B, L, Di, Do) in [(1, 2, 64, 64), (1, 8, 128, 256), (2, 3, 20, 12)]:
            t = cases.rand_bounds(401, B, L, Di, Do, -0.7, 0.2)
            o = getattr(O.OBounds(2.0, 0.5, *t), name)()
            lw, lb, uw, ub = [v.to(DEV) for v in t]
            tl, tu = lw.transpose(2, 3).contiguous(), uw.transpose(2, 3).contiguous()
            o_lw, o_uw = torch.zeros_like(tl), torch.zeros_like(tu)
            o_lb, o_ub = torch.zeros_like(lb), torch.zeros_like(ub)
            fn(lb, ub, tl, tu, o_lb, o_ub, o_lw, o_uw, L, Di, Do, 0.5)
            helpers.assert_close(o_lw.transpose(2, 3), o.lw, name + " lw")
            helpers.assert_close(o_uw.transpose(2, 3), o.uw, name + " uw")
            helpers.assert_close(o_lb, o.lb, name + " lb")
            helpers.assert_close(o_ub, o.ub, name + " ub")


@pytest.mark.parametrize("B,L,Di,K", [(1, 2, 64, 16), (2, 8, 64, 64), (4, 16, 128, 16), (1, 5, 24, 10)])
def test_c_bound_dot_product_qk(B, L, Di, K):
    from faith_b200 import c_bound
    tx = cases.rand_bounds(402, B, L, Di, K, -0.5, 1.0)
    ty = cases.rand_bounds(403, B, L, Di, K, -0.5, 1.0)
    ox, oy = O.OBounds(2.0, 0.5, *tx), O.OBounds(2.0, 0.5, *ty)
    o = ox.dot_product(oy)
    x = [v.to(DEV) for v in tx]
    y = [v.to(DEV) for v in ty]
    z_lw = torch.zeros(B, L, L, Di, device=DEV)
    z_uw = torch.zeros_like(z_lw)
    z_lb = torch.zeros(B, L, L, device=DEV)
    z_ub = torch.zeros_like(z_lb)
    x_l, x_u, y_l, y_u = (torch.zeros(B, L, K, device=DEV) for _ in range(4))
    c_bound.c_dot_product_verification_QK(
        x_l, y_l, x_u, y_u, x[1], x[3], y[1], y[3],
        x[0].transpose(2, 3).contiguous(), x[2].transpose(2, 3).contiguous(),
        y[0].transpose(2, 3).contiguous(), y[2].transpose(2, 3).contiguous(),
        z_lb, z_ub, z_lw, z_uw, B, L, K, Di, 0.5)
    o64 = O.OBounds(2.0, 0.5, *[v.double() for v in tx]).dot_product(O.OBounds(2.0, 0.5, *[v.double() for v in ty]))
    helpers.assert_arbitrated(z_lw.transpose(2, 3), o.lw, o64.lw, "c_bound qk lw")
    helpers.assert_arbitrated(z_uw.transpose(2, 3), o.uw, o64.uw, "c_bound qk uw")
    helpers.assert_arbitrated(z_lb, o.lb, o64.lb, "c_bound qk lb")
    helpers.assert_arbitrated(z_ub, o.ub, o64.ub, "c_bound qk ub")
    # the caller-visible scratch receives the concretised operand ranges
    lx, ux = ox.concretize()
    ly, uy = oy.concretize()
    helpers.assert_close(x_l, lx, "x_l"); helpers.assert_close(x_u, ux, "x_u")
    helpers.assert_close(y_l, ly, "y_l"); helpers.assert_close(y_u, uy, "y_u")


@pytest.mark.parametrize("B,L,Di,Dout", [(1, 2, 64, 10), (2, 8, 64, 20), (4, 16, 128, 64)])
def test_c_bound_dot_product_v(B, L, Di, Dout):
    from faith_b200 import c_bound
    tp = cases.rand_bounds(404, B, L, Di, L, 0.0, 0.2)          # probabilities [B, L, Di, L]
    tv = cases.rand_bounds(405, B, Dout, Di, L, -0.5, 1.0)      # value.t()     [B, Dout, Di, L]
    o = O.OBounds(2.0, 0.5, *tp).dot_product(O.OBounds(2.0, 0.5, *tv))
    x = [v.to(DEV) for v in tp]
    y = [v.to(DEV) for v in tv]
    z_lw = torch.zeros(B, L, Dout, Di, device=DEV)
    z_uw = torch.zeros_like(z_lw)
    z_lb = torch.zeros(B, L, Dout, device=DEV)
    z_ub = torch.zeros_like(z_lb)
    x_l, x_u = torch.zeros(B, L, L, device=DEV), torch.zeros(B, L, L, device=DEV)
    y_l, y_u = torch.zeros(B, Dout, L, device=DEV), torch.zeros(B, Dout, L, device=DEV)
    c_bound.c_dot_product_verification_V(
        x_l, y_l, x_u, y_u, x[1], x[3], y[1], y[3],
        x[0].transpose(2, 3).contiguous(), x[2].transpose(2, 3).contiguous(),
        y[0].transpose(2, 3).contiguous(), y[2].transpose(2, 3).contiguous(),
        z_lb, z_ub, z_lw, z_uw, B, L, Dout, Di, 0.5)
    o64 = O.OBounds(2.0, 0.5, *[v.double() for v in tp]).dot_product(O.OBounds(2.0, 0.5, *[v.double() for v in tv]))
    helpers.assert_arbitrated(z_lw.transpose(2, 3), o.lw, o64.lw, "c_bound v lw")
    helpers.assert_arbitrated(z_uw.transpose(2, 3), o.uw, o64.uw, "c_bound v uw")
    helpers.assert_arbitrated(z_lb, o.lb, o64.lb, "c_bound v lb")
    helpers.assert_arbitrated(z_ub, o.ub, o64.ub, "c_bound v ub")


def test_c_bound_matmul():
    from faith_b200 import c_bound
    B, L, Di, Do, Dy = 1, 4, 64, 64, 64
    t = cases.rand_bounds(406, B, L, Di, Do)
    W = (torch.rand(Dy, Do, generator=torch.Generator().manual_seed(0)) - 0.5) / 4
    o = O.OBounds(2.0, 0.5, *t).matmul(W)
    lw, lb, uw, ub = [v.to(DEV) for v in t]
    y_lw = torch.zeros(B, L, Di, Dy, device=DEV); y_uw = torch.zeros_like(y_lw)
    y_lb = torch.zeros(B, L, Dy, device=DEV); y_ub = torch.zeros_like(y_lb)
    c_bound.c_matmul_verification(lb, ub, lw, uw, W.to(DEV), y_lb, y_ub, y_lw, y_uw, B, L, Di, Do, Dy)
    o64 = O.OBounds(2.0, 0.5, *[v.double() for v in t]).matmul(W.double())
    for got, k in ((y_lw, "lw"), (y_uw, "uw"), (y_lb, "lb"), (y_ub, "ub")):
        helpers.assert_arbitrated(got, getattr(o, k), getattr(o64, k), "c_bound matmul " + k)


# ------------------------------------------------------------------- conv
@pytest.mark.parametrize("cfg", [dict(B=1, Di=12, C=3, H=32, W=32, Co=16, k=3, s=1, p=1),
                                 dict(B=2, Di=5, C=16, H=32, W=32, Co=32, k=3, s=2, p=1),
                                 dict(B=1, Di=3, C=5, H=9, W=11, Co=7, k=3, s=1, p=0),
                                 dict(B=1, Di=4, C=2, H=8, W=8, Co=20, k=5, s=2, p=2)])
def test_conv_bounds(cfg):
    from faith_b200 import ops
    g = torch.Generator().manual_seed(501)
    B, Di, C, H, W = cfg["B"], cfg["Di"], cfg["C"], cfg["H"], cfg["W"]
    lw = torch.rand(B, Di, C, H, W, generator=g) - 0.5
    uw = torch.rand(B, Di, C, H, W, generator=g) - 0.5
    lb = torch.rand(B, C, H, W, generator=g)
    ub = lb + torch.rand(B, C, H, W, generator=g)
    wt = torch.randn(cfg["Co"], C, cfg["k"], cfg["k"], generator=g) * math.sqrt(2.0 / (C * cfg["k"] ** 2))
    bias = torch.randn(cfg["Co"], generator=g) * 0.1
    o = O.conv_bounds(O.OBounds(float("inf"), 0.01, lw, lb, uw, ub), wt, bias, cfg["s"], cfg["p"])
    r = ops.conv2d((lw.to(DEV), uw.to(DEV), lb.to(DEV), ub.to(DEV)), wt.to(DEV), bias.to(DEV), cfg["s"], cfg["p"])
    o64 = O.conv_bounds(O.OBounds(float("inf"), 0.01, lw.double(), lb.double(), uw.double(), ub.double()), wt.double(),
                        bias.double(), cfg["s"], cfg["p"])
    what = "conv %dx%d s%d" % (cfg["k"], cfg["k"], cfg["s"])
    for got, k in zip(r, ("lw", "uw", "lb", "ub")):
        helpers.assert_arbitrated(got, getattr(o, k), getattr(o64, k), what + " " + k)


@pytest.mark.parametrize("C,H,W,Co,k,s,p", [(16, 32, 32, 32, 3, 2, 1), (3, 32, 32, 16, 3, 1, 1), (5, 9, 11, 7, 3, 1, 0),
                                           (2, 8, 8, 20, 5, 2, 2)])
def test_conv_of_a_few_images_equals_the_tiled_kernel_bit_for_bit(C, H, W, Co, k, s, p):
    """One image goes through the thread-per-output kernel, many through the tiled one: same accumulation order, same
    bits (the image is row 0 of a batch of 600 copies in the second call)."""
    from faith_b200 import ops
    g = torch.Generator().manual_seed(503)
    lo = torch.rand(1, 1, C, H, W, generator=g) - 0.5
    up = lo + torch.rand(1, 1, C, H, W, generator=g) * 0.3
    wt = (torch.randn(Co, C, k, k, generator=g) * 0.3).to(DEV)
    bias = (torch.randn(Co, generator=g) * 0.1).to(DEV)
    one = ops.conv2d((lo.to(DEV), up.to(DEV), lo[0].to(DEV), up[0].to(DEV)), wt, bias, s, p)
    n = 600
    many = ops.conv2d((lo.expand(1, n, C, H, W).contiguous().to(DEV), up.expand(1, n, C, H, W).contiguous().to(DEV),
                       lo[0].to(DEV), up[0].to(DEV)), wt, bias, s, p)
    assert torch.equal(one[0][0, 0], many[0][0, 0]) and torch.equal(one[1][0, 0], many[1][0, 0])
    assert torch.equal(one[0][0, 0], many[0][0, n - 1])
    # the bias part of both calls is one image (small kernel); without the bias it equals the weight part
    assert torch.equal(one[2] - bias.view(1, -1, 1, 1), one[0][0]) or float((one[2] - bias.view(1, -1, 1, 1) - one[0][0]).abs().max()) < 1e-6


def test_context_of_a_single_query_row_reads_the_values_in_projection_layout():
    """fb_context_given_f32 with Lx = 1 (a last layer run for the first token only): the thread-per-output kernel with the
    values as [B, K, Di, Ly] against the dot product with the transposed copy, head-merged store included."""
    from faith_b200 import ops
    B, L, Di, d, H = 8, 32, 64, 32, 4
    g0 = torch.Generator().manual_seed(24)

    def mk(shape_w, shape_b, sc):
        lw = torch.randn(*shape_w, generator=g0) * sc
        uw = lw + torch.rand(*shape_w, generator=g0) * 0.05
        lb = torch.rand(*shape_b, generator=g0)
        ub = lb + torch.rand(*shape_b, generator=g0) * 0.05
        return [t.to(DEV) for t in (lw, uw, lb, ub)]
    x = mk((B, 1, Di, L), (B, 1, L), 0.05)           # probabilities of one query row [B, 1, Di, K]
    v = mk((B, L, Di, d), (B, L, d), 0.3)            # values [B, K, Di, Ly]
    vt = [v[0].permute(0, 3, 2, 1).contiguous(), v[1].permute(0, 3, 2, 1).contiguous(),
          v[2].permute(0, 2, 1).contiguous(), v[3].permute(0, 2, 1).contiguous()]
    ref = ops.dot_product(x, vt, 2.0, 0.02, 2, 1.0)
    got = ops.context_kmajor(x, v, 2.0, 0.02, 2, 1.0, 1)
    for a, b, name in zip(got, ref, ("lw", "uw", "lb", "ub")):
        helpers.assert_close(a, b.cpu(), "single-row context " + name, rtol=1e-6, atol=1e-7)
    merged = ops.context_kmajor(x, v, 2.0, 0.02, 2, 1.0, H)
    m_ref = ops.merge_heads(ref, H)
    for a, b, name in zip(merged, m_ref, ("lw", "uw", "lb", "ub")):
        helpers.assert_close(a, b.cpu(), "single-row merged context " + name, rtol=1e-6, atol=1e-7)


def test_dot_product_with_merged_head_store():
    """fb_dot_product_heads_f32 writes the context head-merged; same values as dot product + merge."""
    from faith_b200 import _lib, ops
    lib = _lib.load()
    S, H, L, Di, d = 2, 4, 8, 16, 12
    tp = [v.to(DEV) for v in cases.rand_bounds(601, S * H, L, Di, L, 0.0, 0.2)]
    tv = [v.to(DEV) for v in cases.rand_bounds(602, S * H, d, Di, L, -0.5, 1.0)]
    x = (tp[0], tp[2], tp[1], tp[3])
    y = (tv[0], tv[2], tv[1], tv[3])
    ref = ops.merge_heads(ops.dot_product(x, y, 2.0, 0.1), H)
    z = [torch.full((S, L, Di, H * d), float("nan"), device=DEV), torch.full((S, L, Di, H * d), float("nan"), device=DEV),
         torch.full((S, L, H * d), float("nan"), device=DEV), torch.full((S, L, H * d), float("nan"), device=DEV)]
    scr = [torch.empty(S * H, L, L, device=DEV), torch.empty(S * H, L, L, device=DEV),
           torch.empty(S * H, d, L, device=DEV), torch.empty(S * H, d, L, device=DEV)]
    ptrs = [t.data_ptr() for t in x + y] + [t.data_ptr() for t in z] + [t.data_ptr() for t in scr]
    _lib.check(lib.fb_dot_product_heads_f32(*ptrs, S * H, L, d, Di, L, 1, _lib.FB_P2, 0.1, 1.0, _lib.FB_NATIVE, H,
                                            torch.cuda.current_stream().cuda_stream), "fb_dot_product_heads_f32")
    for a, b in zip(z, ref):
        assert torch.equal(a, b)


@pytest.mark.parametrize("S,L,Di,H,d", [(2, 8, 32, 2, 32), (3, 4, 64, 4, 64), (2, 5, 12, 4, 8)])
def test_matmul_with_head_split_store(S, L, Di, H, d):
    """fb_matmul_heads_f32 (tensor-core TMA store or CUDA-core path) equals dense followed by the split."""
    from faith_b200 import _lib, ops
    lib = _lib.load()
    D = H * d
    t = [v.to(DEV) for v in cases.rand_bounds(603, S, L, Di, D)]
    g = torch.Generator().manual_seed(9)
    W = (torch.randn(D, D, generator=g) / math.sqrt(D)).to(DEV)
    bias = (torch.randn(D, generator=g) * 0.1).to(DEV)
    y = ops.matmul(t[0], t[2], t[1], t[3], W, bias)
    ref = ops.split_heads(y, H)
    z = [torch.full((S * H, L, Di, d), float("nan"), device=DEV), torch.full((S * H, L, Di, d), float("nan"), device=DEV),
         torch.full((S * H, L, d), float("nan"), device=DEV), torch.full((S * H, L, d), float("nan"), device=DEV)]
    _lib.check(lib.fb_matmul_heads_f32(t[0].data_ptr(), t[2].data_ptr(), t[1].data_ptr(), t[3].data_ptr(), W.data_ptr(),
                                       bias.data_ptr(), *[v.data_ptr() for v in z], S * L, Di, D, D, L, H,
                                       torch.cuda.current_stream().cuda_stream), "fb_matmul_heads_f32")
    for a, b in zip(z, ref):
        assert torch.equal(a, b)


@pytest.mark.parametrize("shape", [(4, 32, 128, 32), (2, 3, 64, 8), (1, 5, 40, 20)])
@pytest.mark.parametrize("p,words", [(2.0, 1), (float("inf"), 1), (1.0, 2)])
def test_fused_softmax_matches_oracle_and_chain(shape, p, words):
    """The fused softmax kernel against the oracle and against the four-kernel chain it replaces."""
    import faith_b200
    from faith_b200 import ops
    B, L, Di, Do = shape
    t = cases.rand_bounds(604, B, L, Di, Do, -0.5, 0.2)
    o = O.OBounds(p, 0.1, *t, words=words).softmax()
    g = faith_b200.BoundsLite(p, 0.1, *[v.to(DEV) for v in t], perturbed_words=words)
    fused = ops.softmax_fused(g._t4(), p, 0.1, words)
    assert fused is not None
    e = g.exp()
    s = ops.rowsum(e._t4())
    chain = e.divide(g._new(s[0], s[1], s[2], s[3]))
    for k, i in (("lw", 0), ("uw", 1), ("lb", 2), ("ub", 3)):
        helpers.assert_close(fused[i], getattr(o, k), "fused softmax %s vs oracle" % k)
        helpers.assert_close(fused[i], getattr(chain, k), "fused softmax %s vs chain" % k)


@pytest.mark.parametrize("p,words,S", [(float("inf"), 1, 2), (2.0, 1, 2), (1.0, 1, 2), (2.0, 2, 2), (float("inf"), 2, 2),
                                       (float("inf"), 1, 8), (2.0, 2, 8)])
def test_projection_returns_ranges_for_the_dot_product(p, words, S):
    """fb_matmul_heads_ranges_f32: same bounds as fb_matmul_heads_f32 bit for bit, ranges equal to a
    concretisation pass over them, and the dot product / context product fed with those ranges
    (fb_dot_product_given_f32, fb_context_given_f32) equal to the ones that concretise themselves."""
    from faith_b200 import _lib, ops
    lib = _lib.load()
    L, H, d = 32, 4, 32     # S = 8: 256 bias rows, which then also go through the tensor-core kernel
    D, Di, eps = H * d, 128 * words, 0.05
    st = torch.cuda.current_stream().cuda_stream
    g = torch.Generator().manual_seed(11)

    def project(seed):
        t = [v.to(DEV) for v in cases.rand_bounds(seed, S, L, Di, D)]
        W = (torch.randn(D, D, generator=g) / math.sqrt(D)).to(DEV)
        bias = (torch.randn(D, generator=g) * 0.1).to(DEV)
        y = ops.matmul_heads_ranges(t[0], t[2], t[1], t[3], W, bias, H, p, eps, words)
        z = [torch.empty_like(y[0]), torch.empty_like(y[0]), torch.empty_like(y[2]), torch.empty_like(y[2])]
        _lib.check(lib.fb_matmul_heads_f32(t[0].data_ptr(), t[2].data_ptr(), t[1].data_ptr(), t[3].data_ptr(), W.data_ptr(),
                                           bias.data_ptr(), *[v.data_ptr() for v in z], S * L, Di, D, D, L, H, st),
                   "fb_matmul_heads_f32")
        assert torch.equal(y[0], z[0]) and torch.equal(y[1], z[1])
        if S * L < 256:
            assert torch.equal(y[2], z[2]) and torch.equal(y[3], z[3])
        else:   # bias rows on the tensor cores (3xTF32) here, on the CUDA cores in fb_matmul_heads_f32
            helpers.assert_close(y[2], z[2], "lb", atol=2e-6)
            helpers.assert_close(y[3], z[3], "ub", atol=2e-6)
        l, u = ops.concretize(y[0], y[1], y[2], y[3], p, eps, words)
        helpers.assert_close(y[4], l, "range l from the GEMM epilogue")
        helpers.assert_close(y[5], u, "range u from the GEMM epilogue")
        return y

    q, k = project(701), project(702)
    B = S * H

    def run(fn, name, x, y, zshape, zbshape, ranges, extra):
        z = [torch.full(zshape, float("nan"), device=DEV), torch.full(zshape, float("nan"), device=DEV),
             torch.full(zbshape, float("nan"), device=DEV), torch.full(zbshape, float("nan"), device=DEV)]
        ptrs = [t.data_ptr() for t in x[:4]] + [t.data_ptr() for t in y[:4]] + [t.data_ptr() for t in z] + \
               [t.data_ptr() for t in ranges]
        _lib.check(fn(*ptrs, *extra, st), name)
        return z

    # The products fed with ranges (here: the ones a concretisation pass computes, so that the comparison
    # is exact) equal the products that concretise themselves, and the given ranges stay untouched.
    def conc(b):
        return [v.contiguous() for v in ops.concretize(b[0], b[1], b[2], b[3], p, eps, words)]

    ql, qu = conc(q)
    kl, ku = conc(k)
    rg = [ql.clone(), qu.clone(), kl.clone(), ku.clone()]
    rs = [torch.empty_like(v) for v in rg]
    common = (B, L, L, Di, d, words, ops.norm_code(p), eps, 0.25)
    zg = run(lib.fb_dot_product_given_f32, "fb_dot_product_given_f32", q, k, (B, L, Di, L), (B, L, L), rg,
             common + (_lib.FB_NATIVE, 1, 3))
    zs = run(lib.fb_dot_product_given_f32, "fb_dot_product_given_f32", q, k, (B, L, Di, L), (B, L, L), rs,
             common + (_lib.FB_NATIVE, 1, 0))
    for a, b in zip(rg, (ql, qu, kl, ku)):
        assert torch.equal(a, b)
    for a, b in zip(rs, (ql, qu, kl, ku)):
        assert torch.equal(a, b)
    for a, b in zip(zg, zs):
        assert torch.equal(a, b)
    # with the epilogue's own ranges (last-bit differences in the norms): close
    re_ = [q[4].clone(), q[5].clone(), k[4].clone(), k[5].clone()]
    ze = run(lib.fb_dot_product_given_f32, "fb_dot_product_given_f32", q, k, (B, L, Di, L), (B, L, L), re_,
             common + (_lib.FB_NATIVE, 1, 3))
    for a, b, name in zip(ze, zs, ("lw", "uw", "lb", "ub")):
        helpers.assert_close(a, b, "scores %s with the epilogue's ranges" % name, atol=4e-6)
    # context: x = the scores scaled down, values = k in the projection's layout [B, K, Di, Ly], value ranges given
    x = [v * 0.05 for v in zs]
    vr = [torch.empty(B, L, L, device=DEV), torch.empty(B, L, L, device=DEV), kl.clone(), ku.clone()]
    vs = [torch.empty(B, L, L, device=DEV), torch.empty(B, L, L, device=DEV), torch.empty(B, d, L, device=DEV),
          torch.empty(B, d, L, device=DEV)]
    ccommon = (B, L, d, Di, L, words, ops.norm_code(p), eps, 1.0, H)
    cg = run(lib.fb_context_given_f32, "fb_context_given_f32", x, k, (S, L, Di, D), (S, L, D), vr, ccommon + (2,))
    cs = run(lib.fb_context_given_f32, "fb_context_given_f32", x, k, (S, L, Di, D), (S, L, D), vs, ccommon + (0,))
    for a, b in zip(vr, vs):
        assert torch.equal(a, b)          # both hold the transposed value ranges now
    for a, b in zip(cg, cs):
        assert torch.equal(a, b)


@pytest.mark.parametrize("op_name", ["relu", "tanh"])
@pytest.mark.parametrize("p,words", [(float("inf"), 1), (2.0, 2), (1.0, 1)])
def test_relaxation_slopes_from_given_ranges(op_name, p, words):
    """fb_relax_coef_given_f32 (ranges handed over by the producer) equals fb_relax_coef_f32 (ranges from a
    pass over lw / uw) bit for bit when it is given the ranges of a concretisation pass; and a hidden layer
    produced by fb_matmul_heads_ranges_f32 (heads = 1) yields slopes within the per-operator bar."""
    from faith_b200 import ops, _lib
    op = {"relu": _lib.FB_RELU, "tanh": _lib.FB_TANH}[op_name]
    S, L, D, F, eps = 2, 4, 64, 96, 0.05
    Di = 128 * words
    t = [v.to(DEV) for v in cases.rand_bounds(95, S, L, Di, D, -0.4, 0.6)]
    g0 = torch.Generator().manual_seed(8)
    W = (torch.randn(F, D, generator=g0) / math.sqrt(D)).to(DEV)
    bias = (torch.randn(F, generator=g0) * 0.1).to(DEV)
    y = ops.matmul_heads_ranges(t[0], t[2], t[1], t[3], W, bias, 1, p, eps, words)   # hidden bounds [S, L, Di, F] + ranges
    ref = ops.relax_coef(op, y[0], y[1], y[2], y[3], p, eps, words)
    l, u = ops.concretize(y[0], y[1], y[2], y[3], p, eps, words)
    same = ops.relax_coef_given(op, y[2], y[3], l.contiguous(), u.contiguous())
    for a, b, name in zip(same, ref, ("c_l", "c_u", "lb", "ub")):
        assert torch.equal(a, b), name
    got = ops.relax_coef_given(op, y[2], y[3], y[4], y[5])
    for a, b, name in zip(got, ref, ("c_l", "c_u", "lb", "ub")):
        helpers.assert_close(a, b, "%s %s from the epilogue's ranges" % (op_name, name), atol=2e-6)


@pytest.mark.parametrize("shape", [(4, 32, 128, 32), (2, 3, 64, 8), (1, 5, 40, 20)])
@pytest.mark.parametrize("p,words", [(2.0, 1), (float("inf"), 1), (1.0, 2), (2.0, 2)])
def test_fused_softmax_returns_the_range_of_its_result(shape, p, words):
    """fb_softmax_ranges_f32: the bounds are those of fb_softmax_f32 bit for bit, and the range it
    accumulates while writing equals a concretisation pass over the written bounds."""
    import faith_b200
    from faith_b200 import ops
    B, L, Di, Do = shape
    t = cases.rand_bounds(604, B, L, Di, Do, -0.5, 0.2)
    g = faith_b200.BoundsLite(p, 0.1, *[v.to(DEV) for v in t], perturbed_words=words)
    plain = ops.softmax_fused(g._t4(), p, 0.1, words)
    withr = ops.softmax_fused(g._t4(), p, 0.1, words, ranges=True)
    assert plain is not None and withr is not None and len(withr) == 6
    for a, b in zip(plain, withr[:4]):
        assert torch.equal(a, b)
    l, u = ops.concretize(plain[0], plain[1], plain[2], plain[3], p, 0.1, words)
    helpers.assert_close(withr[4], l, "softmax range l")
    helpers.assert_close(withr[5], u, "softmax range u")


@pytest.mark.parametrize("residual", [False, True])
def test_layer_norm_of_128_features_matches_oracle(residual):
    """Do == 128 takes the single-pass kernel with 128-bit accesses (a row per warp, kept in registers);
    compared with the oracle's layer_norm (after add for the residual form)."""
    from faith_b200 import ops
    B, L, Di, Do = 2, 5, 24, 128
    t = cases.rand_bounds(801, B, L, Di, Do)
    r = cases.rand_bounds(802, B, L, Di, Do)
    g0 = torch.Generator().manual_seed(12)
    gamma = torch.randn(Do, generator=g0)
    beta = 0.1 * torch.randn(Do, generator=g0)
    o = O.OBounds(2.0, 0.1, *t)
    if residual:
        o = o.add(O.OBounds(2.0, 0.1, *r))
    o = o.layer_norm(gamma, beta, "no_var")
    x = tuple(v.to(DEV) for v in (t[0], t[2], t[1], t[3]))      # lw, uw, lb, ub
    res = tuple(v.to(DEV) for v in (r[0], r[2], r[1], r[3])) if residual else None
    got = ops.layernorm_novar(x, gamma.to(DEV), beta.to(DEV), res)
    for a, k in zip(got, ("lw", "uw", "lb", "ub")):
        helpers.assert_close(a, getattr(o, k), "layer norm %s" % k)


@pytest.mark.parametrize("with_slopes", [False, True])
@pytest.mark.parametrize("Do,Dy", [(128, 128), (512, 96)])
def test_dense_with_residual_added_in_the_epilogue(with_slopes, Do, Dy):
    """fb_matmul_residual_f32 equals fb_matmul_f32 (or fb_relax_coef_f32 + fb_matmul_coef_f32) followed by
    fb_add_f32 bit for bit; ten launches give identical results; shapes without 256 bias rows are refused."""
    from faith_b200 import ops, _lib
    S, L, Di, eps, p = 8, 32, 128, 0.05, float("inf")
    t = cases.rand_bounds(901, S, L, Di, Do, -0.4, 0.6)
    r = cases.rand_bounds(902, S, L, Di, Dy)
    g0 = torch.Generator().manual_seed(13)
    W = (torch.randn(Dy, Do, generator=g0) / math.sqrt(Do)).to(DEV)
    bias = (torch.randn(Dy, generator=g0) * 0.1).to(DEV)
    lw, lb, uw, ub = [v.to(DEV) for v in t]
    res = tuple(v.to(DEV) for v in (r[0], r[2], r[1], r[3]))
    if with_slopes:
        c_l, c_u, nlb, nub = ops.relax_coef(_lib.FB_RELU, lw, uw, lb, ub, p, eps, 1)
        y = ops.matmul_coef(lw, uw, nlb, nub, c_l, c_u, W, bias)
        args = (lw, uw, nlb, nub, W, bias, res, c_l, c_u)
    else:
        y = ops.matmul(lw, uw, lb, ub, W, bias)
        args = (lw, uw, lb, ub, W, bias, res)
    ref = ops.add(y, res)
    first = ops.matmul_residual(*args)
    for a, b, name in zip(first, ref, ("lw", "uw", "lb", "ub")):
        assert torch.equal(a, b), name
    for _ in range(9):
        again = ops.matmul_residual(*args)
        for a, b in zip(again, first):
            assert torch.equal(a, b)
    flag = __import__("ctypes").c_int(0)
    _lib.check(_lib.load().fb_tc_error_flag(__import__("ctypes").byref(flag)), "fb_tc_error_flag")
    assert flag.value == 0
    with pytest.raises(_lib.FaithError):   # 64 bias rows: below the tensor-core kernel's minimum
        ops.matmul_residual(lw[:2].contiguous(), uw[:2].contiguous(), lb[:2].contiguous(), ub[:2].contiguous(), W, bias,
                            tuple(v[:2].contiguous() for v in res))


@pytest.mark.parametrize("p,words", [(float("inf"), 1), (2.0, 2)])
def test_projection_of_a_point_bound_takes_the_zero_radius_kernel(p, words):
    """One tensor passed as both lw and uw (every stage before the first relaxation) selects the GEMM
    instantiation that skips the radius half; its results equal those of the general kernel, fed a separate
    copy of the tensor, bit for bit; lower and upper outputs coincide."""
    from faith_b200 import ops
    S, L, H, d = 2, 32, 4, 32
    D, Di, eps = H * d, 128 * words, 0.05
    t = [v.to(DEV) for v in cases.rand_bounds(903, S, L, Di, D)]
    g = torch.Generator().manual_seed(14)
    W = (torch.randn(D, D, generator=g) / math.sqrt(D)).to(DEV)
    bias = (torch.randn(D, generator=g) * 0.1).to(DEV)
    lw, lb = t[0], t[1]
    general = ops.matmul_heads_ranges(lw, lw.clone(), lb, lb.clone(), W, bias, H, p, eps, words)
    point = ops.matmul_heads_ranges(lw, lw, lb, lb, W, bias, H, p, eps, words)
    for a, b, name in zip(point, general, ("lw", "uw", "lb", "ub", "l", "u")):
        assert torch.equal(a, b), name
    assert torch.equal(point[0], point[1])
    for _ in range(5):
        again = ops.matmul_heads_ranges(lw, lw, lb, lb, W, bias, H, p, eps, words)
        for a, b in zip(again, point):
            assert torch.equal(a, b)


def test_tensor_core_give_up_path_reports_a_timeout_and_leaves_the_gpu_usable():
    """A wait that runs out must surface, not vanish: the product is launched with the operand loads of one k-block
    of the first thread block left out and every wait limited to about half a millisecond.  The block has to drain,
    free its tensor memory and return; the call reports FB_ERR_TIMEOUT, bit 2 of the status word is set, the flag is
    clear afterwards, and the next product on the same device is correct."""
    import ctypes
    from faith_b200 import ops, _lib
    lib = _lib.load()
    g = torch.Generator().manual_seed(77)
    rows, Di, Do, Dy = 4, 128, 128, 128
    lw = torch.randn(rows, Di, Do, generator=g).to(DEV)
    uw = (lw.cpu() + torch.rand(rows, Di, Do, generator=g)).to(DEV)
    W = (torch.randn(Dy, Do, generator=g) / 8).to(DEV)
    y = [torch.empty(rows, Di, Dy, device=DEV) for _ in range(2)]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    rc = lib.fb_tc_selftest_timeout(lw.data_ptr(), uw.data_ptr(), W.data_ptr(), y[0].data_ptr(), y[1].data_ptr(),
                                    rows * Di, Dy, Do, 1, 25, status.data_ptr(), st)
    assert rc == 6, lib.fb_status_string(rc)          # FB_ERR_TIMEOUT
    assert int(status.item()) & 4
    assert lib.fb_tc_check() == 0                     # the flag was cleared by the read
    lb = torch.zeros(rows, Do, device=DEV)
    got = ops.matmul(lw, uw, lb, lb, W, None)
    assert lib.fb_tc_check() == 0
    ref_l = lw.double() @ W.double().clamp(min=0).t() + uw.double() @ W.double().clamp(max=0).t()
    assert float((got[0].double() - ref_l).abs().max()) < 1e-4


# ------------------------------------------------------------------------------------------------
# Interval mode against the reference itself, live on the GPU: its interval relu and its interval products move
# constants to the device with .cuda() (Bounds.py:925, :676), so those branches only run where there is a GPU.
@pytest.mark.parametrize("name", sorted(n for n, c in cases.OP_CASES.items() if not c.get("golden", True)))
def test_interval_mode_matches_the_reference_on_the_gpu(name):
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir, "oracle"))
    import reference_loader
    if not reference_loader.reference_available():
        pytest.skip("reference modules not staged")
    mod = reference_loader.load_reference_bounds()
    c = cases.OP_CASES[name]
    args = reference_loader.make_args(p=c["p"], perturbed_words=c["words"], method="ibp")
    x_t, ex = cases.case_inputs(c)

    def mk(t):
        return mod.Bounds(args, c["p"], c["eps"], lw=t[0].to(DEV), lb=t[1].to(DEV), uw=t[2].to(DEV), ub=t[3].to(DEV))

    x = mk(x_t)
    op = c["op"]
    if op == "dot":
        ref = x.dot_product(mk(ex["y"]))
    elif op == "mul_bounds":
        ref = x.multiply(mk(ex["y"]))
    else:
        ref = getattr(x, op)()
    got = run_gpu_op(c)
    for k in ("lw", "uw", "lb", "ub"):
        helpers.assert_close(got[k], getattr(ref, k), "%s/%s vs the reference on the GPU" % (name, k))


@pytest.mark.parametrize("S", [8, 9])
def test_bias_rows_in_the_grid_of_the_weight_rows_bit_for_bit(S, monkeypatch):
    """The bias terms of a bound ride as extra tiles in the tensor-core launch of its weight rows (plain product,
    product with ranges, with slopes, with the residual; zero radius or not).  Every tile is computed as a launch of
    its own computes it: results equal those with FB_TC_SEPARATE_BIAS_ROWS=1 bit for bit, also with a last tile of
    the bias rows that is cut short (S = 9: 288 rows)."""
    from faith_b200 import ops, _lib
    L, Di, D, F, H, eps, p = 32, 128, 128, 256, 4, 0.05, float("inf")
    t = [v.to(DEV) for v in cases.rand_bounds(911, S, L, Di, D, -0.4, 0.6)]
    lw, lb, uw, ub = t
    r = [v.to(DEV) for v in cases.rand_bounds(912, S, L, Di, F)]
    res = (r[0], r[2], r[1], r[3])
    g = torch.Generator().manual_seed(15)
    W = (torch.randn(F, D, generator=g) / math.sqrt(D)).to(DEV)
    Wq = (torch.randn(D, D, generator=g) / math.sqrt(D)).to(DEV)
    bias = (torch.randn(F, generator=g) * 0.1).to(DEV)
    bq = (torch.randn(D, generator=g) * 0.1).to(DEV)
    c_l, c_u, nlb, nub = ops.relax_coef(_lib.FB_RELU, lw, uw, lb, ub, p, eps, 1)

    def run_all():
        out = []
        out += ops.matmul(lw, uw, lb, ub, W, bias)
        out += ops.matmul(lw, uw, lb, ub, W, None)
        out += ops.matmul_heads_ranges(lw, uw, lb, ub, Wq, bq, H, p, eps, 1)
        out += ops.matmul_heads_ranges(lw, lw, lb, lb, Wq, bq, H, 2.0, eps, 1)     # zero radius on both parts
        out += ops.matmul_heads_ranges(lw, lw, lb, ub, Wq, bq, H, p, eps, 1)       # zero radius on one: not merged
        out += ops.matmul_heads_ranges(lw, uw, lb, ub, Wq, bq, 1, p, eps, 1)       # one head: bias rows stored in place
        out += ops.matmul_coef(lw, uw, nlb, nub, c_l, c_u, W, bias)
        out += ops.matmul_residual(lw, uw, lb, ub, W, bias, res)
        out += ops.matmul_residual(lw, uw, nlb, nub, W, bias, res, c_l, c_u)
        torch.cuda.synchronize()
        return out
    monkeypatch.setenv("FB_TC_SEPARATE_BIAS_ROWS", "1")
    separate = run_all()
    monkeypatch.delenv("FB_TC_SEPARATE_BIAS_ROWS")
    merged = run_all()
    assert len(merged) == len(separate)
    for k, (a, b) in enumerate(zip(merged, separate)):
        assert torch.equal(a, b), k
    for _ in range(3):
        for k, (a, b) in enumerate(zip(run_all(), merged)):
            assert torch.equal(a, b), k
    assert _lib.load().fb_tc_check() == 0


def test_bias_rows_in_the_grid_with_a_ragged_last_tile_of_weight_rows(monkeypatch):
    """Weight rows that do not fill their last 128-row tile (288 x 50 rows = 112.5 tiles): the bias rows start at a
    tile of their own behind it; plain product and product with residual, merged and separate launches bit for bit,
    and both against the fp64 statement of the split-sign product."""
    from faith_b200 import ops
    S, L, Di, D, F = 9, 32, 50, 64, 96
    lw, lb, uw, ub = [v.to(DEV) for v in cases.rand_bounds(921, S, L, Di, D, -0.4, 0.6)]
    r = [v.to(DEV) for v in cases.rand_bounds(922, S, L, Di, F)]
    res = (r[0], r[2], r[1], r[3])
    g = torch.Generator().manual_seed(16)
    W = (torch.randn(F, D, generator=g) / math.sqrt(D)).to(DEV)
    bias = (torch.randn(F, generator=g) * 0.1).to(DEV)

    def run_all():
        out = list(ops.matmul(lw, uw, lb, ub, W, bias)) + list(ops.matmul_residual(lw, uw, lb, ub, W, bias, res))
        torch.cuda.synchronize()
        return out
    monkeypatch.setenv("FB_TC_SEPARATE_BIAS_ROWS", "1")
    separate = run_all()
    monkeypatch.delenv("FB_TC_SEPARATE_BIAS_ROWS")
    merged = run_all()
    for k, (a, b) in enumerate(zip(merged, separate)):
        assert torch.equal(a, b), k
    Wp, Wn = W.double().clamp(min=0).t(), W.double().clamp(max=0).t()
    ref = [lw.double() @ Wp + uw.double() @ Wn, uw.double() @ Wp + lw.double() @ Wn,
           lb.double() @ Wp + ub.double() @ Wn + bias.double(), ub.double() @ Wp + lb.double() @ Wn + bias.double()]
    for k in range(4):
        assert float((merged[k].double() - ref[k]).abs().max()) < 2e-5, k
        assert float((merged[4 + k].double() - ref[k] - res[k].double()).abs().max()) < 2e-5, k


@pytest.mark.parametrize("with_slopes,Do", [(False, 128), (True, 512), (False, 64)])
def test_layer_norm_applied_by_the_epilogue_of_the_product(with_slopes, Do):
    """fb_matmul_residual_ln_f32 against fb_matmul_residual_f32 followed by fb_layernorm_novar_f32: same bounds to
    rounding (the row means are rounded in another order, so the bar is the fp64 arbiter's, not bit identity), the
    row sums it leaves behind are those of its result, a second product chained on them works, and ten launches
    give identical bits."""
    from faith_b200 import ops, _lib
    S, L, Di, Dy, eps, p = 9, 32, 128, 128, 0.05, float("inf")
    t = cases.rand_bounds(931, S, L, Di, Do, -0.4, 0.6)
    r = cases.rand_bounds(932, S, L, Di, Dy)
    g0 = torch.Generator().manual_seed(17)
    W = (torch.randn(Dy, Do, generator=g0) / math.sqrt(Do)).to(DEV)
    bias = (torch.randn(Dy, generator=g0) * 0.1).to(DEV)
    gamma = (torch.randn(Dy, generator=g0)).to(DEV)       # both signs
    beta = (torch.randn(Dy, generator=g0) * 0.1).to(DEV)
    lw, lb, uw, ub = [v.to(DEV) for v in t]
    res = tuple(v.to(DEV) for v in (r[0], r[2], r[1], r[3]))
    rs = ops.row_sums(*res)
    if with_slopes:
        c_l, c_u, nlb, nub = ops.relax_coef(_lib.FB_RELU, lw, uw, lb, ub, p, eps, 1)
        x = (lw, uw, nlb, nub)
        extra = (c_l, c_u)
    else:
        x = (lw, uw, lb, ub)
        extra = ()
    y = ops.matmul_residual(*x, W, bias, res, *extra)
    want = ops.layernorm_novar(y, gamma, beta)
    got = ops.matmul_residual_ln(*x, W, bias, res, rs, gamma, beta, *extra)
    # fp64 statement of the whole chain from the inputs: split-sign product, bias, residual, norm
    xl, xu = (x[0] * extra[0].unsqueeze(-2), x[1] * extra[1].unsqueeze(-2)) if with_slopes else (x[0], x[1])
    Wp, Wn = W.double().clamp(min=0).t(), W.double().clamp(max=0).t()
    y64 = [xl.double() @ Wp + xu.double() @ Wn + res[0].double(), xu.double() @ Wp + xl.double() @ Wn + res[1].double(),
           x[2].double() @ Wp + x[3].double() @ Wn + bias.double() + res[2].double(),
           x[3].double() @ Wp + x[2].double() @ Wn + bias.double() + res[3].double()]
    g64, b64 = gamma.double(), beta.double()
    gp, gn = g64.clamp(min=0), g64.clamp(max=0)
    cl = [y64[0] - y64[1].mean(-1, keepdim=True), y64[2] - y64[3].mean(-1, keepdim=True)]
    cu = [y64[1] - y64[0].mean(-1, keepdim=True), y64[3] - y64[2].mean(-1, keepdim=True)]
    ref64 = [cl[0] * gp + cu[0] * gn, cu[0] * gp + cl[0] * gn, cl[1] * gp + cu[1] * gn + b64, cu[1] * gp + cl[1] * gn + b64]
    for k, name in enumerate(("lw", "uw", "lb", "ub")):
        helpers.assert_arbitrated(got[k], want[k], ref64[k], "layer norm in the epilogue, " + name)
    sums = ops.row_sums(*got[:4])
    assert torch.allclose(got[4].sum(1), sums.sum(1), rtol=1e-5, atol=2e-4)
    # chained: the result as the residual of the next product, with the row sums this launch left behind
    nxt_want = ops.layernorm_novar(ops.matmul_residual(lw[..., :128].contiguous(), uw[..., :128].contiguous(),
                                                       lb[..., :128].contiguous(), ub[..., :128].contiguous(),
                                                       W[:, :128].contiguous(), bias, want), gamma, beta) if Do >= 128 else None
    if nxt_want is not None:
        nxt = ops.matmul_residual_ln(lw[..., :128].contiguous(), uw[..., :128].contiguous(), lb[..., :128].contiguous(),
                                     ub[..., :128].contiguous(), W[:, :128].contiguous(), bias, got[:4], got[4], gamma, beta)
        for k in range(4):
            helpers.assert_close(nxt[k], nxt_want[k], "chained %d" % k, atol=2e-4, rtol=1e-4)
    for _ in range(9):
        again = ops.matmul_residual_ln(*x, W, bias, res, rs, gamma, beta, *extra)
        for a, b in zip(again, got):
            assert torch.equal(a, b)
    assert _lib.load().fb_tc_check() == 0
    with pytest.raises(_lib.FaithError):   # 64 output features: not a shape of the fused kernel
        ops.matmul_residual_ln(*x, W[:64].contiguous(), bias[:64].contiguous(), tuple(v[..., :64].contiguous() for v in res),
                               rs, gamma[:64].contiguous(), beta[:64].contiguous(), *extra)
