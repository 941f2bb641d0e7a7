"""The CPU oracle against the committed golden vectors (outputs of the reference's own
Python `Bounds`, see tests/golden/make_golden.py)."""
import pytest
import numpy as np
import torch

import cases
import helpers
from oracle import bounds_oracle as O


@pytest.fixture(scope="module")
def golden_ops():
    return helpers.load_golden("ops.npz")


@pytest.mark.parametrize("name", sorted(n for n, c in cases.OP_CASES.items() if c.get("golden", True)))
def test_op_matches_golden(name, golden_ops):
    torch.set_num_threads(1)
    out = helpers.run_oracle_op(cases.OP_CASES[name])
    for k, v in out.items():
        helpers.assert_close(v, golden_ops["%s/%s" % (name, k)], "%s/%s" % (name, k))


def test_encoder_matches_golden():
    torch.set_num_threads(1)
    g = helpers.load_golden("encoder.npz")
    c = cases.ENCODER_CASE
    model = O.make_encoder(c["seed"], c["layers"], c["d_model"], c["heads"], c["ffn"], c["std"])
    emb = cases.encoder_inputs(c)
    trace, trace64 = [], []
    l, u = O.encoder_forward(model, emb, [c["index"]], c["p"], c["eps"], trace=trace)
    l64, u64 = O.encoder_forward(O.model_to(model, torch.float64), emb.double(), [c["index"]], c["p"], c["eps"],
                                 trace=trace64)
    # Single operators meet the per-op bar (test above); over a whole pass the fp32 noise of the
    # reference itself is amplified, so the pass is judged against the fp64 run (see helpers).
    helpers.assert_within_noise(l, g["l"], l64, "logit lower")
    helpers.assert_within_noise(u, g["u"], u64, "logit upper")
    stages, stages64 = dict(trace), dict(trace64)
    for s in range(c["B"]):
        for nm in ("embedding", "layer0.scores", "layer0.probs", "layer0.output", "pooled"):
            bl, bu = stages[nm].concretize()
            bl64, bu64 = stages64[nm].concretize()
            heads = c["heads"] if nm in ("layer0.scores", "layer0.probs") else 1
            sl = slice(s * heads, (s + 1) * heads)
            helpers.assert_within_noise(bl[sl], g["s%d/%s/l" % (s, nm)], bl64[sl], "s%d %s l" % (s, nm))
            helpers.assert_within_noise(bu[sl], g["s%d/%s/u" % (s, nm)], bu64[sl], "s%d %s u" % (s, nm))


def test_bounds_contain_concrete_forward():
    """Soundness of the oracle pass: sampled points of the eps-ball map inside [l, u]."""
    c = cases.ENCODER_CASE
    model = O.make_encoder(c["seed"], c["layers"], c["d_model"], c["heads"], c["ffn"], c["std"])
    emb = cases.encoder_inputs(c)[:1]
    l, u = O.encoder_forward(model, emb, [c["index"]], c["p"], c["eps"])
    g = torch.Generator().manual_seed(5)
    n = 512
    delta = (torch.randint(0, 2, (n, c["d_model"]), generator=g).float() * 2 - 1) * c["eps"]  # vertices
    delta[: n // 2] *= torch.rand(n // 2, 1, generator=g)
    x = emb.repeat(n, 1, 1)
    x[:, c["index"], :] += delta
    y = O.concrete_forward(model, x)
    assert float(y.min()) >= float(l[0]) - 1e-5 and float(y.max()) <= float(u[0]) + 1e-5
    assert float(u[0] - l[0]) < 2.0  # and the bound is finite and of sane width at this eps


@pytest.mark.parametrize("stride,pad,k", [(1, 1, 3), (2, 1, 3), (2, 0, 3), (1, 2, 5)])
def test_conv_oracle_agrees_with_im2col_matmul(stride, pad, k):
    """Ties the (otherwise unpinned) conv restatement to the pinned matmul: unfold + matmul, for the strides and
    paddings of the benchmark CNN (3x3: stride 1 pad 1, stride 2 pad 1) and two more."""
    import torch.nn.functional as F
    g = torch.Generator().manual_seed(502)
    B, Di, C, H, W, Co = 1, 6, 3, 8, 8, 5
    lw = torch.rand(B, Di, C, H, W, generator=g) - 0.5
    uw = torch.rand(B, Di, C, H, W, generator=g) - 0.5
    lb = torch.rand(B, C, H, W, generator=g)
    ub = lb + torch.rand(B, C, H, W, generator=g)
    wt = torch.randn(Co, C, k, k, generator=g) * 0.3
    o = O.conv_bounds(O.OBounds(2.0, 0.1, lw, lb, uw, ub), wt, None, stride, pad)
    Ho, Wo = o.lw.shape[-2:]

    def cols(t):  # [N, C, H, W] -> [N, Ho*Wo, C*k*k]
        return F.unfold(t, k, padding=pad, stride=stride).transpose(1, 2)

    xw = O.OBounds(2.0, 0.1, cols(lw[0]).transpose(0, 1).unsqueeze(0), cols(lb), cols(uw[0]).transpose(0, 1).unsqueeze(0),
                   cols(ub))
    m = xw.matmul(wt.reshape(Co, -1))  # lw [1, Ho*Wo, Di, Co]
    # two fp32 summation orders of K = C*k*k terms of magnitude ~0.1: absolute part scaled to the summed magnitude
    helpers.assert_close(m.lw[0].permute(1, 2, 0).reshape(Di, Co, Ho, Wo), o.lw[0], "lw", atol=2e-6)
    helpers.assert_close(m.uw[0].permute(1, 2, 0).reshape(Di, Co, Ho, Wo), o.uw[0], "uw", atol=2e-6)
    helpers.assert_close(m.lb[0].transpose(0, 1).reshape(Co, Ho, Wo), o.lb[0], "lb", atol=2e-6)
    helpers.assert_close(m.ub[0].transpose(0, 1).reshape(Co, Ho, Wo), o.ub[0], "ub", atol=2e-6)


def test_oracle_search_loop_matches_the_reference_verifier():
    """The restated search loop against the radii the reference's own Verifier.verify found (tests/golden/search.npz).
    A bisection probe whose bound lands within fp32 rounding noise of zero could be answered the other way by another
    summation order, which would move the answer by at most the width of the last steps; with this model's noise that
    is rare, so at most one position may differ."""
    c = sc = cases.SEARCH_CASE
    model = O.make_encoder(c["seed"], c["layers"], c["d_model"], c["heads"], c["ffn"], c["std"])
    emb = cases.encoder_inputs(c)
    g = helpers.load_golden("search.npz")
    n, same = 0, 0
    for s in range(c["B"]):
        got = O.epsilon_search(model, emb[s:s + 1], int(g["labels"][s]), c["p"], sc["max_eps"], sc["iters"])
        assert sorted(got) == [int(i) for i in g["s%d/positions" % s]]
        for i, e in zip(g["s%d/positions" % s], g["s%d/eps" % s]):
            # the reference keeps its answer in a float32 tensor (Verifier.py:92, :137)
            n += 1
            same += np.float32(got[int(i)]) == np.float32(e)
            assert abs(got[int(i)] - float(e)) <= 2.001 * sc["max_eps"] / 2 ** sc["iters"], (s, int(i), got[int(i)], float(e))
    assert same >= n - 1, "%d of %d radii differ from the reference" % (n - same, n)


def test_oracle_two_word_search_matches_the_reference_verifier():
    """Two perturbed words (Verifier.py:149-201): the warmed-up max_eps and the radius per pair of positions of the
    first sentence, against what the reference's own loop found."""
    c = cases.SEARCH_CASE
    model = O.make_encoder(c["seed"], c["layers"], c["d_model"], c["heads"], c["ffn"], c["std"])
    emb = cases.encoder_inputs(c)
    g = helpers.load_golden("search.npz")
    got, warmed = O.epsilon_search_pairs(model, emb[:1], int(g["labels"][0]), c["p"], c["max_eps"], c["iters2"])
    assert warmed == float(g["s0/warmed_max_eps"])
    pairs = [tuple(int(v) for v in q) for q in g["s0/pairs"]]
    assert sorted(got) == pairs
    diff = [q for q, e in zip(pairs, g["s0/pair_eps"]) if np.float32(got[q]) != np.float32(e)]
    assert len(diff) <= 1, diff


def test_layer_norm_after_a_product_from_the_weight_column_means():
    """The identity behind the layer norm applied in a GEMM epilogue (fb_matmul_residual_ln_f32), in double precision on
    the oracle: for y = matmul(x, W) + bias + r the feature mean of a row of y_lw is x's centre row times the column
    means of W minus x's radius row times the column means of |W|, plus the mean of the bias (bias rows), plus the row
    sum of r over the number of features; with those means, (y_lw - mean(y_uw)) gamma+ + (y_uw - mean(y_lw)) gamma-
    (+ beta on the bias rows) is Bounds.layer_norm in mode no_var (Bounds.py:1111-1131)."""
    g = torch.Generator().manual_seed(41)
    B, L, Di, K, N = 2, 3, 5, 12, 8
    dt = torch.float64
    lw = torch.randn(B, L, Di, K, generator=g, dtype=dt)
    uw = lw + torch.rand(B, L, Di, K, generator=g, dtype=dt) * torch.randn(B, L, Di, K, generator=g, dtype=dt).sign()
    lb = torch.randn(B, L, K, generator=g, dtype=dt)
    ub = lb + torch.rand(B, L, K, generator=g, dtype=dt)
    x = O.OBounds(2.0, 0.01, lw, lb, uw, ub)
    r = O.OBounds(2.0, 0.01, torch.randn(B, L, Di, N, generator=g, dtype=dt), torch.randn(B, L, N, generator=g, dtype=dt),
                 torch.randn(B, L, Di, N, generator=g, dtype=dt), torch.randn(B, L, N, generator=g, dtype=dt))
    W = torch.randn(N, K, generator=g, dtype=dt)
    bias, gamma, beta = (torch.randn(N, generator=g, dtype=dt) for _ in range(3))
    y = x.matmul(W).add(bias).add(r)
    want = y.layer_norm(gamma, beta, "no_var")

    wbar, abar = W.mean(0), W.abs().mean(0)
    gp, gn = gamma.clamp(min=0), gamma.clamp(max=0)

    def fused(lo, up, r_lo, r_up, y_lo, y_up, with_bias):
        c, rad = (lo + up) / 2, (up - lo) / 2
        extra = bias.mean() if with_bias else 0.0
        mean_lo = c @ wbar - rad @ abar + r_lo.sum(-1) / N + extra
        mean_up = c @ wbar + rad @ abar + r_up.sum(-1) / N + extra
        dl, du = y_lo - mean_up.unsqueeze(-1), y_up - mean_lo.unsqueeze(-1)
        shift = beta if with_bias else 0.0
        return dl * gp + du * gn + shift, du * gp + dl * gn + shift

    z_lw, z_uw = fused(x.lw, x.uw, r.lw, r.uw, y.lw, y.uw, False)
    z_lb, z_ub = fused(x.lb, x.ub, r.lb, r.ub, y.lb, y.ub, True)
    for got, ref in ((z_lw, want.lw), (z_uw, want.uw), (z_lb, want.lb), (z_ub, want.ub)):
        assert float((got - ref).abs().max()) < 1e-12
