"""Seeded input generators shared by the golden-vector generator and the tests.

Inputs are always produced by `torch.Generator().manual_seed(seed)` on the CPU, so every
machine regenerates identical bits; only the *outputs* of the reference are stored in the
golden files.  Distributions follow the reference's own kernel test
(HandTunedKernels/kernel_test/transformer_forward_test_bound.py:746-754,778): lb ~ U[0,1),
ub = lb + U[0,1), lw, uw ~ U[-0.5,0.5), W ~ U[-0.5,0.5).
"""
import torch

INF = float("inf")


def rand_bounds(seed, B, L, Di, Do, shift=0.0, wscale=1.0, gap=1.0):
    """Returns lw, lb, uw, ub.  `shift` moves lb/ub (to create negative and crossing columns),
    `wscale` scales lw/uw, `gap` scales the distance between lb and ub."""
    g = torch.Generator().manual_seed(seed)
    lb = torch.rand(B, L, Do, generator=g) + shift
    ub = lb + torch.rand(B, L, Do, generator=g) * gap
    lw = (torch.rand(B, L, Di, Do, generator=g) - 0.5) * wscale
    uw = (torch.rand(B, L, Di, Do, generator=g) - 0.5) * wscale
    return lw, lb, uw, ub


def rand_weight(seed, Dy, Do):
    g = torch.Generator().manual_seed(seed)
    return torch.rand(Dy, Do, generator=g) - 0.5, torch.rand(Dy, generator=g) - 0.5


# name -> (op, kwargs).  Every case is small enough for the CPU suite to run in seconds.
OP_CASES = {}
for _p, _pn in ((1.0, "p1"), (2.0, "p2"), (INF, "pinf")):
    for _w in (1, 2):
        tag = "%s_w%d" % (_pn, _w)
        OP_CASES["concretize_" + tag] = dict(op="concretize", p=_p, words=_w, eps=0.5, seed=11, B=2, L=3, Di=16, Do=24)
        # shift -0.7 / wscale 0.2 gives a mix of positive, negative and crossing columns
        OP_CASES["relu_" + tag] = dict(op="relu", p=_p, words=_w, eps=0.5, seed=12, B=2, L=3, Di=16, Do=24, shift=-0.7, wscale=0.2)
        OP_CASES["tanh_" + tag] = dict(op="tanh", p=_p, words=_w, eps=0.5, seed=13, B=2, L=3, Di=16, Do=24, shift=-0.7, wscale=0.2)
        OP_CASES["exp_" + tag] = dict(op="exp", p=_p, words=_w, eps=0.5, seed=14, B=2, L=3, Di=16, Do=24, shift=-0.7, wscale=0.2)
        OP_CASES["reciprocal_" + tag] = dict(op="reciprocal", p=_p, words=_w, eps=0.05, seed=15, B=2, L=3, Di=16, Do=24, shift=1.0, wscale=0.2)
        OP_CASES["sqr_" + tag] = dict(op="sqr", p=_p, words=_w, eps=0.5, seed=17, B=2, L=3, Di=16, Do=24, shift=-0.7, wscale=0.2)
        OP_CASES["sqrt_" + tag] = dict(op="sqrt", p=_p, words=_w, eps=0.05, seed=18, B=2, L=3, Di=16, Do=24, shift=1.0, wscale=0.2)
# interval mode (--method ibp): the weight tensors are cut to `words` rows and every operator takes its interval branch
for _op, _sh, _eps in (("relu", -0.7, 0.5), ("tanh", -0.7, 0.5), ("exp", -0.7, 0.5), ("reciprocal", 1.0, 0.05),
                       ("sqr", -0.7, 0.5), ("sqrt", 1.0, 0.05)):
    for _w in (1, 2):
        # (the reference's interval relu and its interval products move constants to the GPU with .cuda(), Bounds.py:925,
        # :676: those branches cannot run where the golden files are made; they are pinned live on the GPU instead)
        OP_CASES["ibp_%s_w%d" % (_op, _w)] = dict(op=_op, ibp=True, p=INF, words=_w, eps=_eps, seed=19, B=2, L=3, Di=16,
                                                  Do=24, shift=_sh, wscale=0.2, golden=_op != "relu")
OP_CASES["ibp_mul_bounds"] = dict(op="mul_bounds", ibp=True, p=INF, words=1, eps=0.5, seed=43, B=2, L=3, Di=16, Do=24,
                                  shift=-0.5, wscale=0.0, golden=False)
OP_CASES["ibp_dot_w1"] = dict(op="dot", ibp=True, p=INF, words=1, eps=0.1, seed=34, B=2, L=5, Di=16, Do=8, Ly=6,
                              shift=-0.5, wscale=0.0)
OP_CASES["ibp_dot_w2"] = dict(op="dot", ibp=True, p=INF, words=2, eps=0.1, seed=35, B=2, L=5, Di=16, Do=8, Ly=6,
                              shift=-0.5, wscale=0.0, golden=False)
OP_CASES["ibp_softmax"] = dict(op="softmax", ibp=True, p=INF, words=1, eps=0.1, seed=52, B=2, L=3, Di=16, Do=6, shift=-0.5,
                               wscale=0.0, golden=False)
OP_CASES["dot_dim_in_1"] = dict(op="dot", p=2.0, words=1, eps=0.5, seed=36, B=2, L=5, Di=1, Do=8, Ly=6, shift=-0.5)
# (tight input bounds: the variance of the centred features must stay provably positive, Bounds.py:894)
OP_CASES["layer_norm_standard"] = dict(op="layer_norm_std", p=2.0, words=1, eps=0.05, seed=64, B=2, L=3, Di=16, Do=24,
                                       shift=-0.5, wscale=0.02, gap=0.02)
OP_CASES["mul_tensor"] = dict(op="mul_tensor", p=2.0, words=1, eps=0.5, seed=65, B=2, L=3, Di=16, Do=24, shift=-0.5)
OP_CASES["exp_large"] = dict(op="exp", p=2.0, words=1, eps=0.5, seed=16, B=1, L=2, Di=8, Do=32, shift=11.0, wscale=1.0)
OP_CASES["matmul"] = dict(op="matmul", p=2.0, words=1, eps=0.5, seed=21, B=2, L=3, Di=16, Do=24, Dy=40)
OP_CASES["dense"] = dict(op="dense", p=2.0, words=1, eps=0.5, seed=22, B=1, L=5, Di=8, Do=33, Dy=7)
OP_CASES["dot_qk_p2"] = dict(op="dot", p=2.0, words=1, eps=0.5, seed=31, B=2, L=5, Di=16, Do=8, Ly=5, shift=-0.5)
OP_CASES["dot_qk_pinf_w2"] = dict(op="dot", p=INF, words=2, eps=0.1, seed=32, B=3, L=4, Di=16, Do=8, Ly=6, shift=-0.5)
OP_CASES["context_p2"] = dict(op="context", p=2.0, words=1, eps=0.5, seed=33, B=2, L=5, Di=16, Do=8, shift=-0.5)
OP_CASES["mul_bounds_p2"] = dict(op="mul_bounds", p=2.0, words=1, eps=0.5, seed=41, B=2, L=3, Di=16, Do=24, shift=-0.5)
OP_CASES["mul_bounds_p1_w2"] = dict(op="mul_bounds", p=1.0, words=2, eps=0.5, seed=42, B=2, L=3, Di=16, Do=24, shift=-0.5)
OP_CASES["softmax_p2"] = dict(op="softmax", p=2.0, words=1, eps=0.1, seed=51, B=2, L=3, Di=16, Do=6, shift=-0.5, wscale=0.2)
OP_CASES["layer_norm"] = dict(op="layer_norm", p=2.0, words=1, eps=0.5, seed=61, B=2, L=3, Di=16, Do=24)
OP_CASES["scale_neg"] = dict(op="scale", p=2.0, words=1, eps=0.5, seed=62, B=1, L=3, Di=8, Do=12, c=-0.25)
OP_CASES["add_bounds"] = dict(op="add", p=2.0, words=1, eps=0.5, seed=63, B=1, L=3, Di=8, Do=12)

# small encoder for the end-to-end golden (eps small enough that bounds stay tight)
ENCODER_CASE = dict(seed=71, layers=2, d_model=32, heads=2, ffn=64, L=8, B=2, eps=1e-3, p=INF, index=1, std=0.1)

# search for the largest certified radius (Verifier.py:106-147): per word a probe at max_eps and `iters` bisection
# steps.  A small encoder with BERT-like initialisation (std 0.02): its fp32 rounding noise (1e-7 on the logit bounds) is
# four orders of magnitude below what one bisection step changes, so every implementation must take the same
# decisions; max_eps sits above the radius where certification stops and below the one where a softmax denominator
# is no longer provably positive.
SEARCH_CASE = dict(seed=72, layers=2, d_model=32, heads=2, ffn=64, L=8, B=2, std=0.02, p=INF, max_eps=1.0, iters=8,
                   iters2=5)   # iters2: bisection steps of the two-word search


def case_inputs(c):
    """Materialises the input tensors of an operator case: (x_bounds_tuple, extras)."""
    sh = c.get("shift", 0.0)
    ws = c.get("wscale", 1.0)
    x = rand_bounds(c["seed"], c["B"], c["L"], c["Di"], c["Do"], sh, ws, c.get("gap", 1.0))
    extra = {}
    op = c["op"]
    if op in ("matmul", "dense"):
        extra["W"], extra["bias"] = rand_weight(c["seed"] + 1000, c["Dy"], c["Do"])
    elif op in ("layer_norm_std", "mul_tensor"):
        extra["W"], extra["bias"] = rand_weight(c["seed"] + 1000, 1, c["Do"])
        extra["W"] = extra["W"][0] * 2 + 0.3   # gains of both signs
        extra["bias"] = torch.rand(c["Do"], generator=torch.Generator().manual_seed(c["seed"] + 2000)) - 0.5
    elif op == "dot":
        extra["y"] = rand_bounds(c["seed"] + 1000, c["B"], c["Ly"], c["Di"], c["Do"], sh, ws)
    elif op == "context":
        # self plays the probabilities [B, L, Di, L]; the value operand is [B, L, Di, Do]
        x = rand_bounds(c["seed"], c["B"], c["L"], c["Di"], c["L"], 0.0, 0.2)
        extra["y"] = rand_bounds(c["seed"] + 1000, c["B"], c["L"], c["Di"], c["Do"], sh, ws)
    elif op in ("mul_bounds", "add"):
        extra["y"] = rand_bounds(c["seed"] + 1000, c["B"], c["L"], c["Di"], c["Do"], sh, ws)
    elif op == "layer_norm":
        extra["W"], extra["bias"] = rand_weight(c["seed"] + 1000, 1, c["Do"])
        extra["W"] = extra["W"][0]
        extra["bias"] = torch.rand(c["Do"], generator=torch.Generator().manual_seed(c["seed"] + 2000)) - 0.5
    return x, extra


def encoder_inputs(c=ENCODER_CASE):
    g = torch.Generator().manual_seed(c["seed"])
    return torch.randn(c["B"], c["L"], c["d_model"], generator=g)
