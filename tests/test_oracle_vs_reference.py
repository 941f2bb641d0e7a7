"""The CPU oracle against the reference module itself, imported unchanged.  Skipped where
the reference checkout is absent (the golden-vector test covers those machines)."""
import pytest
import torch

import cases
import helpers
import ref_loader
from oracle import bounds_oracle as O

pytestmark = pytest.mark.skipif(not ref_loader.reference_available(), reason="reference checkout not present")


@pytest.mark.parametrize("name", sorted(n for n, c in cases.OP_CASES.items() if c.get("golden", True)))
def test_op_matches_reference(name):
    import make_golden
    torch.set_num_threads(1)
    c = cases.OP_CASES[name]
    ref = make_golden.run_reference_op(c)
    out = helpers.run_oracle_op(c)
    for k in ref:
        helpers.assert_close(out[k], ref[k], "%s/%s" % (name, k))


@pytest.mark.parametrize("op,shape", [("relu", (1, 4, 64, 64)), ("tanh", (1, 2, 64, 128)),
                                      ("dot_qk", (2, 8, 64, 16)), ("dot_v", (2, 8, 64, 10)), ("matmul", (1, 4, 64, 64))])
def test_reference_kernel_test_class(op, shape):
    """The second, test-local `Bounds(p, eps, lw, lb, uw, ub)` class of the reference's kernel
    test (transformer_forward_test_bound.py:33-347) on its own input distribution, p=2, eps=0.5
    (:746-754,774).  Its tanh omits the crossing-case lower line (:416-431), so only the upper
    line is compared for tanh."""
    from oracle import bounds_oracle as O
    kt = ref_loader.load_reference_kernel_test()
    torch.manual_seed(0)
    B, L, Di, Do = shape
    if op == "dot_v":
        lw, lb, uw, ub = cases.rand_bounds(1, B, L, Di, L)
        y = cases.rand_bounds(2, B, Do, Di, L)
    else:
        lw, lb, uw, ub = cases.rand_bounds(1, B, L, Di, Do)
        y = cases.rand_bounds(2, B, L, Di, Do)
    rb = kt.Bounds(p=2, eps=0.5, lw=lw, lb=lb, uw=uw, ub=ub)
    ob = O.OBounds(2, 0.5, lw, lb, uw, ub)
    if op == "relu":
        r, o = rb.relu(), ob.relu()
    elif op == "tanh":
        r, o = rb.tanh(), ob.tanh()
        helpers.assert_close(o.uw, r.uw, "tanh uw")
        helpers.assert_close(o.ub, r.ub, "tanh ub")
        return
    elif op == "matmul":
        W, _ = cases.rand_weight(3, Di, Do)
        r, o = rb.matmul(W), ob.matmul(W)
    else:
        ry = kt.Bounds(p=2, eps=0.5, lw=y[0], lb=y[1], uw=y[2], ub=y[3])
        oy = O.OBounds(2, 0.5, *y)
        r, o = rb.dot_product(ry), ob.dot_product(oy)
    for k in ("lw", "lb", "uw", "ub"):
        helpers.assert_close(getattr(o, k), getattr(r, k), "%s %s" % (op, k), rtol=1e-5, atol=2e-6)


def test_encoder_pass_matches_reference():
    from oracle import bounds_oracle as O
    torch.set_num_threads(1)
    c = cases.ENCODER_CASE
    model = O.make_encoder(c["seed"], c["layers"], c["d_model"], c["heads"], c["ffn"], c["std"])
    emb = cases.encoder_inputs(c)
    ver = ref_loader.build_reference_verifier(model, c["p"])
    l, u = O.encoder_forward(model, emb, [c["index"]], c["p"], c["eps"])
    l64, u64 = O.encoder_forward(O.model_to(model, torch.float64), emb.double(), [c["index"]], c["p"], c["eps"])
    for s in range(c["B"]):
        rl, ru, _ = ref_loader.reference_encoder_pass(ver, emb[s:s + 1], c["index"], c["eps"])
        helpers.assert_within_noise(l[s], rl, l64[s], "l")
        helpers.assert_within_noise(u[s], ru, u64[s], "u")


def test_encoder_pass_with_standard_layer_norm_matches_reference():
    """layer_norm="standard" (Bounds.py:1122-1124: variance through sqr, division through sqrt and reciprocal) over a
    whole pass of the reference's VerifierForward, against the oracle."""
    c = dict(cases.ENCODER_CASE, std=0.02, eps=1e-3)
    model = O.make_encoder(c["seed"], c["layers"], c["d_model"], c["heads"], c["ffn"], c["std"], layer_norm="standard")
    emb = cases.encoder_inputs(c)
    ver = ref_loader.build_reference_verifier(model, c["p"])
    l, u = O.encoder_forward(model, emb, [c["index"]], c["p"], c["eps"])
    l64, u64 = O.encoder_forward(O.model_to(model, torch.float64), emb.double(), [c["index"]], c["p"], c["eps"])
    y = O.concrete_forward(model, emb)
    for s in range(c["B"]):
        rl, ru, _ = ref_loader.reference_encoder_pass(ver, emb[s:s + 1], c["index"], c["eps"])
        helpers.assert_within_noise(l[s:s + 1], rl.reshape(1), l64[s:s + 1], "logit lower")
        helpers.assert_within_noise(u[s:s + 1], ru.reshape(1), u64[s:s + 1], "logit upper")
        assert float(rl) <= float(y[s]) <= float(ru)
