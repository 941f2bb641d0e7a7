"""The reference's own kernel parity test, run unchanged against this library.

HandTunedKernels/kernel_test/transformer_forward_test_bound.py builds the reference's extension at import
(:24-31) and compares, operator by operator, its test-local PyTorch `Bounds` with the extension's kernels
(`relu_test`, `tanh_test`, `dot_product_QK_test`, `dot_product_V_test`, :590-676).  Here the module is imported
as it is, with the one `load(...)` call answered by `faith_b200.c_bound`, and its own test functions are run on
CUDA over the corner and centre points of its sweep (:725-737, :796-799), with its input distributions
(:746-754, :810-818), p = 2, eps = 0.5 (:774).  On top of the module's one-sided comparator the same results
are compared two-sided against an fp64 evaluation (the CPU oracle's restatement, which is pinned to the
reference, run in double precision: the module's own class casts to fp32 inside its dot product).
"""
import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, os.pardir, "oracle"))
sys.path.insert(0, os.path.join(HERE, os.pardir))
import reference_loader  # noqa: E402
from oracle import bounds_oracle as O  # noqa: E402

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not reference_loader.reference_available(), reason="reference modules not staged")]

DEV = "cuda:0"


def _module():
    import faith_b200.c_bound as cb
    return reference_loader.load_reference_kernel_test(c_bound=cb)


def _rand_bound(kt, g, batch, length, dim_in, dim_out):
    lb = torch.rand(batch, length, dim_out, generator=g).to(DEV)
    ub = lb + torch.rand(batch, length, dim_out, generator=g).to(DEV)
    lw = (torch.rand(batch, length, dim_in, dim_out, generator=g) - 0.5).to(DEV)
    uw = (torch.rand(batch, length, dim_in, dim_out, generator=g) - 0.5).to(DEV)
    return kt.Bounds(p=2, eps=0.5, lw=lw, lb=lb, uw=uw, ub=ub)


def _two_sided(kt, got, ref, arbiter, what, c=4.0):
    """|got - ref64| <= c * |ref32 - ref64|_max + 1e-6 + 1e-5 |ref64| elementwise: the kernel may be as far
    from an fp64 evaluation as the reference's own fp32 evaluation is (times c), no further."""
    for k in ("lb", "ub", "lw", "uw"):
        a, r, x = getattr(got, k).double(), getattr(ref, k).double(), getattr(arbiter, k)
        noise = float((r - x).abs().max())
        bad = (a - x).abs() > c * noise + 1e-6 + 1e-5 * x.abs()
        assert not bool(bad.any()), "%s %s: %d elements off, worst %.3e (reference fp32 noise %.3e)" % (
            what, k, int(bad.sum()), float((a - x).abs().max()), noise)


def _as64(kt, b):
    return O.OBounds(2.0, 0.5, b.lw.double(), b.lb.double(), b.uw.double(), b.ub.double())


SWEEP = [(2, 64, 64), (2, 512, 512), (16, 256, 128), (128, 64, 512), (128, 512, 64), (32, 128, 128)]


@pytest.mark.parametrize("length,dim_in,dim_out", SWEEP)
def test_reference_relu_test(length, dim_in, dim_out):
    kt = _module()
    b = _rand_bound(kt, torch.Generator().manual_seed(0), 1, length, dim_in, dim_out)
    kt.relu_test(b)
    _two_sided(kt, b.cuda_relu(), b.relu(), _as64(kt, b).relu(), "relu")


@pytest.mark.parametrize("length,dim_in,dim_out", SWEEP)
def test_reference_tanh_test(length, dim_in, dim_out):
    """The module's torch `tanh` leaves out the lower line of columns whose range crosses zero (its lines
    :416-431 are commented out) while the reference kernel and Verifiers/Bounds.py:1065-1080 compute it, so the
    module's own `tanh_test` can only hold on the upper line there: the lower line is compared on the other columns."""
    kt = _module()
    b = _rand_bound(kt, torch.Generator().manual_seed(1), 1, length, dim_in, dim_out)
    ref, got = b.tanh(), b.cuda_tanh()
    assert kt.relative_error_threshold(ref.ub, got.ub, 0.000001)
    assert kt.relative_error_threshold(ref.uw, got.uw, 0.000001)
    l = b.lb + b.concretize_l()
    u = b.ub + b.concretize_u()
    plain = ((l > 0) | (u < 0))
    assert kt.relative_error_threshold(ref.lb[plain], got.lb[plain], 0.000001)
    m = plain.unsqueeze(2).expand_as(ref.lw)
    assert kt.relative_error_threshold(ref.lw[m], got.lw[m], 0.000001)
    assert torch.allclose(got.ub, ref.ub, rtol=1e-5, atol=1e-6) and torch.allclose(got.uw, ref.uw, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("batch,length,dim_in,dim_out",
                         [(1, 2, 64, 16), (4, 2, 512, 512), (2, 16, 256, 128), (1, 128, 64, 64), (4, 32, 128, 32),
                          (1, 64, 512, 16)])
def test_reference_dot_product_QK_test(batch, length, dim_in, dim_out):
    kt = _module()
    g = torch.Generator().manual_seed(2)
    x = _rand_bound(kt, g, batch, length, dim_in, dim_out)
    y = _rand_bound(kt, g, batch, length, dim_in, dim_out)
    kt.dot_product_QK_test(x, y)
    _two_sided(kt, x.cuda_dot_product_QK(y), x.dot_product(y), _as64(kt, x).dot_product(_as64(kt, y)), "QK")


@pytest.mark.parametrize("batch,length,dim_in,dim_out",
                         [(1, 2, 64, 10), (4, 2, 512, 512), (2, 16, 256, 20), (1, 128, 64, 64), (4, 32, 128, 32)])
def test_reference_dot_product_V_test(batch, length, dim_in, dim_out):
    kt = _module()
    g = torch.Generator().manual_seed(3)
    lb = torch.rand(batch, length, length, generator=g).to(DEV)
    ub = lb + torch.rand(batch, length, length, generator=g).to(DEV)
    lw = (torch.rand(batch, length, dim_in, length, generator=g) - 0.5).to(DEV)
    uw = (torch.rand(batch, length, dim_in, length, generator=g) - 0.5).to(DEV)
    lb1 = torch.rand(batch, dim_out, length, generator=g).to(DEV)
    ub1 = lb1 + torch.rand(batch, dim_out, length, generator=g).to(DEV)
    lw1 = (torch.rand(batch, dim_out, dim_in, length, generator=g) - 0.5).to(DEV)
    uw1 = (torch.rand(batch, dim_out, dim_in, length, generator=g) - 0.5).to(DEV)
    x = kt.Bounds(p=2, eps=0.5, lw=lw, lb=lb, uw=uw, ub=ub)
    y = kt.Bounds(p=2, eps=0.5, lw=lw1, lb=lb1, uw=uw1, ub=ub1)
    kt.dot_product_V_test(x, y)
    _two_sided(kt, x.cuda_dot_product_V(y), x.dot_product(y), _as64(kt, x).dot_product(_as64(kt, y)), "V")


# ------------------------------------------------------------------------------------------------
# The reference's forward verifier, unchanged, on this library's operators: VerifierForward imports
# `Bounds` by name (VerifierForward.py:7); with that name bound to faith_b200.Bounds every operator of
# _bound_input / _bound_layer / _bound_attention / _bound_pooling / _bound_classifier (:127-319) runs on
# the GPU through the C ABI, while the control flow, the head split and merge (:208-229, :253-265) and the
# classifier fold (:289-292) are the reference's own code.

def _verifier_pass(model, emb, positions, p, eps, method="forward"):
    import faith_b200
    words = len(positions)
    ver = reference_loader.build_reference_verifier(model, p, perturbed_words=words, device=DEV, method=method)
    index = positions[0] if words == 1 else positions
    out = []
    for s in range(emb.shape[0]):
        out.append(reference_loader.reference_encoder_pass(ver, emb[s:s + 1].to(DEV), index, eps,
                                                           bounds_cls=faith_b200.Bounds))
    return out


def _noise_ok(got, ref32, ref64, what, c=8.0, floor=0.0):
    """max|got - ref64| <= c * noise + tolerance, the noise being the distance of the oracle's own fp32 evaluation from
    its fp64 evaluation at this stage or, if larger, at an earlier stage (`floor`): one fp32 evaluation is a single
    sample of the rounding noise, and at a late stage that sample can land much closer to the fp64 value than the
    noise it inherited (measured: pooled bias terms 1.7e-4 behind layer outputs at 1.5e-3)."""
    got, ref32, ref64 = got.detach().cpu().double(), ref32.double(), ref64.double()
    noise = max(float((ref32 - ref64).abs().max()), floor)
    err = float((got - ref64).abs().max())
    assert err <= c * noise + 1e-6 + 1e-5 * float(ref64.abs().max()), "%s: error %.3e, fp32 noise of the oracle %.3e" % (
        what, err, noise)
    return noise


@pytest.mark.parametrize("p,positions,eps", [(float("inf"), [1], 0.01), (2.0, [1, 2], 5e-4)])
def test_reference_verifier_runs_unchanged_on_the_gpu_operators(p, positions, eps):
    sys.path.insert(0, os.path.join(HERE, "golden"))
    import cases
    c = cases.ENCODER_CASE
    model = O.make_encoder(c["seed"], c["layers"], c["d_model"], c["heads"], c["ffn"], c["std"])
    emb = cases.encoder_inputs(c)[:2]
    res = _verifier_pass(model, emb, positions, p, eps)
    m64 = O.model_to(model, torch.float64)
    for s, (l, u, stages) in enumerate(res):
        t32, t64 = [], []
        l32, u32 = O.encoder_forward(model, emb[s:s + 1], positions, p, eps, trace=t32)
        l64, u64 = O.encoder_forward(m64, emb[s:s + 1].double(), positions, p, eps, trace=t64)
        t32, t64 = dict(t32), dict(t64)
        floor = 0.0
        for name, b in stages:
            if name not in t32:
                continue
            gl, gu = b.concretize()
            r32l, r32u = t32[name].concretize()
            r64l, r64u = t64[name].concretize()
            # the attention stages live on another scale than the layer outputs: the floor only carries over between
            # the residual-stream stages (layer outputs, pooled, logits)
            stream = name.endswith(".output") or name == "pooled"
            n1 = _noise_ok(gl, r32l, r64l, "sentence %d %s l" % (s, name), floor=floor if stream else 0.0)
            n2 = _noise_ok(gu, r32u, r64u, "sentence %d %s u" % (s, name), floor=floor if stream else 0.0)
            if stream:
                floor = max(floor, n1, n2)
        _noise_ok(l.reshape(1), l32.reshape(1), l64.reshape(1), "logit lower", floor=floor)
        _noise_ok(u.reshape(1), u32.reshape(1), u64.reshape(1), "logit upper", floor=floor)


def test_reference_verifier_on_the_headline_model():
    """One sentence of the headline configuration (3 layers, d_model 128, 4 heads, FFN 512, L 32, one perturbed
    word, L-inf) at eps = 1e-3 through the reference's VerifierForward on faith_b200.Bounds, against the oracle
    and against the C++ whole-model driver."""
    import faith_b200
    model = O.make_encoder(4)
    emb = torch.randn(2, 32, 128, generator=torch.Generator().manual_seed(4))[:1]
    (l, u, _), = _verifier_pass(model, emb, [1], float("inf"), 1e-3)
    l32, u32 = O.encoder_forward(model, emb, [1], float("inf"), 1e-3)
    l64, u64 = O.encoder_forward(O.model_to(model, torch.float64), emb.double(), [1], float("inf"), 1e-3)
    _noise_ok(l.reshape(1), l32.reshape(1), l64.reshape(1), "logit lower")
    _noise_ok(u.reshape(1), u32.reshape(1), u64.reshape(1), "logit upper")
    dl, du, viol = faith_b200.EncoderVerifier(model, DEV).forward(emb.to(DEV), [1], float("inf"), 1e-3)
    assert int(viol.item()) == 0
    _noise_ok(dl.reshape(1), l32.reshape(1), l64.reshape(1), "driver logit lower")
    _noise_ok(du.reshape(1), u32.reshape(1), u64.reshape(1), "driver logit upper")


@pytest.mark.parametrize("method,layer_norm,positions", [("forward", "standard", [1]), ("ibp", "no_var", [1]),
                                                         ("ibp", "standard", [1, 2])])
def test_reference_verifier_other_modes_on_the_gpu_operators(method, layer_norm, positions):
    """The other configurations of the reference verifier, unchanged on faith_b200.Bounds: layer_norm="standard"
    (variance through sqr / sqrt / divide, Bounds.py:1122-1124) and interval mode (--method ibp, every operator's
    interval branch), against the oracle and by containment of the unperturbed forward pass."""
    sys.path.insert(0, os.path.join(HERE, "golden"))
    import cases
    c = dict(cases.ENCODER_CASE, std=0.02, eps=1e-3)
    p = float("inf")
    model = O.make_encoder(c["seed"], c["layers"], c["d_model"], c["heads"], c["ffn"], c["std"], layer_norm=layer_norm)
    emb = cases.encoder_inputs(c)
    res = _verifier_pass(model, emb, positions, p, c["eps"], method=method)
    ibp = method == "ibp"
    l32, u32 = O.encoder_forward(model, emb, positions, p, c["eps"], ibp=ibp)
    l64, u64 = O.encoder_forward(O.model_to(model, torch.float64), emb.double(), positions, p, c["eps"], ibp=ibp)
    y = O.concrete_forward(model, emb)
    for s, (l, u, _) in enumerate(res):
        _noise_ok(l.reshape(1), l32[s:s + 1], l64[s:s + 1], "logit lower", floor=1e-6)
        _noise_ok(u.reshape(1), u32[s:s + 1], u64[s:s + 1], "logit upper", floor=1e-6)
        assert float(l) - 1e-6 <= float(y[s]) <= float(u) + 1e-6
