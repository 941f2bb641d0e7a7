"""Parity at the benchmark's own operator configurations (shapes, seeds, norms and radii of the
benchmark description; synthetic inputs stand in for the reference's SST / Yelp data and trained
checkpoints, which are not available):

  C1  Linear + ReLU   lw [1,16,64,64] -> [1,16,64,128], identity lw at word 0, L-inf, eps 0.01
  C2  Q K^T           two perturbed words (dim_in 128), p = 2, eps 0.05, 4 heads of 32 features
  C3  Tanh + Linear   [8,64,256,256], four perturbed words, p = 1 (q = inf), eps 0.1
  C4  the headline pass: 32 of the 256 benchmark sentences through the whole-model driver, eps 0.01 and 1e-3
  C5  the CNN pass on one 3x32x32 image, every pixel perturbed (dim_in 3072)

Each is compared with the oracle (pinned to the reference in tests/test_oracle_*.py) on identical
seeded inputs within the per-operator bar; C3 is compared operator by operator on two of its eight
batch rows and checked for finiteness and ordering at full size.
"""
import math
import types

import pytest
import torch

import helpers
from oracle import bounds_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _input_bounds(x0, positions):
    """Identity weights at the perturbed positions (VerifierForward.py:127-156)."""
    B, L, D = x0.shape
    Di = D * len(positions)
    lw = torch.zeros(B, L, Di, D)
    for w, pos in enumerate(positions):
        lw[:, pos, w * D:(w + 1) * D] = torch.eye(D)
    return lw, x0.clone(), lw.clone(), x0.clone()    # lw, lb, uw, ub


def _gpu(p, eps, t, words):
    import faith_b200
    return faith_b200.BoundsLite(p, eps, *[v.to(DEV) for v in t], perturbed_words=words)


def _dbl(t):
    return [v.double() for v in t]


def _cmp(g, o, what, rtol=1e-5, atol=1e-6):
    for k in ("lw", "uw", "lb", "ub"):
        helpers.assert_close(getattr(g, k), getattr(o, k), "%s %s" % (what, k), rtol=rtol, atol=atol)


def test_config1_linear_relu():
    g0 = torch.Generator().manual_seed(1)
    x0 = torch.randn(1, 16, 64, generator=g0)
    W = torch.randn(128, 64, generator=g0) / 8
    bias = 0.1 * torch.randn(128, generator=g0)
    t = _input_bounds(x0, [0])
    p, eps = float("inf"), 0.01
    o = O.OBounds(p, eps, *t).dense(W, bias).relu()
    o64 = O.OBounds(p, eps, *_dbl(t)).dense(W.double(), bias.double()).relu()
    g = _gpu(p, eps, t, 1).dense(types.SimpleNamespace(weight=W.to(DEV), bias=bias.to(DEV))).relu()
    helpers.assert_bounds_arbitrated(g, o, o64, "C1 linear+relu")
    gl, gu = g.concretize()
    ol, ou = o.concretize()
    ol64, ou64 = o64.concretize()
    helpers.assert_arbitrated(gl, ol, ol64, "C1 concretised l")
    helpers.assert_arbitrated(gu, ou, ou64, "C1 concretised u")


def test_config2_query_key_product():
    from faith_b200 import ops
    g0 = torch.Generator().manual_seed(2)
    x0 = torch.randn(1, 32, 64, generator=g0)
    Wq = torch.randn(128, 64, generator=g0) / math.sqrt(128)
    Wk = torch.randn(128, 64, generator=g0) / math.sqrt(128)
    zero = torch.zeros(128)
    t = _input_bounds(x0, [1, 2])
    p, eps, heads = 2.0, 0.05, 4
    ox = O.OBounds(p, eps, *t, words=2)
    oq, ok = O.split_heads(ox.dense(Wq, zero), heads), O.split_heads(ox.dense(Wk, zero), heads)
    oz = oq.dot_product(ok)
    ox64 = O.OBounds(p, eps, *_dbl(t), words=2)
    oz64 = O.split_heads(ox64.dense(Wq.double(), zero.double()), heads).dot_product(
        O.split_heads(ox64.dense(Wk.double(), zero.double()), heads))
    gx = _gpu(p, eps, t, 2)

    def proj(W):
        y = gx.dense(types.SimpleNamespace(weight=W.to(DEV), bias=zero.to(DEV)))
        s = ops.split_heads(y._t4(), heads, False)
        return y._new(s[0], s[1], s[2], s[3])

    gq, gk = proj(Wq), proj(Wk)
    assert tuple(gq.lw.shape) == (4, 32, 128, 32)
    gz = gq.dot_product(gk)
    assert tuple(gz.lw.shape) == (4, 32, 128, 32) and tuple(gz.lb.shape) == (4, 32, 32)
    # GEMM-shaped: two fp32 summation orders; the fp64 run of the same algorithm is the arbiter
    helpers.assert_bounds_arbitrated(gz, oz, oz64, "C2 q k^T")


def test_config3_tanh_linear():
    g0 = torch.Generator().manual_seed(3)
    x0 = torch.randn(8, 64, 64, generator=g0)
    W1 = torch.randn(256, 64, generator=g0) / 16
    W2 = torch.randn(256, 256, generator=g0) / 16
    positions = [1, 2, 3, 4]
    t = _input_bounds(x0, positions)
    p, eps = 1.0, 0.1
    gh = _gpu(p, eps, t, 4).matmul(W1.to(DEV))
    assert tuple(gh.lw.shape) == (8, 64, 256, 256)
    gt = gh.tanh()
    gy = gt.matmul(W2.to(DEV))
    for b in (gt, gy):
        for k in ("lw", "uw", "lb", "ub"):
            assert bool(torch.isfinite(getattr(b, k)).all())
        l, u = b.concretize()
        assert bool((l <= u + 1e-5).all())
    # Oracle on two batch rows, operator by operator on identical inputs: each oracle operator is fed
    # the GPU result of the previous one.  (Chained end to end, the 10-step bisection of the tanh
    # relaxation turns a last-bit difference of its input range into a different tangent point for a few
    # per cent of the columns, i.e. 1e-5-sized jumps that say nothing about either implementation.)
    t2 = [v[:2] for v in t]
    oh = O.OBounds(p, eps, *t2, words=4).matmul(W1)
    sub = lambda b: types.SimpleNamespace(lw=b.lw[:2], uw=b.uw[:2], lb=b.lb[:2], ub=b.ub[:2])
    helpers.assert_bounds_arbitrated(sub(gh), oh, O.OBounds(p, eps, *_dbl(t2), words=4).matmul(W1.double()), "C3 first linear")
    cpu = lambda b, dt=torch.float32: O.OBounds(p, eps, b.lw[:2].cpu().to(dt), b.lb[:2].cpu().to(dt), b.uw[:2].cpu().to(dt),
                                                b.ub[:2].cpu().to(dt), words=4)
    # The tanh relaxation finds its tangent points by a 10-step bisection on tanhf / coshf values: a last-bit difference
    # between two libm implementations (the GPU's, the host's, which itself varies with the host's vector unit) moves
    # a tangent point by one step for a few per cent of the columns here (ranges of several units), a 1e-5-sized jump
    # in the line that says nothing about either implementation.  The fp64 run of the same algorithm is the arbiter.
    helpers.assert_bounds_arbitrated(sub(gt), cpu(gh).tanh(), cpu(gh, torch.float64).tanh(), "C3 tanh")
    helpers.assert_bounds_arbitrated(sub(gy), cpu(gt).matmul(W2), cpu(gt, torch.float64).matmul(W2.double()),
                                     "C3 linear after tanh")


def test_config5_cnn_full_size_properties():
    """C5: 3x32x32 image, every pixel perturbed (dim_in = 3072), L-inf eps 2/255; conv 3->16, relu, conv 16->32
    stride 2, relu, linear 8192->10.  At full size: finite, ordered, and 512 sampled images of the ball
    (half of them on vertices) plus the unperturbed image land inside the interval.  (Parity of the same pass
    with the oracle is checked on a smaller image in test_gpu_sharded.py, parity of the conv operator at the
    first layer's full shape in test_gpu_ops.py::test_conv_bounds.)"""
    import torch.nn.functional as F
    from faith_b200.sharded import CnnVerifier
    layers = O.make_cnn(5)
    img = torch.rand(3, 32, 32, generator=torch.Generator().manual_seed(5))
    eps = 2.0 / 255
    l, u = CnnVerifier(layers, DEV).forward(img, float("inf"), eps)
    l, u = l.cpu(), u.cpu()
    assert tuple(l.shape) == (10,) or l.numel() == 10
    assert bool(torch.isfinite(l).all()) and bool(torch.isfinite(u).all())
    assert bool((l <= u).all())

    def net(x):
        for ly in layers:
            if ly[0] == "conv":
                x = F.conv2d(x, ly[1], ly[2], ly[3], ly[4])
            elif ly[0] == "relu":
                x = torch.relu(x)
            else:
                x = F.linear(x.flatten(1), ly[1], ly[2])
        return x
    g = torch.Generator().manual_seed(6)
    n = 512
    delta = (torch.randint(0, 2, (n, 3, 32, 32), generator=g).float() * 2 - 1) * eps
    delta[: n // 2] *= torch.rand(n // 2, 1, 1, 1, generator=g)
    x = torch.cat([img.unsqueeze(0), img.unsqueeze(0) + delta])
    y = net(x)
    assert bool((y >= l.reshape(1, -1) - 1e-4).all()) and bool((y <= u.reshape(1, -1) + 1e-4).all())


def test_config5_cnn_full_size_against_the_oracle():
    """C5 at full size against the CPU oracle: the whole pass (both paths of the driver: the structured one and the one
    that materialises the identity and runs every convolution densely), and the two convolutions on their own at
    dim_in = 3072, the second one (16 -> 32, stride 2) on the relaxed output of the first."""
    from faith_b200 import ops
    from faith_b200.sharded import CnnVerifier
    layers = O.make_cnn(5)
    img = torch.rand(3, 32, 32, generator=torch.Generator().manual_seed(5))
    eps, p = 2.0 / 255, float("inf")
    ol, ou = O.cnn_forward(layers, img, p, eps)
    l64, u64 = O.cnn_forward([tuple(t.double() if isinstance(t, torch.Tensor) else t for t in ly) for ly in layers],
                             img.double(), p, eps)
    ver = CnnVerifier(layers, DEV)
    for dense in (False, True):
        l, u = ver.forward(img, p, eps, dense=dense)
        helpers.assert_within_noise(l, ol, l64, "l dense=%s" % dense)
        helpers.assert_within_noise(u, ou, u64, "u dense=%s" % dense)
    di = 3072
    eye = torch.eye(di).view(1, di, 3, 32, 32)
    x0 = O.OBounds(p, eps, eye, img.unsqueeze(0), eye.clone(), img.unsqueeze(0))
    o1 = O.conv_bounds(x0, layers[0][1], layers[0][2], layers[0][3], layers[0][4])
    g1 = ops.conv2d((eye.to(DEV), eye.to(DEV), img.unsqueeze(0).to(DEV), img.unsqueeze(0).to(DEV)),
                    layers[0][1].to(DEV), layers[0][2].to(DEV), layers[0][3], layers[0][4])
    for a, k in zip(g1, ("lw", "uw", "lb", "ub")):
        helpers.assert_close(a, getattr(o1, k), "conv1 " + k)
    r1 = O.tokens_as_conv(O.conv_as_tokens(o1).relu(), *o1.lb.shape[1:])
    o2 = O.conv_bounds(r1, layers[2][1], layers[2][2], layers[2][3], layers[2][4])
    g2 = ops.conv2d((r1.lw.to(DEV), r1.uw.to(DEV), r1.lb.to(DEV), r1.ub.to(DEV)), layers[2][1].to(DEV), layers[2][2].to(DEV),
                    layers[2][3], layers[2][4])
    r64 = O.OBounds(p, eps, r1.lw.double(), r1.lb.double(), r1.uw.double(), r1.ub.double())
    o2_64 = O.conv_bounds(r64, layers[2][1].double(), layers[2][2].double(), layers[2][3], layers[2][4])
    for a, k in zip(g2, ("lw", "uw", "lb", "ub")):
        # K = 144 products: two fp32 summation orders, the fp64 run is the arbiter
        helpers.assert_arbitrated(a, getattr(o2, k), getattr(o2_64, k), "C5 conv2 at dim_in 3072 " + k)


@pytest.mark.parametrize("eps", [0.01, 1e-3])
def test_config4_headline_sentences_of_the_benchmark(eps):
    """C4, the measured configuration itself: 3-layer encoder (d_model 128, 4 heads, FFN 512), L = 32, word 1 perturbed,
    L-inf, on every eighth of the benchmark's 256 sentences (same seed, same generator call) at the benchmark's
    eps = 0.01 and at 1e-3.  Finite, ordered, no violation or give-up bit; within the fp32 noise of the fp64 oracle on
    four of them; and 10 240 concrete forward passes of the full-size model (per sentence 160 vertices of the ball and
    160 interior points, run with plain torch on the GPU) land inside [l, u]."""
    import faith_b200
    model = O.make_encoder(4)
    emb_all = torch.randn(256, 32, 128, generator=torch.Generator().manual_seed(4))
    emb = emb_all[::8].contiguous()
    p, index = float("inf"), 1
    ver = faith_b200.EncoderVerifier(model, DEV)
    l, u, viol = ver.forward(emb.to(DEV), [index], p, eps)
    assert ver.check_status(viol) == 0
    assert bool(torch.isfinite(l).all()) and bool(torch.isfinite(u).all())
    assert bool((l <= u).all())
    l32, u32 = O.encoder_forward(model, emb[:4], [index], p, eps)
    l64, u64 = O.encoder_forward(O.model_to(model, torch.float64), emb[:4].double(), [index], p, eps)
    helpers.assert_within_noise(l[:4], l32, l64, "l eps=%g" % eps)
    helpers.assert_within_noise(u[:4], u32, u64, "u eps=%g" % eps)
    model_dev = O.model_to(model, DEV)
    g = torch.Generator().manual_seed(10)
    n = 320
    for s in range(emb.shape[0]):
        delta = (torch.randint(0, 2, (n, 128), generator=g).float() * 2 - 1) * eps
        delta[: n // 2] *= torch.rand(n // 2, 1, generator=g)
        x = emb[s:s + 1].repeat(n, 1, 1)
        x[:, index, :] += delta
        y = O.concrete_forward(model_dev, x.to(DEV))
        assert float(y.min()) >= float(l[s]) - 1e-5, (s, float(y.min()), float(l[s]))
        assert float(y.max()) <= float(u[s]) + 1e-5, (s, float(y.max()), float(u[s]))
