"""dim_in-sharded relaxation and the CNN pass on one GPU: the shards of several ranks are processed
one after the other, their partial norms combined on the host side of the test, and the result
compared with the unsharded kernel and the oracle."""
import pytest
import torch

import cases
import helpers
from oracle import bounds_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("p", [1.0, 2.0, float("inf")])
@pytest.mark.parametrize("world", [1, 2, 3])
def test_sharded_relu_matches_unsharded(p, world):
    from faith_b200 import ops, sharded
    from faith_b200._lib import FB_RELU
    lw, lb, uw, ub = [t.to(DEV) for t in cases.rand_bounds(801, 2, 3, 50, 36, -0.7, 0.2)]
    shards = [sharded.shard_bounds(lw, uw, r, world) for r in range(world)]
    parts = [ops.norm_partials(s[0], s[1], p) for s in shards]
    red = torch.max if p == 1 else torch.add
    nl, nu = parts[0]
    for pl, pu in parts[1:]:
        nl, nu = red(nl, pl), red(nu, pu)
    outs = [ops.relax_with_norms(FB_RELU, s[0], s[1], lb, ub, nl.contiguous(), nu.contiguous(), p, 0.5) for s in shards]
    g_lw = torch.cat([o[0] for o in outs], dim=-2)
    g_uw = torch.cat([o[1] for o in outs], dim=-2)
    ref = O.OBounds(p, 0.5, lw.cpu(), lb.cpu(), uw.cpu(), ub.cpu()).relu()
    helpers.assert_close(g_lw, ref.lw, "lw")
    helpers.assert_close(g_uw, ref.uw, "uw")
    for o in outs:   # bias terms are replicated
        helpers.assert_close(o[2], ref.lb, "lb")
        helpers.assert_close(o[3], ref.ub, "ub")


def test_cnn_pass_matches_oracle():
    from faith_b200.sharded import CnnVerifier
    layers = O.make_cnn(5, c_in=3, hw=8)
    img = torch.rand(3, 8, 8, generator=torch.Generator().manual_seed(5))
    ol, ou = O.cnn_forward(layers, img, float("inf"), 2.0 / 255)
    l64, u64 = O.cnn_forward([tuple(t.double() if isinstance(t, torch.Tensor) else t for t in ly) for ly in layers],
                             img.double(), float("inf"), 2.0 / 255)
    l, u = CnnVerifier(layers, DEV).forward(img, float("inf"), 2.0 / 255)
    helpers.assert_within_noise(l, ol, l64, "l")
    helpers.assert_within_noise(u, ou, u64, "u")
    # soundness: the unperturbed image and random points of the ball land inside
    import torch.nn.functional as F

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
    x = img.unsqueeze(0) + (torch.rand(256, 3, 8, 8, generator=g) * 2 - 1) * (2.0 / 255)
    y = net(x)
    assert bool((y >= l.cpu() - 1e-5).all()) and bool((y <= u.cpu() + 1e-5).all())


@pytest.mark.parametrize("stride,pad,hw", [(1, 1, 8), (2, 1, 9)])
def test_first_convolution_from_the_filter_alone(stride, pad, hw):
    """fb_conv2d_identity_relax_f32 (first convolution + relu of an all-pixels-perturbed image, written from the filter
    alone, for a shard of the rows) against the general kernels on the materialised identity and against the oracle."""
    from faith_b200 import ops, sharded
    from faith_b200._lib import FB_RELU
    g = torch.Generator().manual_seed(31)
    C, Co, eps = 3, 5, 0.05
    img = torch.rand(C, hw, hw, generator=g)
    wt = torch.randn(Co, C, 3, 3, generator=g) * 0.3
    bias = torch.randn(Co, generator=g) * 0.1
    di = C * hw * hw
    eye = torch.eye(di).view(1, di, C, hw, hw)
    for p in (1.0, 2.0, float("inf")):
        ob = O.conv_bounds(O.OBounds(p, eps, eye, img.unsqueeze(0), eye.clone(), img.unsqueeze(0)), wt, bias, stride, pad)
        flat = O.conv_as_tokens(ob)
        ref = O.tokens_as_conv(flat.relu(), *ob.lb.shape[1:])
        start, rows = 17, di - 40      # a shard in the middle of dim_in
        lb = img.unsqueeze(0).to(DEV)
        got = sharded.conv_identity_relax(FB_RELU, lb, lb.clone(), wt.to(DEV), bias.to(DEV), rows, start, stride, pad, p, eps)
        helpers.assert_close(got[0][0], ref.lw[0, start:start + rows], "lw p=%s" % p)
        helpers.assert_close(got[1][0], ref.uw[0, start:start + rows], "uw p=%s" % p)
        helpers.assert_close(got[2], ref.lb, "lb p=%s" % p)
        helpers.assert_close(got[3], ref.ub, "ub p=%s" % p)
        plain = sharded.conv_identity_relax(None, lb, lb.clone(), wt.to(DEV), bias.to(DEV), rows, start, stride, pad, p, eps)
        helpers.assert_close(plain[0][0], ob.lw[0, start:start + rows], "conv lw")
        helpers.assert_close(plain[3], ob.ub, "conv ub")


@pytest.mark.parametrize("hw,geoms,start,drop", [
    (10, [(3, 1, 1), (3, 2, 1)], 0, 0),                # the benchmark CNN's geometry; width 5 after: scalar stores
    (16, [(3, 1, 1), (3, 2, 1), (3, 1, 1)], 0, 0),     # three convolutions; widths 16, 8, 8: 16-byte stores
    (12, [(3, 2, 1), (5, 1, 2), (3, 2, 0)], 29, 61),   # strided first layer, 5x5 taps, no padding; a shard of dim_in
    (9, [(2, 3, 0), (3, 1, 1)], 0, 0),                 # stride above the kernel size: some pixels reach nothing
])
def test_windowed_convolution_equals_the_dense_kernel_bit_for_bit(hw, geoms, start, drop):
    """Later convolutions of rows that are zero outside the window of their pixel: the windowed kernel against the dense
    one on the same rows, layer after layer (geoms: kernel size, stride, padding per convolution)."""
    from faith_b200 import ops, sharded
    from faith_b200._lib import FB_RELU
    g = torch.Generator().manual_seed(32)
    C, eps = 3, 0.05
    chans = [C, 6, 7, 5][:len(geoms) + 1]
    img = torch.rand(C, hw, hw, generator=g)
    ws = [(torch.randn(chans[i + 1], chans[i], k, k, generator=g) * 0.3).to(DEV) for i, (k, _, _) in enumerate(geoms)]
    bs = [(torch.randn(chans[i + 1], generator=g) * 0.1).to(DEV) for i in range(len(geoms))]
    di = C * hw * hw
    rows = di - start - drop
    lb = img.unsqueeze(0).to(DEV)
    k, stride, pad = geoms[0]
    x = sharded.conv_identity_relax(FB_RELU, lb, lb.clone(), ws[0], bs[0], rows, start, stride, pad, float("inf"), eps)
    chain = [(k, k, stride, pad)]
    for (k, stride, pad), w, b in zip(geoms[1:], ws[1:], bs[1:]):
        dense = ops.conv2d(x, w, b, stride, pad)
        win = sharded.conv_windowed(x, w, b, stride, pad, start, hw, hw, chain)
        for got, want, name in zip(win, dense, ("lw", "uw", "lb", "ub")):
            assert torch.equal(got, want), (name, len(chain))
        assert float(dense[0].abs().max()) > 0
        chain.append((k, k, stride, pad))
        x = win


@pytest.mark.parametrize("hw,geoms,start,drop", [
    (10, [(3, 1, 1), (3, 2, 1)], 0, 0),
    (16, [(3, 1, 1), (3, 2, 1), (3, 1, 1)], 0, 0),
    (12, [(3, 2, 1), (5, 1, 2), (3, 2, 0)], 29, 61),
    (9, [(2, 3, 0), (3, 1, 1)], 0, 0),
])
def test_compact_rows_expand_to_the_dense_rows_bit_for_bit(hw, geoms, start, drop):
    """The compact form of the CNN operators (a row stored as its window only) against the dense-row kernels, layer
    after layer: first convolution + relu, later convolutions, the relaxation between them (given the same norms), all
    expanded and compared bit for bit; the gathered column norms against the dense reduction within rounding; the
    linear head on compact rows against the dense product."""
    from faith_b200 import ops, sharded
    from faith_b200._lib import FB_RELU
    g = torch.Generator().manual_seed(33)
    C, eps, p = 3, 0.05, float("inf")
    chans = [C, 6, 7, 5][:len(geoms) + 1]
    img = torch.rand(C, hw, hw, generator=g)
    ws = [(torch.randn(chans[i + 1], chans[i], k, k, generator=g) * 0.3).to(DEV) for i, (k, _, _) in enumerate(geoms)]
    bs = [(torch.randn(chans[i + 1], generator=g) * 0.1).to(DEV) for i in range(len(geoms))]
    rows = C * hw * hw - start - drop
    lb = img.unsqueeze(0).to(DEV)
    k, stride, pad = geoms[0]
    dense = sharded.conv_identity_relax(FB_RELU, lb, lb.clone(), ws[0], bs[0], rows, start, stride, pad, p, eps)
    z = sharded.cw_identity_relax(FB_RELU, lb, lb.clone(), ws[0], bs[0], rows, start, stride, pad, p, eps)
    chain = [(k, k, stride, pad)]
    h = dense[0].shape[-1]

    def same(z_pair, dense_pair, what):
        e = sharded.cw_expand(z_pair[0], z_pair[1], start, hw, hw, chain, h, h)
        assert torch.equal(e[0], dense_pair[0][0]) and torch.equal(e[1], dense_pair[1][0]), what

    same(z, dense, "first convolution + relu")
    assert torch.equal(z[2], dense[2]) and torch.equal(z[3], dense[3])
    for (k, stride, pad), w, b in zip(geoms[1:], ws[1:], bs[1:]):
        d2 = sharded.conv_windowed(dense, w, b, stride, pad, start, hw, hw, chain)
        z2 = sharded.cw_conv(z[0], z[1], w, stride, pad, start, hw, hw, chain, h, h)
        chain = chain + [(k, k, stride, pad)]
        h = d2[0].shape[-1]
        same(z2, d2, "convolution %d" % len(chain))
        # the relaxation behind it: norms by the gather over compact rows against the dense reduction
        feat = d2[2].numel()
        pl, pu = ops.norm_partials(d2[0].reshape(1, rows, feat), d2[1].reshape(1, rows, feat), p)
        cl, cu = sharded.cw_norm_partials(z2[0], z2[1], start, C, hw, hw, chain, h, h, p)
        helpers.assert_close(cl, pl.reshape(-1), "norm partials l", rtol=1e-6, atol=1e-7)
        helpers.assert_close(cu, pu.reshape(-1), "norm partials u", rtol=1e-6, atol=1e-7)
        for pp in (1.0, 2.0):
            ql, _ = ops.norm_partials(d2[0].reshape(1, rows, feat), d2[1].reshape(1, rows, feat), pp)
            rl, _ = sharded.cw_norm_partials(z2[0], z2[1], start, C, hw, hw, chain, h, h, pp)
            helpers.assert_close(rl, ql.reshape(-1), "norm partials p=%s" % pp, rtol=1e-6, atol=1e-7)
        dr = ops.relax_with_norms(FB_RELU, d2[0].reshape(1, rows, feat), d2[1].reshape(1, rows, feat), d2[2].reshape(1, feat),
                                  d2[3].reshape(1, feat), pl, pu, p, eps)
        zr = sharded.cw_relax_apply(FB_RELU, z2[0], z2[1], d2[2].reshape(-1), d2[3].reshape(-1), pl.reshape(-1), pu.reshape(-1),
                                    start, hw, hw, chain, h, h, p, eps)
        dense = (dr[0].view(d2[0].shape), dr[1].view(d2[1].shape), dr[2].view(d2[2].shape), dr[3].view(d2[3].shape))
        z = zr
        same(z, dense, "relaxation %d" % len(chain))
        assert torch.equal(z[2], dense[2].reshape(-1)) and torch.equal(z[3], dense[3].reshape(-1))
    # the head: 11 outputs (two groups of eight in the kernel)
    feat = dense[2].numel()
    wl = (torch.randn(11, feat, generator=g) / feat ** 0.5).to(DEV)
    dl = ops.matmul(dense[0].reshape(1, 1, rows, feat), dense[1].reshape(1, 1, rows, feat), dense[2].reshape(1, 1, feat),
                    dense[3].reshape(1, 1, feat), wl, None)
    yl, yu = sharded.cw_linear(z[0], z[1], wl, start, hw, hw, chain, h, h)
    helpers.assert_close(yl, dl[0].reshape(rows, 11), "linear lw", atol=2e-6)
    helpers.assert_close(yu, dl[1].reshape(rows, 11), "linear uw", atol=2e-6)


def test_windowed_convolution_rejects_a_chain_that_does_not_lead_to_its_input():
    from faith_b200 import sharded, FaithError
    x = tuple(torch.zeros(s, device=DEV) for s in ((1, 4, 2, 6, 6), (1, 4, 2, 6, 6), (1, 2, 6, 6), (1, 2, 6, 6)))
    w = torch.zeros(3, 2, 3, 3, device=DEV)
    with pytest.raises(FaithError):
        sharded.conv_windowed(x, w, None, 1, 1, 0, 6, 6, [(3, 3, 2, 1)])    # 6x6 through stride 2 is 3x3, not 6x6


@pytest.mark.parametrize("rows,Di,Do", [(1, 3072, 10), (2, 700, 36), (1, 1000, 64), (1, 2048, 96), (3, 513, 7)])
def test_norm_partials_of_tall_operands(rows, Di, Do):
    """Few column tiles, many dim_in rows: the cluster-split kernels (flat walk for narrow outputs, column tiles
    otherwise) against a plain reduction, for the three norms."""
    from faith_b200 import ops
    g = torch.Generator().manual_seed(91)
    lw = torch.randn(rows, Di, Do, generator=g)
    uw = torch.randn(rows, Di, Do, generator=g)
    for p, red in ((float("inf"), lambda t: t.abs().sum(1)), (2.0, lambda t: (t.double() ** 2).sum(1).float()),
                   (1.0, lambda t: t.abs().amax(1))):
        pl, pu = ops.norm_partials(lw.to(DEV), uw.to(DEV), p)
        helpers.assert_close(pl, red(lw), "partials l p=%s" % p, rtol=2e-6, atol=1e-6)
        helpers.assert_close(pu, red(uw), "partials u p=%s" % p, rtol=2e-6, atol=1e-6)
        again = ops.norm_partials(lw.to(DEV), uw.to(DEV), p)
        assert torch.equal(again[0], pl) and torch.equal(again[1], pu)    # fixed order of additions


def test_cnn_pass_structured_path_equals_dense_path():
    """The C driver by both of its routes (compact rows; dense rows with windowed convolutions) against the operator-by-
    operator pass on the materialised identity."""
    from faith_b200.sharded import CnnVerifier
    layers = O.make_cnn(5, c_in=3, hw=8)
    img = torch.rand(3, 8, 8, generator=torch.Generator().manual_seed(5))
    ver = CnnVerifier(layers, DEV)
    ver_rows = CnnVerifier(layers, DEV, compact=False)
    for p in (1.0, 2.0, float("inf")):
        l0, u0 = ver.forward(img, p, 2.0 / 255, dense=True)
        for v, name in ((ver, "compact"), (ver_rows, "dense rows")):
            l1, u1 = v.forward(img, p, 2.0 / 255)
            helpers.assert_close(l1, l0, "l p=%s %s" % (p, name))
            helpers.assert_close(u1, u0, "u p=%s %s" % (p, name))


def test_cnn_driver_other_layer_sequences():
    """Networks the driver has to take other ways through: no relu behind the first convolution, three convolutions, a
    hidden linear layer with a relu behind it, and a network that ends on a feature map (no linear layer)."""
    from faith_b200.sharded import CnnVerifier
    g = torch.Generator().manual_seed(44)

    def conv(co, ci, k, s, p):
        return ("conv", torch.randn(co, ci, k, k, generator=g) * (2.0 / (ci * k * k)) ** 0.5, torch.randn(co, generator=g) * 0.1, s, p)

    def lin(n, k):
        return ("linear", torch.randn(n, k, generator=g) / k ** 0.5, torch.randn(n, generator=g) * 0.1)

    img = torch.rand(2, 8, 8, generator=g)
    nets = [
        [conv(4, 2, 3, 1, 1), conv(6, 4, 3, 2, 1), ("relu",), lin(5, 6 * 4 * 4)],
        [conv(4, 2, 3, 1, 1), ("relu",), conv(6, 4, 3, 2, 1), ("relu",), conv(3, 6, 3, 1, 1), ("relu",), lin(7, 3 * 4 * 4)],
        [conv(4, 2, 3, 2, 1), ("relu",), lin(20, 4 * 4 * 4), ("relu",), lin(3, 20)],
        [conv(4, 2, 3, 1, 1), ("relu",), conv(5, 4, 3, 2, 1)],
    ]
    for i, layers in enumerate(nets):
        ref = CnnVerifier(layers, DEV).forward(img, float("inf"), 0.01, dense=True)
        for compact in (True, False):
            got = CnnVerifier(layers, DEV, compact=compact).forward(img, float("inf"), 0.01)
            helpers.assert_close(got[0], ref[0], "net %d l compact=%s" % (i, compact), atol=2e-6)
            helpers.assert_close(got[1], ref[1], "net %d u compact=%s" % (i, compact), atol=2e-6)
