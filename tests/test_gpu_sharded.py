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
