"""`Bounds`: the reference's bound container and operator API, with every operator on the GPU.

Mirrors Transformer_Verification_Code/Verifiers/Bounds.py: the same constructor
`Bounds(args, p, eps, w=None, b=None, lw=None, lb=None, uw=None, ub=None, clone=True)`, the same
attributes (`lw, uw [B, L, dim_in, dim_out]`, `lb, ub [B, L, dim_out]`, `p`, `eps`,
`perturbed_words`, `batch_size`, `length`, `dim_in`, `dim_out`) and the same methods
(`concretize`, `add`, `multiply`, `matmul`, `dense`, `dot_product`, `context`, `relu`, `tanh`,
`exp`, `reciprocal`, `sqr`, `sqrt`, `divide`, `softmax`, `layer_norm`, `act`, `t`, `clone`), so the reference's
forward verifier (Verifiers/VerifierForward.py) runs on it unchanged, in both of its modes: linear bounds
(`args.method == "forward"`) and interval bounds (`"ibp"`, where the weight tensors shrink to `perturbed_words`
zero rows, Bounds.py:285-288, and every operator takes its interval branch).  All arithmetic is done
by libfaith_b200.so; PyTorch only owns the memory.  There is no CPU path.

`BoundsLite(p, eps, lw, lb, uw, ub)` is the constructor form of the reference's kernel test
(HandTunedKernels/kernel_test/transformer_forward_test_bound.py:33-48).
"""
import math
import types

import torch

from . import ops
from ._lib import FB_EXP, FB_INTERVAL, FB_RECIPROCAL, FB_RELU, FB_SQR, FB_SQRT, FB_TANH, FaithError

EPSILON = 1e-12   # the guard the reference adds to a variance before the root (Bounds.py:27, :1123)


def _c(t):
    return t if t.is_contiguous() else t.contiguous()


class Bounds:
    def __init__(self, args, p, eps, w=None, b=None, lw=None, lb=None, uw=None, ub=None, clone=True):
        self.args = args
        self.ibp = getattr(args, "method", "forward") == "ibp"
        self.p = p
        self.q = 1.0 / (1.0 - 1.0 / p) if p != 1 else float("inf")
        self.eps = eps
        self.perturbed_words = args.perturbed_words
        self.lw = lw if lw is not None else (w.clone() if clone else w)
        self.uw = uw if uw is not None else (w.clone() if clone else w)
        self.lb = lb if lb is not None else (b.clone() if clone else b)
        self.ub = ub if ub is not None else (b.clone() if clone else b)
        self.device = self.lw.device
        self.FLAG = getattr(args, "current_flag", 1)
        if self.ibp:   # interval mode keeps `perturbed_words` rows of (zero) weights, Bounds.py:285-288
            self.lw, self.uw = self.lw[:, :, :self.perturbed_words, :], self.uw[:, :, :self.perturbed_words, :]
        self.update_shape()

    # -------------------------------------------------------------- plumbing
    def update_shape(self):
        self.batch_size, self.length, self.dim_in, self.dim_out = self.lw.shape

    def _new(self, lw, uw, lb, ub):
        return Bounds(self.args, self.p, self.eps, lw=lw, lb=lb, uw=uw, ub=ub)

    def _t4(self):
        return _c(self.lw), _c(self.uw), _c(self.lb), _c(self.ub)

    def clone(self):
        return self._new(self.lw.clone(), self.uw.clone(), self.lb.clone(), self.ub.clone())

    def t(self):
        return self._new(self.lw.transpose(1, 3), self.uw.transpose(1, 3),
                         self.lb.transpose(1, 2), self.ub.transpose(1, 2))

    # ------------------------------------------------------------- operators
    def concretize(self):
        lw, uw, lb, ub = self._t4()
        return ops.concretize(lw, uw, lb, ub, self.p, self.eps, self.perturbed_words)

    def add(self, delta):
        if isinstance(delta, Bounds):
            lw, uw, lb, ub = ops.add(self._t4(), delta._t4())
            return self._new(lw, uw, lb, ub)
        # a constant only moves the bias terms; memory-only op
        return self._new(self.lw, self.uw, self.lb + delta, self.ub + delta)

    def multiply(self, W):
        if isinstance(W, float):
            lw, uw, lb, ub = ops.scale(self._t4(), W)
            return self._new(lw, uw, lb, ub)
        if isinstance(W, Bounds):
            assert self.lw.shape == W.lw.shape
            if self.ibp:
                # box times box: the McCormick planes degenerate to the interval product (Bounds.py:667-678)
                l_a, u_a = self.concretize()
                l_b, u_b = W.concretize()
                lb, ub = ops.interval_mul(l_a, u_a, l_b, u_b)
                zero = torch.zeros_like(self.lw)
                return self._new(zero, zero.clone(), lb, ub)
            lw, uw, lb, ub = ops.mul_bounds(self._t4(), W._t4(), self.p, self.eps, self.perturbed_words)
            return self._new(lw, uw, lb, ub)
        # constant vector over the feature axis (the gain of a layer norm), split by sign (Bounds.py:653-664)
        lw, uw, lb, ub = ops.mul_features(self._t4(), _c(W.detach().reshape(-1)))
        return self._new(lw, uw, lb, ub)

    def matmul(self, W, *unused, **unused_kw):
        if isinstance(W, Bounds) or W.dim() != 2:
            raise NotImplementedError
        lw, uw, lb, ub = self._t4()
        y = ops.matmul(lw, uw, lb, ub, _c(W.detach()), None)
        return self._new(y[0], y[1], y[2], y[3])

    def dense(self, dense, *unused, **unused_kw):
        lw, uw, lb, ub = self._t4()
        y = ops.matmul(lw, uw, lb, ub, _c(dense.weight.detach()), _c(dense.bias.detach()))
        return self._new(y[0], y[1], y[2], y[3])

    def dot_product(self, other, debug=False, verbose=False, lower=True, upper=True):
        if self.dim_in == 1 or self.ibp:
            # interval product of the bias boxes, zero weights: the dim_in == 1 branch (Bounds.py:711-721); in interval
            # mode with two perturbed words the general path reduces to the same sums (its planes are constants)
            lb, ub = ops.interval_dot(_c(self.lb), _c(self.ub), _c(other.lb), _c(other.ub))
            w = torch.zeros(lb.shape[0], lb.shape[1], self.dim_in, lb.shape[2], device=lb.device)
            return self._new(w, w.clone(), lb, ub)
        z = ops.dot_product(self._t4(), other._t4(), self.p, self.eps, self.perturbed_words)
        return self._new(z[0], z[1], z[2], z[3])

    def context(self, value):
        return self.dot_product(value.t())

    def _relax(self, op):
        lw, uw, lb, ub = self._t4()
        violation = None
        if op in (FB_RECIPROCAL, FB_SQRT):
            violation = torch.zeros(1, dtype=torch.int32, device=lw.device)
        o = ops.relax(op + (FB_INTERVAL if self.ibp else 0), lw, uw, lb, ub, self.p, self.eps, self.perturbed_words,
                      violation=violation)
        if violation is not None and int(violation.item()) != 0:
            raise AssertionError("reciprocal or square root of a bound that is not strictly positive")
        return self._new(o[0], o[1], o[2], o[3])

    def sqr(self):
        return self._relax(FB_SQR)

    def sqrt(self):
        return self._relax(FB_SQRT)

    def relu(self):
        return self._relax(FB_RELU)

    def tanh(self):
        return self._relax(FB_TANH)

    def exp(self):
        return self._relax(FB_EXP)

    def reciprocal(self):
        return self._relax(FB_RECIPROCAL)

    def act(self, act_name):
        if act_name == "relu":
            return self.relu()
        raise NotImplementedError

    def divide(self, W):
        if isinstance(W, Bounds):
            return self.multiply(W.reciprocal())
        raise NotImplementedError

    def softmax(self, verbose=False):
        violation = torch.zeros(1, dtype=torch.int32, device=self.lw.device)
        fused = None if self.ibp else ops.softmax_fused(self._t4(), self.p, self.eps, self.perturbed_words, violation)
        if fused is not None:
            if int(violation.item()) != 0:
                raise AssertionError("reciprocal of a bound that is not strictly positive")
            return self._new(fused[0], fused[1], fused[2], fused[3])
        e = self.exp()
        s = ops.rowsum(e._t4())
        return e.divide(self._new(s[0], s[1], s[2], s[3]))

    def layer_norm(self, normalizer, layer_norm):
        if layer_norm == "no":
            return self
        if layer_norm == "no_var":
            o = ops.layernorm_novar(self._t4(), _c(normalizer.weight.detach()), _c(normalizer.bias.detach()))
            return self._new(o[0], o[1], o[2], o[3])
        if layer_norm != "standard":
            raise NotImplementedError("layer_norm mode %r" % (layer_norm,))
        # Bounds.py:1111-1131: x - mean, variance = mean of the squares, division by its root, gain and shift; the mean
        # subtraction is the no_var kernel with unit gain, the rest is the reference's own chain of operators
        ones = torch.ones(self.dim_out, device=self.device)
        zeros = torch.zeros(self.dim_out, device=self.device)
        o = ops.layernorm_novar(self._t4(), ones, zeros)
        minus_mu = self._new(o[0], o[1], o[2], o[3])
        w_avg = torch.full((self.dim_out, self.dim_out), 1.0 / self.dim_out, device=self.device)
        variance = minus_mu.sqr().matmul(w_avg)
        normalized = minus_mu.divide(variance.add(EPSILON).sqrt())
        return normalized.multiply(normalizer.weight).add(normalizer.bias)

    def print(self, message):
        print(message)
        l, u = self.concretize()
        print("mean abs %.5f %.5f" % (torch.mean(torch.abs(l)), torch.mean(torch.abs(u))))
        print("diff %.5f %.5f %.5f" % (torch.min(u - l), torch.max(u - l), torch.mean(u - l)))


def BoundsLite(p, eps, lw, lb, uw, ub, perturbed_words=1, ibp=False):
    """Constructor form of the reference's kernel test class (ibp=True: interval mode, `--method ibp`)."""
    args = types.SimpleNamespace(method="ibp" if ibp else "forward", perturbed_words=perturbed_words, current_flag=1)
    return Bounds(args, p, eps, lw=lw, lb=lb, uw=uw, ub=ub)
