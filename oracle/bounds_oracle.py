"""CPU oracle for forward linear-bound propagation (TEST INFRASTRUCTURE, not product code).

A restatement, in plain PyTorch on the CPU, of the arithmetic of the reference's
`Bounds` operators (Transformer_Verification_Code/Verifiers/Bounds.py).  It exists so
that the CUDA path can be checked on machines where the reference checkout is not
present.  Only tests, the smoke check and the CPU-baseline legs of the benchmark may
import it; the product package never does.

Pinning: every operator here is compared with the reference module itself (imported
unchanged, on CPU) by `tests/test_oracle_vs_reference.py` when the reference checkout is
available, and with the committed golden vectors under `tests/golden/` (generated from
the reference by `tests/golden/make_golden.py`) everywhere else.  The convolution operator
is the exception: the reference has no runnable Python for it, so it is "parity unpinned"
at the level of the reference's own tests and is tied to the pinned `matmul` through an
im2col cross-check instead.

A bound object carries, for every activation x[b, l, j], two affine functions of the
perturbation delta (one block of `dim_in / words` coordinates per perturbed word):

    lw[b,l,:,j] . delta + lb[b,l,j]  <=  x[b,l,j]  <=  uw[b,l,:,j] . delta + ub[b,l,j]

with lw, uw : [B, L, Di, Do] and lb, ub : [B, L, Do]      (Bounds.py:270-297).
The dtype of the tensors decides the arithmetic (float32 = the oracle proper,
float64 = the arbiter used for end-to-end error budgets).
"""
import math

import torch
import torch.nn.functional as F

GUARD = 1e-12  # the additive guard in every chord slope (Bounds.py:27)


def dual_exponent(p):
    """q with 1/p + 1/q = 1 (Bounds.py:277)."""
    if p == 1:
        return float("inf")
    return 1.0 / (1.0 - 1.0 / p)


class OBounds:
    def __init__(self, p, eps, lw, lb, uw, ub, words=1, ibp=False):
        self.p = float(p)
        self.q = dual_exponent(self.p)
        self.eps = eps
        self.words = words
        # interval mode (`--method ibp`): every operator takes its interval branch and the weight tensors are
        # cut down to `words` rows (Bounds.py:274, 285-288)
        self.ibp = ibp
        if ibp:
            lw, uw = lw[:, :, :words, :], uw[:, :, :words, :]
        self.lw, self.lb, self.uw, self.ub = lw, lb, uw, ub

    # ------------------------------------------------------------------ helpers
    def like(self, lw, lb, uw, ub):
        return OBounds(self.p, self.eps, lw, lb, uw, ub, self.words, self.ibp)

    def _box(self, lb, ub):
        """Result of an interval branch: constant bounds, zero weights."""
        return self.like(torch.zeros_like(self.lw), lb, torch.zeros_like(self.uw), ub)

    def _line(self, mask, k, x0, y0, lower):
        """One call of add_linear (Bounds.py:362-381): mask * (line of slope k through (x0, y0) applied to this bound),
        for the lower (lower=True) or upper output; a positive slope keeps the side, any other swaps it."""
        dt = k.dtype
        own_w, own_b, oth_w, oth_b = (self.lw, self.lb, self.uw, self.ub) if lower else (self.uw, self.ub, self.lw, self.lb)
        kp = (k > 0).to(dt)
        w = mask.unsqueeze(2) * kp.unsqueeze(2) * own_w * k.unsqueeze(2)
        b = mask * kp * ((own_b - x0) * k + y0)
        w = w + mask.unsqueeze(2) * (1 - kp).unsqueeze(2) * oth_w * k.unsqueeze(2)
        b = b + mask * (1 - kp) * ((oth_b - x0) * k + y0)
        return w, b

    @property
    def shape(self):
        return tuple(self.lw.shape)

    def clone(self):
        return self.like(self.lw.clone(), self.lb.clone(), self.uw.clone(), self.ub.clone())

    def t(self):
        """Swap the position axis with the feature axis (Bounds.py:335-346)."""
        return self.like(self.lw.transpose(1, 3), self.lb.transpose(1, 2),
                         self.uw.transpose(1, 3), self.ub.transpose(1, 2))

    # ------------------------------------------------------------ concretize
    def concretize(self):
        """l = lb - eps * sum_w ||lw_w||_q ; u = ub + eps * sum_w ||uw_w||_q, the norm taken
        over the dim_in axis per perturbed-word block (Bounds.py:311-326)."""
        di = self.lw.shape[-2]
        blk = di // self.words
        l = self.lb.clone()
        u = self.ub.clone()
        for w in range(self.words):
            sl = slice(blk * w, blk * (w + 1))
            l += -self.eps * torch.norm(self.lw[:, :, sl, :], p=self.q, dim=-2)
            u += self.eps * torch.norm(self.uw[:, :, sl, :], p=self.q, dim=-2)
        return l, u

    # ------------------------------------------------- affine (exact) operators
    def add(self, other):
        """Bounds + Bounds, or Bounds + constant on the bias terms (Bounds.py:383-395)."""
        if isinstance(other, OBounds):
            return self.like(self.lw + other.lw, self.lb + other.lb,
                             self.uw + other.uw, self.ub + other.ub)
        return self.like(self.lw, self.lb + other, self.uw, self.ub + other)

    def scale(self, c):
        """Multiplication by a python float (Bounds.py:594-607)."""
        if c > 0:
            return self.like(self.lw * c, self.lb * c, self.uw * c, self.ub * c)
        return self.like(self.uw * c, self.ub * c, self.lw * c, self.lb * c)

    def mul_tensor(self, w):
        """Elementwise product with a constant tensor broadcast over the last axis, split by
        the sign of the constant (Bounds.py:653-664)."""
        wp = w * (w > 0).to(w.dtype)
        wn = w - wp
        return self.like(self.lw * wp + self.uw * wn, self.lb * wp + self.ub * wn,
                         self.lw * wn + self.uw * wp, self.lb * wn + self.ub * wp)

    def matmul(self, weight):
        """Product with a constant weight [Dy, Do] (nn.Linear layout): positive weights keep
        the side of a bound, negative weights swap it (Bounds.py:397-413)."""
        w = weight.t()
        wp = w * (w > 0).to(w.dtype)
        wn = w - wp
        return self.like(self.lw.matmul(wp) + self.uw.matmul(wn),
                         self.lb.matmul(wp) + self.ub.matmul(wn),
                         self.lw.matmul(wn) + self.uw.matmul(wp),
                         self.lb.matmul(wn) + self.ub.matmul(wp))

    def dense(self, weight, bias):
        """matmul followed by the bias on lb/ub (Bounds.py:1016-1025)."""
        return self.matmul(weight).add(bias)

    # ---------------------------------------------- one-input relaxations
    def _rescale(self, kl, l_from_upper, new_lb, ku, u_from_lower, new_ub):
        """Column rescale shared by every relaxation: each output line is a per-column slope
        times one of the two input lines (which one follows the sign rule of add_linear,
        Bounds.py:362-381)."""
        src_l = torch.where(l_from_upper.unsqueeze(2), self.uw, self.lw)
        src_u = torch.where(u_from_lower.unsqueeze(2), self.lw, self.uw)
        return self.like(src_l * kl.unsqueeze(2), new_lb, src_u * ku.unsqueeze(2), new_ub)

    def relu(self):
        """Bounds.py:921-963.  Columns with l > 0 pass through, columns with u < 0 become zero,
        crossing columns get the chord through (l, 0) above and slope [|u| > |l|] below."""
        l, u = self.concretize()
        dt = l.dtype
        if self.ibp:  # Bounds.py:924-926
            return self._box(torch.clamp(l, min=0), torch.clamp(u, min=0))
        pos = (l > 0).to(dt)
        neg = (u < 0).to(dt)
        both = 1 - pos - neg
        k_up = u / (u - l + GUARD)
        k_lo = (u.abs() > l.abs()).to(dt)
        up_pos = (k_up > 0).to(dt)
        lo_pos = (k_lo > 0).to(dt)
        # pos columns: slope 1 on own line; crossing columns: the two slopes above.
        lw = pos.unsqueeze(2) * self.lw + both.unsqueeze(2) * (
            lo_pos.unsqueeze(2) * self.lw * k_lo.unsqueeze(2)
            + (1 - lo_pos).unsqueeze(2) * self.uw * k_lo.unsqueeze(2))
        lb = pos * self.lb + both * (lo_pos * (self.lb * k_lo) + (1 - lo_pos) * (self.ub * k_lo))
        uw = pos.unsqueeze(2) * self.uw + both.unsqueeze(2) * (
            up_pos.unsqueeze(2) * self.uw * k_up.unsqueeze(2)
            + (1 - up_pos).unsqueeze(2) * self.lw * k_up.unsqueeze(2))
        ub = pos * self.ub + both * (up_pos * ((self.ub - l) * k_up) + (1 - up_pos) * ((self.lb - l) * k_up))
        return self.like(lw, lb, uw, ub)

    @staticmethod
    def _dtanh(x):
        return 1.0 / torch.cosh(x).pow(2)

    def tanh(self):
        """Bounds.py:1027-1103.  One-sided columns: tangent at the midpoint on the convex side,
        chord on the other.  Crossing columns: for each line, ten bisection steps for the
        point whose tangent passes through the far end point."""
        l, u = self.concretize()
        dt = l.dtype
        if self.ibp:  # Bounds.py:1030-1032
            return self._box(torch.tanh(l), torch.tanh(u))
        pos = (l > 0).to(dt)
        neg = (u < 0).to(dt)
        both = 1 - pos - neg
        th, dth = torch.tanh, self._dtanh

        m = (l + u) / 2
        k_tan = dth(m)
        y_tan = th(m)
        k_chd = (th(u) - th(l)) / (u - l + GUARD)
        y_chd = th(l)

        # crossing, lower line: tangent point d in [l, 0] seen from u
        d = l / 2
        lo, hi = l, torch.zeros_like(l)
        for _ in range(10):
            v = (th(u) - th(d)) / (u - d + GUARD) - dth(d)
            gp = (v > 0).to(dt)
            lo = d * gp + lo * (1 - gp)
            hi = d * (1 - gp) + hi * gp
            d = (d + hi) / 2 * gp + (d + lo) / 2 * (1 - gp)
        d_lo = d
        k_blo = (th(d) - th(u)) / (d - u + GUARD)
        # crossing, upper line: tangent point d in [0, u] seen from l
        d = u / 2
        lo, hi = torch.zeros_like(l), u
        for _ in range(10):
            v = (th(d) - th(l)) / (d - l + GUARD) - dth(d)
            gp = (v > 0).to(dt)
            lo = d * (1 - gp) + lo * gp
            hi = d * gp + hi * (1 - gp)
            d = (d + hi) / 2 * (1 - gp) + (d + lo) / 2 * gp
        d_up = d
        k_bup = (th(d) - th(l)) / (d - l + GUARD)

        def line(mask, k, x0, y0, own_w, own_b, oth_w, oth_b):
            kp = (k > 0).to(dt)
            w = mask.unsqueeze(2) * (kp.unsqueeze(2) * own_w * k.unsqueeze(2)
                                     + (1 - kp).unsqueeze(2) * oth_w * k.unsqueeze(2))
            b = mask * (kp * ((own_b - x0) * k + y0) + (1 - kp) * ((oth_b - x0) * k + y0))
            return w, b

        lo_args = (self.lw, self.lb, self.uw, self.ub)
        up_args = (self.uw, self.ub, self.lw, self.lb)
        w1, b1 = line(neg, k_tan, m, y_tan, *lo_args)
        w2, b2 = line(pos, k_chd, l, y_chd, *lo_args)
        w3, b3 = line(both, k_blo, d_lo, th(d_lo), *lo_args)
        lw, lb = w1 + w2 + w3, b1 + b2 + b3
        w1, b1 = line(pos, k_tan, m, y_tan, *up_args)
        w2, b2 = line(neg, k_chd, l, y_chd, *up_args)
        w3, b3 = line(both, k_bup, d_up, th(d_up), *up_args)
        uw, ub = w1 + w2 + w3, b1 + b2 + b3
        return self.like(lw, lb, uw, ub)

    def exp(self):
        """Bounds.py:970-1003.  Lower: tangent at min(midpoint, l + 0.99) (keeps the bound
        positive); upper: chord.  Above 12 the exponential is continued linearly."""
        l, u = self.concretize()
        dt = l.dtype
        if self.ibp:  # Bounds.py:973-975
            return self._box(torch.exp(l), torch.exp(u))
        thres = torch.tensor(12.0, dtype=dt)

        def exp_capped(x):
            below = (x < thres).to(dt)
            return below * torch.exp(torch.min(x, thres)) + (1 - below) * (torch.exp(thres) * (x - thres + 1))

        m = torch.min((l + u) / 2, l + 0.99)
        kl = torch.exp(torch.min(m, thres))
        ku = (exp_capped(u) - exp_capped(l)) / (u - l + GUARD)
        return self.like(self.lw * kl.unsqueeze(2), kl * (self.lb - m + 1),
                         self.uw * ku.unsqueeze(2), self.ub * ku - ku * l + exp_capped(l))

    def reciprocal(self):
        """Bounds.py:1136-1161.  Input must be positive.  Lower: tangent at the midpoint;
        upper: chord.  Both slopes are negative, so each output line uses the opposite input."""
        l, u = self.concretize()
        if self.ibp:  # Bounds.py:1139-1143 (no positivity check in this branch)
            return self._box(1.0 / u, 1.0 / l)
        if not bool(torch.min(l) >= GUARD):
            raise AssertionError("reciprocal of a bound that is not strictly positive")
        m = (l + u) / 2
        kl = -1 / m.pow(2)
        ku = -1.0 / (l * u)
        return self.like(self.uw * kl.unsqueeze(2), self.ub * kl + 2 / m,
                         self.lw * ku.unsqueeze(2), self.lb * ku - ku * l + 1 / l)

    def sqr(self):
        """Bounds.py:860-890.  Upper: the chord; lower: a tangent placed so that it never goes negative on the
        range (one-sided columns), zero for columns whose range crosses zero."""
        l, u = self.concretize()
        dt = l.dtype
        pos = (l > 0).to(dt)
        neg = (u < 0).to(dt)
        both = 1 - pos - neg
        if self.ibp:
            lo = torch.min(l * l, u * u)
            return self._box(lo - both * lo, torch.max(l * l, u * u))
        one = torch.ones_like(l)
        uw, ub = self._line(one, u + l, l, l.pow(2), lower=False)
        m = torch.max((l + u) / 2, 2 * u)
        w1, b1 = self._line(neg, 2 * m, m, m.pow(2), lower=True)
        m = torch.min((l + u) / 2, 2 * l)
        w2, b2 = self._line(pos, 2 * m, m, m.pow(2), lower=True)
        return self.like(w1 + w2, b1 + b2, uw, ub)

    def sqrt(self):
        """Bounds.py:892-919.  Input must be positive.  Lower: the chord; upper: the tangent at the midpoint."""
        l, u = self.concretize()
        if not bool(torch.min(l) > 0):
            raise AssertionError("square root of a bound that is not strictly positive")
        if self.ibp:
            return self._box(torch.sqrt(l), torch.sqrt(u))
        one = torch.ones_like(l)
        k = (torch.sqrt(u) - torch.sqrt(l)) / (u - l + GUARD)
        lw, lb = self._line(one, k, l, torch.sqrt(l), lower=True)
        m = (l + u) / 2
        uw, ub = self._line(one, 0.5 / torch.sqrt(m), m, torch.sqrt(m), lower=False)
        return self.like(lw, lb, uw, ub)

    # --------------------------------------------------- two-input relaxations
    def mul_bounds(self, other):
        """Elementwise product of two bounded quantities, McCormick planes through
        (l_x, l_y) below and (l_x, u_y) above (Bounds.py:608-651, 680-688)."""
        if self.ibp:  # get_bounds_xy in interval mode: the planes are the constants min / max of the corner products
            la, ua = self.concretize()
            lo, uo = other.concretize()
            p1, p2, p3, p4 = la * lo, la * uo, ua * lo, ua * uo
            return self._box(torch.min(p1, torch.min(p2, torch.min(p3, p4))), torch.max(p1, torch.max(p2, torch.max(p3, p4))))
        la, _ = self.concretize()
        lo, uo = other.concretize()
        dt = la.dtype

        def side(alpha, beta, gamma, s_w, s_b, s_wx, s_bx, o_w, o_b, o_wx, o_bx):
            ap = (alpha > 0).to(dt)
            bp = (beta > 0).to(dt)
            w = ap.unsqueeze(2) * s_w * alpha.unsqueeze(2) + (1 - ap).unsqueeze(2) * s_wx * alpha.unsqueeze(2)
            b = ap * (s_b * alpha + gamma) + (1 - ap) * (s_bx * alpha + gamma)
            w = w + bp.unsqueeze(2) * o_w * beta.unsqueeze(2)
            b = b + bp * (o_b * beta)
            w = w + (1 - bp).unsqueeze(2) * o_wx * beta.unsqueeze(2)
            b = b + (1 - bp) * (o_bx * beta)
            return w, b

        lw, lb = side(lo, la, -lo * la, self.lw, self.lb, self.uw, self.ub,
                      other.lw, other.lb, other.uw, other.ub)
        uw, ub = side(uo, la, -uo * la, self.uw, self.ub, self.lw, self.lb,
                      other.uw, other.ub, other.lw, other.lb)
        return self.like(lw, lb, uw, ub)

    def divide(self, other):
        return self.mul_bounds(other.reciprocal())  # Bounds.py:825-830

    def softmax(self):
        """exp, row sum (an exact linear op on all four tensors), divide (Bounds.py:1005-1014)."""
        e = self.exp()
        do = self.lw.shape[-1]
        s = self.like(e.lw.sum(-1, keepdim=True).repeat(1, 1, 1, do),
                      e.lb.sum(-1, keepdim=True).repeat(1, 1, do),
                      e.uw.sum(-1, keepdim=True).repeat(1, 1, 1, do),
                      e.ub.sum(-1, keepdim=True).repeat(1, 1, do))
        return e.divide(s)

    def dot_product(self, other):
        """z[b,i,j] = sum_k x[b,i,k] * y[b,j,k] for two bounded operands (attention scores;
        Bounds.py:710-823).  With (l_x, u_x), (l_y, u_y) the concretised ranges, the lower plane
        uses alpha = l_y, beta = l_x and the upper plane alpha = u_y, beta = l_x; each slope
        picks the operand line by its sign, and the constant -alpha*beta is summed over k."""
        B, Lx, Di, K = self.lw.shape
        Ly = other.lw.shape[1]
        if Di == 1 or self.ibp:
            # interval product, no symbolic part (Bounds.py:711-721).  In interval mode with two perturbed words the
            # reference takes its general path, whose planes are then the same constants (alpha = beta = 0,
            # gamma = min / max of the corner products, :667-678) and whose ranges equal lb, ub (zero weights).
            l1, u1 = self.lb.unsqueeze(-2), self.ub.unsqueeze(-2)
            l2, u2 = other.lb.unsqueeze(1), other.ub.unsqueeze(1)
            p1, p2, p3, p4 = l1 * l2, l1 * u2, u1 * l2, u1 * u2
            lo = torch.min(torch.min(p1, p2), torch.min(p3, p4)).sum(-1)
            hi = torch.max(torch.max(p1, p2), torch.max(p3, p4)).sum(-1)
            w = (lo.unsqueeze(-2) * 0).expand(B, Lx, Di, Ly).clone()
            return self.like(w, lo, w.clone(), hi)
        lx, _ = self.concretize()
        ly, uy = other.concretize()
        dt = lx.dtype

        def pn(v):
            return v * (v > 0).to(dt), v * (v < 0).to(dt)

        lxp, lxn = pn(lx)   # [B, Lx, K]
        lyp, lyn = pn(ly)   # [B, Ly, K]
        uyp, uyn = pn(uy)

        def w_alpha(xw, a):   # [B,Lx,Di,K] x [B,Ly,K] -> [B,Lx,Di,Ly]
            return torch.matmul(xw, a.transpose(1, 2).unsqueeze(1))

        def w_beta(yw, bta):  # [B,Ly,Di,K] x [B,Lx,K] -> [B,Ly,Di,Lx] -> [B,Lx,Di,Ly]
            return torch.matmul(yw, bta.transpose(1, 2).unsqueeze(1)).transpose(1, 3)

        def b_alpha(xb, a):   # [B,Lx,K] x [B,Ly,K] -> [B,Lx,Ly]
            return torch.matmul(xb, a.transpose(1, 2))

        def b_beta(yb, bta):  # [B,Ly,K] x [B,Lx,K] -> [B,Lx,Ly]
            return torch.matmul(yb, bta.transpose(1, 2)).transpose(1, 2)

        lw = w_alpha(self.lw, lyp)
        lw = lw + w_alpha(self.uw, lyn)
        lw = lw + w_beta(other.lw, lxp)
        lw = lw + w_beta(other.uw, lxn)
        uw = w_alpha(self.uw, uyp)
        uw = uw + w_alpha(self.lw, uyn)
        uw = uw + w_beta(other.uw, lxp)
        uw = uw + w_beta(other.lw, lxn)
        lb = (-(ly.unsqueeze(1)) * lx.unsqueeze(2)).sum(-1)
        lb = lb + b_alpha(self.lb, lyp)
        lb = lb + b_alpha(self.ub, lyn)
        lb = lb + b_beta(other.lb, lxp)
        lb = lb + b_beta(other.ub, lxn)
        ub = (-(uy.unsqueeze(1)) * lx.unsqueeze(2)).sum(-1)
        ub = ub + b_alpha(self.ub, uyp)
        ub = ub + b_alpha(self.lb, uyn)
        ub = ub + b_beta(other.ub, lxp)
        ub = ub + b_beta(other.lb, lxn)
        return self.like(lw, lb, uw, ub)

    def context(self, value):
        """probabilities x values: the same operator against the transposed value bounds
        (Bounds.py:843-850)."""
        return self.dot_product(value.t())

    # --------------------------------------------------------------- layer norm
    def layer_norm(self, gamma, beta, mode="no_var"):
        """Bounds.py:1111-1131: subtract the feature mean (the mean of the *other* line, because of the minus
        sign); mode "standard" divides by the root of the variance (mean of the relaxed squares plus 1e-12);
        scale by gamma, add beta."""
        if mode == "no":
            return self
        if mode not in ("no_var", "standard"):
            raise NotImplementedError("layer_norm mode %r" % (mode,))
        do = self.lw.shape[-1]
        avg = torch.ones((do, do), dtype=self.lw.dtype, device=self.lw.device) * (1.0 / do)
        centred = self.add(self.matmul(avg).scale(-1.0))
        if mode == "standard":
            variance = centred.sqr().matmul(avg)
            centred = centred.divide(variance.add(GUARD).sqrt())
        return centred.mul_tensor(gamma).add(beta)


# ----------------------------------------------------------------------- conv
def conv_bounds(x, weight, bias, stride, padding):
    """Bound of a 2-D convolution with constant weights.

    The reference has no Python implementation; this follows the split-sign rule of
    `matmul` (Bounds.py:403-412) with dim_in acting as the convolution's batch axis
    (HandTunedKernels/convolution_verification.cu:228-238).  x.lw, x.uw : [B, Di, C, H, W];
    x.lb, x.ub : [B, C, H, W]; weight [Cout, C, kh, kw]; bias [Cout] or None.
    """
    wp = weight * (weight > 0).to(weight.dtype)
    wn = weight - wp
    B, Di, C, H, W = x.lw.shape

    def cv(t, w):
        return F.conv2d(t, w, None, stride, padding)

    lwf, uwf = x.lw.reshape(B * Di, C, H, W), x.uw.reshape(B * Di, C, H, W)
    lw = cv(lwf, wp) + cv(uwf, wn)
    uw = cv(lwf, wn) + cv(uwf, wp)
    lb = cv(x.lb, wp) + cv(x.ub, wn)
    ub = cv(x.lb, wn) + cv(x.ub, wp)
    if bias is not None:
        lb = lb + bias.view(1, -1, 1, 1)
        ub = ub + bias.view(1, -1, 1, 1)
    co, ho, wo = lw.shape[1:]
    return x.like(lw.reshape(B, Di, co, ho, wo), lb, uw.reshape(B, Di, co, ho, wo), ub)


def conv_as_tokens(x):
    """View conv-layout bounds [B, Di, C, H, W] / [B, C, H, W] as the [B, 1, Di, C*H*W] /
    [B, 1, C*H*W] token layout so that the column relaxations and `matmul` apply."""
    B, Di = x.lw.shape[:2]
    return x.like(x.lw.reshape(B, 1, Di, -1), x.lb.reshape(B, 1, -1),
                  x.uw.reshape(B, 1, Di, -1), x.ub.reshape(B, 1, -1))


def tokens_as_conv(x, c, h, w):
    B, _, Di, _ = x.lw.shape
    return x.like(x.lw.reshape(B, Di, c, h, w), x.lb.reshape(B, c, h, w),
                  x.uw.reshape(B, Di, c, h, w), x.ub.reshape(B, c, h, w))


# ------------------------------------------------------ encoder forward pass
def split_heads(x, heads):
    """[B, L, Di, H*d] -> [B*H, L, Di, d] (VerifierForward.py:208-229)."""
    B, L, Di, D = x.lw.shape
    d = D // heads

    def w(t):
        return t.reshape(B, L, Di, heads, d).permute(0, 3, 1, 2, 4).reshape(B * heads, L, Di, d)

    def b(t):
        return t.reshape(B, L, heads, d).permute(0, 2, 1, 3).reshape(B * heads, L, d)

    return x.like(w(x.lw), b(x.lb), w(x.uw), b(x.ub))


def merge_heads(x, heads):
    """[B*H, L, Di, d] -> [B, L, Di, H*d] (VerifierForward.py:253-265, generalised from one
    sentence to B sentences)."""
    BH, L, Di, d = x.lw.shape
    B = BH // heads

    def w(t):
        return t.reshape(B, heads, L, Di, d).permute(0, 2, 3, 1, 4).reshape(B, L, Di, heads * d)

    def b(t):
        return t.reshape(B, heads, L, d).permute(0, 2, 1, 3).reshape(B, L, heads * d)

    return x.like(w(x.lw), b(x.lb), w(x.uw), b(x.ub))


def input_bounds(emb, positions, p, eps, ibp=False):
    """Bounds of the embedding output: identity dependence on the perturbed word(s), or in interval mode the box
    of radius eps around the perturbed rows with zero weights (VerifierForward.py:127-152).
    emb [B, L, D]; positions: list of token indices."""
    B, L, D = emb.shape
    words = len(positions)
    lw = torch.zeros(B, L, D * words, D, dtype=emb.dtype)
    lb, ub = emb.clone(), emb.clone()
    for i, pos in enumerate(positions):
        if ibp:
            lb[:, pos] -= eps
            ub[:, pos] += eps
        else:
            lw[:, pos, D * i:D * (i + 1), :] = torch.eye(D, dtype=emb.dtype)
    return OBounds(p, eps, lw, lb, lw.clone(), ub, words, ibp)


def encoder_forward(model, emb, positions, p, eps, trace=None, ibp=False):
    """One forward bound pass of a BERT-style encoder (VerifierForward.py:93-119 without the
    `check` calls and the epsilon search).  `model` is a dict of tensors:

      emb_ln_g, emb_ln_b; per layer i: q_w,q_b,k_w,k_b,v_w,v_b,ao_w,ao_b,ln1_g,ln1_b,
      f1_w,f1_b,f2_w,f2_b,ln2_g,ln2_b (keys "layers"[i][name]); pool_w,pool_b; cls_w [2,D], cls_b [2];
      heads, layer_norm ("no_var" or "no").

    Returns (l, u): concretised bounds [B] of logit0 - logit1.  If `trace` is a list, the
    bounds after each stage are appended to it as (name, OBounds).
    """
    heads, ln = model["heads"], model["layer_norm"]

    def rec(name, b):
        if trace is not None:
            trace.append((name, b))
        return b

    x = input_bounds(emb, positions, p, eps, ibp).layer_norm(model["emb_ln_g"], model["emb_ln_b"], ln)
    rec("embedding", x)
    for i, ly in enumerate(model["layers"]):
        q = split_heads(x.dense(ly["q_w"], ly["q_b"]), heads)
        k = split_heads(x.dense(ly["k_w"], ly["k_b"]), heads)
        v = split_heads(x.dense(ly["v_w"], ly["v_b"]), heads)
        d = q.lw.shape[-1]
        scores = rec("layer%d.scores" % i, q.dot_product(k).scale(1.0 / math.sqrt(d)))
        probs = rec("layer%d.probs" % i, scores.softmax())
        ctx = merge_heads(probs.context(v), heads)
        att = ctx.dense(ly["ao_w"], ly["ao_b"]).add(x).layer_norm(ly["ln1_g"], ly["ln1_b"], ln)
        rec("layer%d.attention" % i, att)
        inter = rec("layer%d.intermediate" % i, att.dense(ly["f1_w"], ly["f1_b"]).relu())
        x = inter.dense(ly["f2_w"], ly["f2_b"]).add(att).layer_norm(ly["ln2_g"], ly["ln2_b"], ln)
        rec("layer%d.output" % i, x)
    if model.get("pooling", "first") == "mean":
        # mean over the positions (a fixed 1/L contraction, exact for linear bounds): the pooling the benchmark
        # description names; the reference itself pools the first token (VerifierForward.py:269-287)
        first = x.like(x.lw.mean(1, keepdim=True), x.lb.mean(1, keepdim=True), x.uw.mean(1, keepdim=True),
                       x.ub.mean(1, keepdim=True))
    else:
        first = x.like(x.lw[:, :1], x.lb[:, :1], x.uw[:, :1], x.ub[:, :1])
    pooled = rec("pooled", first.dense(model["pool_w"], model["pool_b"]).tanh())
    cw = (model["cls_w"][0] - model["cls_w"][1]).unsqueeze(0)
    cb = (model["cls_b"][0] - model["cls_b"][1]).unsqueeze(0)
    logit = rec("logit", pooled.dense(cw, cb))
    l, u = logit.concretize()
    return l[:, 0, 0], u[:, 0, 0]


def concrete_forward(model, emb):
    """Plain forward pass of the same encoder on concrete embeddings [N, L, D]; returns
    logit0 - logit1 [N].  Used for sampled containment checks."""
    heads, ln = model["heads"], model["layer_norm"]

    def norm(t, g, b):
        if ln == "no":
            return t
        c = t - t.mean(-1, keepdim=True)
        if ln == "standard":
            c = c / torch.sqrt((c * c).mean(-1, keepdim=True) + GUARD)
        return c * g + b

    x = norm(emb, model["emb_ln_g"], model["emb_ln_b"])
    N, L, D = x.shape
    d = D // heads
    for ly in model["layers"]:
        def sh(t):
            return t.reshape(N, L, heads, d).permute(0, 2, 1, 3)
        q = sh(F.linear(x, ly["q_w"], ly["q_b"]))
        k = sh(F.linear(x, ly["k_w"], ly["k_b"]))
        v = sh(F.linear(x, ly["v_w"], ly["v_b"]))
        pr = torch.softmax(q.matmul(k.transpose(-1, -2)) / math.sqrt(d), dim=-1)
        ctx = pr.matmul(v).permute(0, 2, 1, 3).reshape(N, L, D)
        att = norm(F.linear(ctx, ly["ao_w"], ly["ao_b"]) + x, ly["ln1_g"], ly["ln1_b"])
        inter = torch.relu(F.linear(att, ly["f1_w"], ly["f1_b"]))
        x = norm(F.linear(inter, ly["f2_w"], ly["f2_b"]) + att, ly["ln2_g"], ly["ln2_b"])
    tok = x.mean(1) if model.get("pooling", "first") == "mean" else x[:, 0]
    pooled = torch.tanh(F.linear(tok, model["pool_w"], model["pool_b"]))
    logits = F.linear(pooled, model["cls_w"], model["cls_b"])
    return logits[:, 0] - logits[:, 1]


def make_encoder(seed, layers=3, d_model=128, heads=4, ffn=512, std=0.02, dtype=torch.float32,
                 layer_norm="no_var"):
    """Random-initialised encoder weights (normal, std `std`; layer-norm gain 1, shift 0)."""
    g = torch.Generator().manual_seed(seed)

    def rn(*shape):
        return (torch.randn(*shape, generator=g) * std).to(dtype)

    def lin(o, i):
        return rn(o, i), rn(o)

    m = {"heads": heads, "layer_norm": layer_norm,
         "emb_ln_g": torch.ones(d_model, dtype=dtype), "emb_ln_b": torch.zeros(d_model, dtype=dtype),
         "layers": []}
    for _ in range(layers):
        ly = {}
        for nm, (o, i) in (("q", (d_model, d_model)), ("k", (d_model, d_model)), ("v", (d_model, d_model)),
                           ("ao", (d_model, d_model)), ("f1", (ffn, d_model)), ("f2", (d_model, ffn))):
            ly[nm + "_w"], ly[nm + "_b"] = lin(o, i)
        for nm in ("ln1", "ln2"):
            ly[nm + "_g"] = torch.ones(d_model, dtype=dtype)
            ly[nm + "_b"] = torch.zeros(d_model, dtype=dtype)
        m["layers"].append(ly)
    m["pool_w"], m["pool_b"] = lin(d_model, d_model)
    m["cls_w"], m["cls_b"] = lin(2, d_model)
    return m


def model_to(model, dtype):
    """Copy of an encoder dict with every tensor cast to `dtype`."""
    def cv(v):
        if isinstance(v, torch.Tensor):
            return v.to(dtype)
        if isinstance(v, list):
            return [cv(e) for e in v]
        if isinstance(v, dict):
            return {k: cv(e) for k, e in v.items()}
        return v
    return cv(model)


# ------------------------------------------------------------------ small CNN
def cnn_forward(layers, image, p, eps):
    """Forward bound pass of a CNN on one image with every pixel perturbed (dim_in = C*H*W):
    layers is a list of ("conv", weight, bias, stride, pad) / ("relu",) / ("linear", W, b).
    Conv bounds follow `conv_bounds`; relu and linear are the pinned `Bounds` operators on the
    flattened [1, 1, Di, C*H*W] view.  Returns the concretised (l, u) of the outputs."""
    C, H, W = image.shape
    di = C * H * W
    lw = torch.eye(di, dtype=image.dtype).view(1, di, C, H, W)
    x = OBounds(p, eps, lw, image.view(1, C, H, W).clone(), lw.clone(), image.view(1, C, H, W).clone())
    for ly in layers:
        if ly[0] == "conv":
            x = conv_bounds(x, ly[1], ly[2], ly[3], ly[4])
        elif ly[0] == "relu":
            if x.lw.dim() == 5:
                c, h, w = x.lw.shape[2:]
                x = tokens_as_conv(conv_as_tokens(x).relu(), c, h, w)
            else:
                x = x.relu()
        elif ly[0] == "linear":
            if x.lw.dim() == 5:
                x = conv_as_tokens(x)
            x = x.dense(ly[1], ly[2])
    if x.lw.dim() == 5:
        x = conv_as_tokens(x)
    l, u = x.concretize()
    return l.reshape(-1), u.reshape(-1)


def make_cnn(seed, c_in=3, hw=32, dtype=torch.float32):
    """conv 3->16 (3x3, s1, p1), relu, conv 16->32 (3x3, s2, p1), relu, linear -> 10; Kaiming-normal
    weights, zero biases."""
    g = torch.Generator().manual_seed(seed)

    def kaiming(*shape):
        fan_in = 1
        for d in shape[1:]:
            fan_in *= d
        return (torch.randn(*shape, generator=g) * math.sqrt(2.0 / fan_in)).to(dtype)

    ho = (hw + 2 - 3) // 2 + 1
    return [("conv", kaiming(16, c_in, 3, 3), torch.zeros(16, dtype=dtype), 1, 1), ("relu",),
            ("conv", kaiming(32, 16, 3, 3), torch.zeros(32, dtype=dtype), 2, 1), ("relu",),
            ("linear", kaiming(10, 32 * ho * ho), torch.zeros(10, dtype=dtype))]


def epsilon_search(model, emb_one, label, p, max_eps, iters, positions=None):
    """Largest certified radius per perturbed position of one sentence (emb_one [1, L, D]): the reference's loop,
    Verifier.verify (Verifiers/Verifier.py:106-147, one perturbed word): a probe at max_eps whose answer is not
    used, then `iters` bisection steps on [0, max_eps] in Python floats; a probe certifies when the concretised
    logit0 - logit1 keeps the sign of the label (VerifierForward.py:306-312).  Returns {position: eps}."""
    L = emb_one.shape[1]
    out = {}
    for i in (positions if positions is not None else range(1, L - 1)):
        def safe(eps):
            l, u = encoder_forward(model, emb_one, [i], p, eps)
            return bool(l[0] > 0) if label == 0 else bool(u[0] < 0)
        lo, hi = 0.0, float(max_eps)
        safe(hi)
        for _ in range(iters):
            m = (lo + hi) / 2
            if safe(m):
                lo = m
            else:
                hi = m
        out[int(i)] = lo
    return out


def epsilon_search_pairs(model, emb_one, label, p, max_eps, iters, pairs=None, warm_up=True):
    """The same search with two perturbed words (Verifiers/Verifier.py:149-201): warm max_eps up on the pair (1, 2)
    (halve until certified, double until not), then per pair of positions double the radius while certified, or halve it
    until certified, and bisect `iters` times from there.  Returns ({(i1, i2): eps}, max_eps after the warm-up)."""
    L = emb_one.shape[1]

    def safe(pos, eps):
        try:
            l, u = encoder_forward(model, emb_one, list(pos), p, eps)
        except AssertionError:   # a failed assertion inside the pass counts as "not certified" (VerifierForward.py:120-125)
            return False
        return bool(l[0] > 0) if label == 0 else bool(u[0] < 0)

    max_eps = float(max_eps)
    if warm_up:
        while not safe((1, 2), max_eps):
            max_eps /= 2
        while safe((1, 2), max_eps):
            max_eps *= 2
    if pairs is None:
        pairs = [(a, b) for a in range(1, L - 1) for b in range(a + 1, L - 1)]
    out = {}
    for pr in pairs:
        lo, hi = 0.0, max_eps
        ok = safe(pr, hi)
        while ok:
            lo = hi
            hi *= 2
            ok = safe(pr, hi)
        if lo == 0:
            while not ok:
                hi /= 2
                ok = safe(pr, hi)
            lo, hi = hi, hi * 2
        for _ in range(iters):
            m = (lo + hi) / 2
            if safe(pr, m):
                lo = m
            else:
                hi = m
        out[tuple(pr)] = lo
    return out, max_eps
