"""Thin tensor-level wrappers over the C ABI: argument checks, output allocation, stream.

PyTorch is used only for device memory and the current stream; all arithmetic happens in
libfaith_b200.so.  Every tensor must be a contiguous float32 CUDA tensor.
"""
import math

import torch

from . import _lib
from ._lib import (FB_EXP, FB_NATIVE, FB_P1, FB_P2, FB_PINF, FB_RECIPROCAL, FB_RELU, FB_TANH, FB_TRANSPOSED,
                   check, load)


def norm_code(p):
    """Maps the perturbation norm p to the C enum (the dual exponent is implied)."""
    if p == 1:
        return FB_P1
    if p == 2:
        return FB_P2
    if p == float("inf") or p >= 10:  # the reference treats p >= 10 as infinity (Verifier.py:17)
        return FB_PINF
    raise ValueError("only p in {1, 2, inf} is supported, got %r" % (p,))


def _chk(*tensors):
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise _lib.FaithError("faith_b200 operators need CUDA tensors (there is no CPU path)")
        if t.dtype != torch.float32:
            raise _lib.FaithError("float32 tensors required, got %s" % t.dtype)
        if not t.is_contiguous():
            raise _lib.FaithError("contiguous tensors required")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise _lib.FaithError("all tensors must live on one device")
    return dev


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _p(t):
    return None if t is None else t.data_ptr()


def concretize(lw, uw, lb, ub, p, eps, words=1, layout=FB_NATIVE):
    dev = _chk(lw, uw, lb, ub)
    rows = lb.numel() // lb.shape[-1]
    Do = lb.shape[-1]
    Di = lw.shape[-2] if layout == FB_NATIVE else lw.shape[-1]
    l, u = torch.empty_like(lb), torch.empty_like(ub)
    with torch.cuda.device(dev):
        check(load().fb_concretize_f32(_p(lw), _p(uw), _p(lb), _p(ub), _p(l), _p(u), rows, Di, Do, words,
                                       norm_code(p), eps, layout, _stream()), "fb_concretize_f32")
    return l, u


def relax(op, lw, uw, lb, ub, p, eps, words=1, layout=FB_NATIVE, out=None, violation=None):
    dev = _chk(lw, uw, lb, ub)
    rows = lb.numel() // lb.shape[-1]
    Do = lb.shape[-1]
    Di = lw.shape[-2] if layout == FB_NATIVE else lw.shape[-1]
    if out is None:
        out = (torch.empty_like(lw), torch.empty_like(uw), torch.empty_like(lb), torch.empty_like(ub))
    o_lw, o_uw, o_lb, o_ub = out
    _chk(o_lw, o_uw, o_lb, o_ub)
    if violation is not None and (violation.dtype != torch.int32 or not violation.is_cuda):
        raise _lib.FaithError("violation flag must be an int32 CUDA tensor")
    with torch.cuda.device(dev):
        check(load().fb_relax_f32(op, _p(lw), _p(uw), _p(lb), _p(ub), _p(o_lw), _p(o_uw), _p(o_lb), _p(o_ub),
                                  rows, Di, Do, words, norm_code(p), eps, layout, _p(violation), _stream()),
              "fb_relax_f32")
    return o_lw, o_uw, o_lb, o_ub


def matmul(lw, uw, lb, ub, W, bias=None):
    dev = _chk(lw, uw, lb, ub, W, bias)
    rows = lb.numel() // lb.shape[-1]
    Di, Do = lw.shape[-2], lw.shape[-1]
    Dy = W.shape[0]
    if W.shape[1] != Do:
        raise _lib.FaithError("weight shape %s does not match feature size %d" % (tuple(W.shape), Do))
    y_lw = torch.empty(lw.shape[:-1] + (Dy,), device=dev, dtype=torch.float32)
    y_uw = torch.empty_like(y_lw)
    y_lb = torch.empty(lb.shape[:-1] + (Dy,), device=dev, dtype=torch.float32)
    y_ub = torch.empty_like(y_lb)
    with torch.cuda.device(dev):
        check(load().fb_matmul_f32(_p(lw), _p(uw), _p(lb), _p(ub), _p(W), _p(bias), _p(y_lw), _p(y_uw), _p(y_lb),
                                   _p(y_ub), rows, Di, Do, Dy, _stream()), "fb_matmul_f32")
    return y_lw, y_uw, y_lb, y_ub


def relax_coef(op, lw, uw, lb, ub, p, eps, words=1, violation=None):
    """Relaxation without the rescale pass: returns (c_l, c_u, out_lb, out_ub), all [rows..., Do]."""
    dev = _chk(lw, uw, lb, ub)
    rows = lb.numel() // lb.shape[-1]
    Di, Do = lw.shape[-2], lw.shape[-1]
    out = tuple(torch.empty_like(lb) for _ in range(4))
    with torch.cuda.device(dev):
        check(load().fb_relax_coef_f32(int(op), _p(lw), _p(uw), _p(lb), _p(ub), *[_p(t) for t in out], rows, Di, Do,
                                       int(words), norm_code(p), float(eps), _p(violation), _stream()), "fb_relax_coef_f32")
    return out


def matmul_residual(lw, uw, lb, ub, W, bias, residual, c_l=None, c_u=None):
    """matmul of (lw, uw, lb, ub) (or of (c_l * lw, c_u * uw, lb, ub)) with W, + bias, + residual (lw, uw, lb, ub)."""
    dev = _chk(lw, uw, lb, ub, W, bias, *residual)
    rows = lb.numel() // lb.shape[-1]
    Di, Do = lw.shape[-2], lw.shape[-1]
    Dy = W.shape[0]
    y_lw = torch.empty(lw.shape[:-1] + (Dy,), device=dev, dtype=torch.float32)
    y_uw = torch.empty_like(y_lw)
    y_lb = torch.empty(lb.shape[:-1] + (Dy,), device=dev, dtype=torch.float32)
    y_ub = torch.empty_like(y_lb)
    with torch.cuda.device(dev):
        check(load().fb_matmul_residual_f32(_p(lw), _p(uw), _p(lb), _p(ub), _p(c_l), _p(c_u), _p(W), _p(bias),
                                            *[_p(t) for t in residual], _p(y_lw), _p(y_uw), _p(y_lb), _p(y_ub), rows, Di, Do,
                                            Dy, _stream()), "fb_matmul_residual_f32")
    return y_lw, y_uw, y_lb, y_ub


def row_sums(lw, uw, lb, ub):
    """Row sums of a bound in the form fb_matmul_residual_ln_f32 reads: [2 lines, 4 partial sums, rows * (Di + 1)], the
    whole sum in the first partial sum (weight rows first, then the bias rows)."""
    D = lw.shape[-1]
    out = torch.zeros(2, 4, lw.numel() // D + lb.numel() // D, device=lw.device, dtype=torch.float32)
    out[0, 0] = torch.cat([lw.reshape(-1, D).sum(-1), lb.reshape(-1, D).sum(-1)])
    out[1, 0] = torch.cat([uw.reshape(-1, D).sum(-1), ub.reshape(-1, D).sum(-1)])
    return out


def matmul_residual_ln(lw, uw, lb, ub, W, bias, residual, residual_rowsum, gamma, beta, c_l=None, c_u=None):
    """layer_norm(matmul(x, W) + bias + residual), mode no_var, in one launch.  Returns (z_lw, z_uw, z_lb, z_ub,
    z_rowsum); residual_rowsum / z_rowsum as row_sums() lays them out."""
    dev = _chk(lw, uw, lb, ub, W, bias, *residual, residual_rowsum, gamma, beta)
    rows = lb.numel() // lb.shape[-1]
    Di, Do = lw.shape[-2], lw.shape[-1]
    Dy = W.shape[0]
    z_lw = torch.empty(lw.shape[:-1] + (Dy,), device=dev, dtype=torch.float32)
    z_uw = torch.empty_like(z_lw)
    z_lb = torch.empty(lb.shape[:-1] + (Dy,), device=dev, dtype=torch.float32)
    z_ub = torch.empty_like(z_lb)
    z_rs = torch.empty(2, 4, rows * (Di + 1), device=dev, dtype=torch.float32)
    with torch.cuda.device(dev):
        check(load().fb_matmul_residual_ln_f32(_p(lw), _p(uw), _p(lb), _p(ub), _p(c_l), _p(c_u), _p(W), _p(bias),
                                               *[_p(t) for t in residual], _p(residual_rowsum), _p(gamma), _p(beta),
                                               _p(z_lw), _p(z_uw), _p(z_lb), _p(z_ub), _p(z_rs), rows, Di, Do, Dy, _stream()),
              "fb_matmul_residual_ln_f32")
    return z_lw, z_uw, z_lb, z_ub, z_rs


def relax_coef_given(op, lb, ub, l, u, violation=None):
    """relax_coef for a bound whose concretised range (l, u) is already known: no pass over lw / uw."""
    dev = _chk(lb, ub, l, u)
    rows = lb.numel() // lb.shape[-1]
    out = tuple(torch.empty_like(lb) for _ in range(4))
    with torch.cuda.device(dev):
        check(load().fb_relax_coef_given_f32(int(op), _p(lb), _p(ub), _p(l), _p(u), *[_p(t) for t in out], rows,
                                             lb.shape[-1], _p(violation), _stream()), "fb_relax_coef_given_f32")
    return out


def matmul_coef(lw, uw, lb, ub, c_l, c_u, W, bias=None):
    """matmul of (c_l * lw, c_u * uw, lb, ub) with W (+ bias): the consumer side of relax_coef."""
    dev = _chk(lw, uw, lb, ub, c_l, c_u, W, bias)
    rows = lb.numel() // lb.shape[-1]
    Di, Do = lw.shape[-2], lw.shape[-1]
    Dy = W.shape[0]
    y_lw = torch.empty(lw.shape[:-1] + (Dy,), device=dev, dtype=torch.float32)
    y_uw = torch.empty_like(y_lw)
    y_lb = torch.empty(lb.shape[:-1] + (Dy,), device=dev, dtype=torch.float32)
    y_ub = torch.empty_like(y_lb)
    with torch.cuda.device(dev):
        check(load().fb_matmul_coef_f32(_p(lw), _p(uw), _p(lb), _p(ub), _p(c_l), _p(c_u), _p(W), _p(bias), _p(y_lw), _p(y_uw),
                                        _p(y_lb), _p(y_ub), rows, Di, Do, Dy, _stream()), "fb_matmul_coef_f32")
    return y_lw, y_uw, y_lb, y_ub


def matmul_heads_ranges(lw, uw, lb, ub, W, bias, heads, p, eps, words=1):
    """Projection with head-split store that also returns the concretised range of its result: lw, uw
    [S, L, Di, Do], lb, ub [S, L, Do] -> (y_lw, y_uw [S*heads, L, Di, d], y_lb, y_ub, y_l, y_u [S*heads, L, d]).
    Raises FaithError (FB_ERR_SHAPE) outside the tensor-core shapes with Di == 128 * words."""
    dev = _chk(lw, uw, lb, ub, W, bias)
    S, L, Di, Do = lw.shape
    Dy = W.shape[0]
    d = Dy // heads
    y_lw = torch.empty((S * heads, L, Di, d), device=dev, dtype=torch.float32)
    y_uw = torch.empty_like(y_lw)
    y_lb, y_ub, y_l, y_u = (torch.empty((S * heads, L, d), device=dev, dtype=torch.float32) for _ in range(4))
    ws = torch.empty(2 * S * L * (words + 1) * Dy, device=dev, dtype=torch.float32)
    with torch.cuda.device(dev):
        check(load().fb_matmul_heads_ranges_f32(_p(lw), _p(uw), _p(lb), _p(ub), _p(W), _p(bias), _p(y_lw), _p(y_uw), _p(y_lb),
                                                _p(y_ub), _p(y_l), _p(y_u), _p(ws), S * L, Di, Do, Dy, L, heads, int(words),
                                                norm_code(p), float(eps), _stream()), "fb_matmul_heads_ranges_f32")
    return y_lw, y_uw, y_lb, y_ub, y_l, y_u


def dot_product(x, y, p, eps, words=1, out_scale=1.0, layout=FB_NATIVE, scratch=None, out=None):
    """x, y: (lw, uw, lb, ub).  Returns (z_lw, z_uw, z_lb, z_ub)."""
    x_lw, x_uw, x_lb, x_ub = x
    y_lw, y_uw, y_lb, y_ub = y
    dev = _chk(*x, *y)
    B, Lx, K = x_lb.shape
    Ly = y_lb.shape[1]
    Di = x_lw.shape[2] if layout == FB_NATIVE else x_lw.shape[3]
    if out is None:
        zshape = (B, Lx, Di, Ly) if layout == FB_NATIVE else (B, Lx, Ly, Di)
        out = (torch.empty(zshape, device=dev), torch.empty(zshape, device=dev),
               torch.empty((B, Lx, Ly), device=dev), torch.empty((B, Lx, Ly), device=dev))
    if scratch is None:
        scratch = (torch.empty_like(x_lb), torch.empty_like(x_lb), torch.empty_like(y_lb), torch.empty_like(y_lb))
    x_l, x_u, y_l, y_u = scratch
    z_lw, z_uw, z_lb, z_ub = out
    _chk(*out, *scratch)
    with torch.cuda.device(dev):
        check(load().fb_dot_product_f32(_p(x_lw), _p(x_uw), _p(x_lb), _p(x_ub), _p(y_lw), _p(y_uw), _p(y_lb), _p(y_ub),
                                        _p(z_lw), _p(z_uw), _p(z_lb), _p(z_ub), _p(x_l), _p(x_u), _p(y_l), _p(y_u),
                                        B, Lx, Ly, Di, K, words, norm_code(p), eps, out_scale, layout, _stream()),
              "fb_dot_product_f32")
    return out


def context_kmajor(x, v, p, eps, words=1, out_scale=1.0, merge_heads=1):
    """Context product with the values in the projection's own layout: x (lw, uw [B, Lx, Di, K], lb, ub
    [B, Lx, K]), v (lw, uw [B, K, Di, Ly], lb, ub [B, K, Ly]).  Returns z as fb_dot_product_heads_f32 does.
    Raises FaithError (FB_ERR_SHAPE) outside the tensor-core shapes."""
    x_lw, x_uw, x_lb, x_ub = x
    v_lw, v_uw, v_lb, v_ub = v
    dev = _chk(*x, *v)
    B, Lx, K = x_lb.shape
    Ly = v_lb.shape[2]
    Di = x_lw.shape[2]
    S = B // merge_heads
    zw = (S, Lx, Di, merge_heads * Ly) if merge_heads > 1 else (B, Lx, Di, Ly)
    zb = (S, Lx, merge_heads * Ly) if merge_heads > 1 else (B, Lx, Ly)
    out = (torch.empty(zw, device=dev), torch.empty(zw, device=dev), torch.empty(zb, device=dev), torch.empty(zb, device=dev))
    scratch = (torch.empty_like(x_lb), torch.empty_like(x_lb), torch.empty((B, Ly, K), device=dev), torch.empty((B, Ly, K), device=dev))
    with torch.cuda.device(dev):
        check(load().fb_context_heads_f32(_p(x_lw), _p(x_uw), _p(x_lb), _p(x_ub), _p(v_lw), _p(v_uw), _p(v_lb), _p(v_ub),
                                          *[_p(t) for t in out], *[_p(t) for t in scratch], B, Lx, Ly, Di, K, words,
                                          norm_code(p), eps, out_scale, merge_heads, _stream()), "fb_context_heads_f32")
    return out


def mul_bounds(x, y, p, eps, words=1):
    dev = _chk(*x, *y)
    x_lw, x_uw, x_lb, x_ub = x
    rows = x_lb.numel() // x_lb.shape[-1]
    Di, Do = x_lw.shape[-2], x_lw.shape[-1]
    out = (torch.empty_like(x_lw), torch.empty_like(x_lw), torch.empty_like(x_lb), torch.empty_like(x_lb))
    with torch.cuda.device(dev):
        check(load().fb_mul_bounds_f32(*[_p(t) for t in x], *[_p(t) for t in y], *[_p(t) for t in out],
                                       rows, Di, Do, words, norm_code(p), eps, _stream()), "fb_mul_bounds_f32")
    return out


def add(x, y):
    dev = _chk(*x, *y)
    x_lw, x_uw, x_lb, x_ub = x
    rows = x_lb.numel() // x_lb.shape[-1]
    Di, Do = x_lw.shape[-2], x_lw.shape[-1]
    out = (torch.empty_like(x_lw), torch.empty_like(x_lw), torch.empty_like(x_lb), torch.empty_like(x_lb))
    with torch.cuda.device(dev):
        check(load().fb_add_f32(*[_p(t) for t in x], *[_p(t) for t in y], *[_p(t) for t in out], rows, Di, Do,
                                _stream()), "fb_add_f32")
    return out


def scale(x, c):
    dev = _chk(*x)
    x_lw, x_uw, x_lb, x_ub = x
    rows = x_lb.numel() // x_lb.shape[-1]
    Di, Do = x_lw.shape[-2], x_lw.shape[-1]
    out = (torch.empty_like(x_lw), torch.empty_like(x_lw), torch.empty_like(x_lb), torch.empty_like(x_lb))
    with torch.cuda.device(dev):
        check(load().fb_scale_f32(*[_p(t) for t in x], *[_p(t) for t in out], rows, Di, Do, float(c), _stream()),
              "fb_scale_f32")
    return out


def mul_features(x, w):
    """x * w with w a vector over the feature axis, split by sign (Bounds.py:653-664)."""
    dev = _chk(*x, w)
    lw, uw, lb, ub = x
    rows, Di, Do = lb.numel() // lb.shape[-1], lw.shape[-2], lw.shape[-1]
    if w.numel() != Do:
        raise _lib.FaithError("feature vector of %d elements against %d features" % (w.numel(), Do))
    z = tuple(torch.empty_like(t) for t in x)
    with torch.cuda.device(dev):
        check(load().fb_mul_features_f32(_p(lw), _p(uw), _p(lb), _p(ub), _p(w), _p(z[0]), _p(z[1]), _p(z[2]), _p(z[3]),
                                         rows, Di, Do, _stream()), "fb_mul_features_f32")
    return z


def interval_mul(xl, xu, yl, yu):
    """Elementwise product of two boxes (Bounds.py:667-678)."""
    dev = _chk(xl, xu, yl, yu)
    zl, zu = torch.empty_like(xl), torch.empty_like(xu)
    with torch.cuda.device(dev):
        check(load().fb_interval_mul_f32(_p(xl), _p(xu), _p(yl), _p(yu), _p(zl), _p(zu), xl.numel(), _stream()),
              "fb_interval_mul_f32")
    return zl, zu


def interval_dot(xl, xu, yl, yu):
    """z[b,i,j] = sum_k [x[b,i,k]] * [y[b,j,k]] for boxes x [B,Lx,K], y [B,Ly,K] (Bounds.py:711-721)."""
    dev = _chk(xl, xu, yl, yu)
    B, Lx, K = xl.shape
    Ly = yl.shape[1]
    if yl.shape[0] != B or yl.shape[2] != K:
        raise _lib.FaithError("interval_dot: shapes %s and %s do not match" % (tuple(xl.shape), tuple(yl.shape)))
    zl = torch.empty(B, Lx, Ly, device=dev, dtype=torch.float32)
    zu = torch.empty_like(zl)
    with torch.cuda.device(dev):
        check(load().fb_interval_dot_f32(_p(xl), _p(xu), _p(yl), _p(yu), _p(zl), _p(zu), B, Lx, Ly, K, _stream()),
              "fb_interval_dot_f32")
    return zl, zu


def rowsum(x):
    dev = _chk(*x)
    x_lw, x_uw, x_lb, x_ub = x
    rows = x_lb.numel() // x_lb.shape[-1]
    Di, Do = x_lw.shape[-2], x_lw.shape[-1]
    out = (torch.empty_like(x_lw), torch.empty_like(x_lw), torch.empty_like(x_lb), torch.empty_like(x_lb))
    with torch.cuda.device(dev):
        check(load().fb_rowsum_f32(*[_p(t) for t in x], *[_p(t) for t in out], rows, Di, Do, _stream()),
              "fb_rowsum_f32")
    return out


def layernorm_novar(x, gamma, beta, residual=None):
    dev = _chk(*x, gamma, beta, *(residual or ()))
    x_lw, x_uw, x_lb, x_ub = x
    rows = x_lb.numel() // x_lb.shape[-1]
    Di, Do = x_lw.shape[-2], x_lw.shape[-1]
    out = (torch.empty_like(x_lw), torch.empty_like(x_lw), torch.empty_like(x_lb), torch.empty_like(x_lb))
    r = [_p(t) for t in residual] if residual is not None else [None] * 4
    with torch.cuda.device(dev):
        check(load().fb_layernorm_novar_f32(*[_p(t) for t in x], *r, _p(gamma), _p(beta), *[_p(t) for t in out],
                                            rows, Di, Do, _stream()), "fb_layernorm_novar_f32")
    return out


def split_heads(x, heads, transpose_ld=False):
    """(lw, uw, lb, ub) [B, L, Di, H*d] -> [B*H, L, Di, d], or [B*H, d, Di, L] with transpose_ld."""
    dev = _chk(*x)
    lw, uw, lb, ub = x
    B, L, Di, D = lw.shape
    d = D // heads
    wshape = (B * heads, d, Di, L) if transpose_ld else (B * heads, L, Di, d)
    bshape = (B * heads, d, L) if transpose_ld else (B * heads, L, d)
    out = (torch.empty(wshape, device=dev), torch.empty(wshape, device=dev),
           torch.empty(bshape, device=dev), torch.empty(bshape, device=dev))
    with torch.cuda.device(dev):
        for w, b, ow, ob in ((lw, lb, out[0], out[2]), (uw, ub, out[1], out[3])):
            check(load().fb_split_heads_f32(_p(w), _p(b), _p(ow), _p(ob), B, L, Di, heads, d, int(transpose_ld),
                                            _stream()), "fb_split_heads_f32")
    return out


def merge_heads(x, heads):
    """(lw, uw, lb, ub) [B*H, L, Di, d] -> [B, L, Di, H*d]."""
    dev = _chk(*x)
    lw, uw, lb, ub = x
    BH, L, Di, d = lw.shape
    B = BH // heads
    out = (torch.empty((B, L, Di, heads * d), device=dev), torch.empty((B, L, Di, heads * d), device=dev),
           torch.empty((B, L, heads * d), device=dev), torch.empty((B, L, heads * d), device=dev))
    with torch.cuda.device(dev):
        for w, b, ow, ob in ((lw, lb, out[0], out[2]), (uw, ub, out[1], out[3])):
            check(load().fb_merge_heads_f32(_p(w), _p(b), _p(ow), _p(ob), B, L, Di, heads, d, _stream()),
                  "fb_merge_heads_f32")
    return out


def conv2d(x, weight, bias, stride, padding):
    """x: (lw, uw, lb, ub) with lw, uw [B, Di, C, H, W] and lb, ub [B, C, H, W]."""
    dev = _chk(*x, weight, bias)
    lw, uw, lb, ub = x
    B, Di, C, H, W = lw.shape
    Co, Ci, Kh, Kw = weight.shape
    if Ci != C:
        raise _lib.FaithError("conv weight expects %d input channels, bounds have %d" % (Ci, C))
    Ho = (H + 2 * padding - Kh) // stride + 1
    Wo = (W + 2 * padding - Kw) // stride + 1
    out = (torch.empty((B, Di, Co, Ho, Wo), device=dev), torch.empty((B, Di, Co, Ho, Wo), device=dev),
           torch.empty((B, Co, Ho, Wo), device=dev), torch.empty((B, Co, Ho, Wo), device=dev))
    with torch.cuda.device(dev):
        check(load().fb_conv2d_f32(*[_p(t) for t in x], _p(weight), _p(bias), *[_p(t) for t in out],
                                   B, Di, C, H, W, Co, Kh, Kw, stride, padding, _stream()), "fb_conv2d_f32")
    return out


def norm_partials(lw, uw, p):
    """Unfinished dual-norm accumulation of the local dim_in rows: (part_l, part_u), each [.., Do]."""
    dev = _chk(lw, uw)
    Di, Do = lw.shape[-2], lw.shape[-1]
    rows = lw.numel() // (Di * Do)
    shape = lw.shape[:-2] + (Do,)
    part_l, part_u = torch.empty(shape, device=dev), torch.empty(shape, device=dev)
    with torch.cuda.device(dev):
        check(load().fb_norm_partials_f32(_p(lw), _p(uw), _p(part_l), _p(part_u), rows, Di, Do, norm_code(p),
                                          _stream()), "fb_norm_partials_f32")
    return part_l, part_u


def relax_with_norms(op, lw, uw, lb, ub, norm_l, norm_u, p, eps, violation=None):
    dev = _chk(lw, uw, lb, ub, norm_l, norm_u)
    Di, Do = lw.shape[-2], lw.shape[-1]
    rows = lw.numel() // (Di * Do)
    out = (torch.empty_like(lw), torch.empty_like(uw), torch.empty_like(lb), torch.empty_like(ub))
    with torch.cuda.device(dev):
        check(load().fb_relax_with_norms_f32(op, _p(lw), _p(uw), _p(lb), _p(ub), _p(norm_l), _p(norm_u),
                                             *[_p(t) for t in out], rows, Di, Do, norm_code(p), eps,
                                             _p(violation), _stream()), "fb_relax_with_norms_f32")
    return out


def softmax_fused(x, p, eps, words=1, violation=None, ranges=False):
    """Fused softmax bound; returns None when the shape needs the unfused chain.  ranges=True appends the
    concretised range (l, u) of the result to the returned tuple."""
    dev = _chk(*x)
    lw, uw, lb, ub = x
    Di, Do = lw.shape[-2], lw.shape[-1]
    rows = lb.numel() // Do
    out = (torch.empty_like(lw), torch.empty_like(uw), torch.empty_like(lb), torch.empty_like(ub))
    if ranges:
        out = out + (torch.empty_like(lb), torch.empty_like(ub))
    with torch.cuda.device(dev):
        rc = load().fb_softmax_ranges_f32(*[_p(t) for t in x], *[_p(t) for t in out], *([] if ranges else [None, None]),
                                          rows, Di, Do, words, norm_code(p), eps, _p(violation), _stream())
    if rc in (2, 3):   # FB_ERR_SHAPE / FB_ERR_ALIGN: not a fused shape
        return None
    check(rc, "fb_softmax_ranges_f32")
    return out
