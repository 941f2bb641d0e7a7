"""Drop-in for the reference's JIT-built extension module `c_relu_verification`.

The reference loads its kernels with
`torch.utils.cpp_extension.load(name="c_relu_verification", sources=[kernel.cpp, *.cu])`
(Verifiers/Bounds.py:14-26) and calls four functions on the result (kernel.cpp:297-304).  This
module exposes functions with the same names, positional arguments and in-place semantics
(outputs are caller-allocated tensors, nothing is returned), plus the two the reference left
commented out (kernel.cpp:243-295).  As in the reference, lw/uw arrive transposed
([.., dim_out, dim_in], Bounds.py:1203-1211), the norm is p = 2 and there is one perturbed
word; `epsilon` is the perturbation radius.

Unlike the reference's wrappers, the row count is taken from the tensors, so batch > 1 works
for relu and tanh as well.
"""
import torch

from . import ops
from ._lib import FB_RELU, FB_TANH, FB_TRANSPOSED, FB_NATIVE


def _relax(op, src_lb, src_ub, src_lw, src_uw, out_lb, out_ub, out_lw, out_uw, length, dim_in, dim_out, epsilon):
    if src_lw.shape[-1] != dim_in or src_lw.shape[-2] != dim_out:
        raise ValueError("expected lw/uw of shape [.., dim_out=%d, dim_in=%d], got %s"
                         % (dim_out, dim_in, tuple(src_lw.shape)))
    ops.relax(op, src_lw, src_uw, src_lb, src_ub, 2, float(epsilon), 1, FB_TRANSPOSED,
              out=(out_lw, out_uw, out_lb, out_ub))


def c_relu_verification(src_lb, src_ub, src_lw, src_uw, out_lb, out_ub, out_lw, out_uw,
                        length, dim_in, dim_out, epsilon):
    _relax(FB_RELU, src_lb, src_ub, src_lw, src_uw, out_lb, out_ub, out_lw, out_uw, length, dim_in, dim_out, epsilon)


def c_tanh_verification(src_lb, src_ub, src_lw, src_uw, out_lb, out_ub, out_lw, out_uw,
                        length, dim_in, dim_out, epsilon):
    _relax(FB_TANH, src_lb, src_ub, src_lw, src_uw, out_lb, out_ub, out_lw, out_uw, length, dim_in, dim_out, epsilon)


def _dot(x_l, y_l, x_u, y_u, x_lb, x_ub, y_lb, y_ub, x_lw, x_uw, y_lw, y_uw, z_lb, z_ub, z_lw, z_uw, epsilon):
    ops.dot_product((x_lw, x_uw, x_lb, x_ub), (y_lw, y_uw, y_lb, y_ub), 2, float(epsilon), 1, 1.0, FB_TRANSPOSED,
                    scratch=(x_l, x_u, y_l, y_u), out=(z_lw, z_uw, z_lb, z_ub))


def c_dot_product_verification_QK(x_l, y_l, x_u, y_u, x_lb, x_ub, y_lb, y_ub, x_lw, x_uw, y_lw, y_uw,
                                  z_lb, z_ub, z_lw, z_uw, batch_size, length, dim_out, dim_in, epsilon):
    """x, y: [batch, length, dim_out(contracted), dim_in]; z: [batch, length, length, dim_in]."""
    _dot(x_l, y_l, x_u, y_u, x_lb, x_ub, y_lb, y_ub, x_lw, x_uw, y_lw, y_uw, z_lb, z_ub, z_lw, z_uw, epsilon)


def c_dot_product_verification_V(x_l, y_l, x_u, y_u, x_lb, x_ub, y_lb, y_ub, x_lw, x_uw, y_lw, y_uw,
                                 z_lb, z_ub, z_lw, z_uw, batch_size, length, dim_out, dim_in, epsilon):
    """x: [batch, length, length(contracted), dim_in]; y: [batch, dim_out, length(contracted), dim_in];
    z: [batch, length, dim_out, dim_in]."""
    _dot(x_l, y_l, x_u, y_u, x_lb, x_ub, y_lb, y_ub, x_lw, x_uw, y_lw, y_uw, z_lb, z_ub, z_lw, z_uw, epsilon)


def c_matmul_verification(x_lb, x_ub, x_lw, x_uw, W, y_lb, y_ub, y_lw, y_uw,
                          batch_size, length, dim_in, dim_out, dim_y_out):
    """Native layout (kernel.cpp:243-266): x_lw [batch, length, dim_in, dim_out], W [dim_y_out, dim_out]."""
    from ._lib import check, load
    dev = ops._chk(x_lb, x_ub, x_lw, x_uw, W, y_lb, y_ub, y_lw, y_uw)
    with torch.cuda.device(dev):
        check(load().fb_matmul_f32(x_lw.data_ptr(), x_uw.data_ptr(), x_lb.data_ptr(), x_ub.data_ptr(), W.data_ptr(),
                                   None, y_lw.data_ptr(), y_uw.data_ptr(), y_lb.data_ptr(), y_ub.data_ptr(),
                                   batch_size * length, dim_in, dim_out, dim_y_out, ops._stream()), "fb_matmul_f32")


def c_convolution_verification(x_lb, x_ub, x_lw, x_uw, W, y_lb, y_ub, y_lw, y_uw,
                               batch_size, Height, Width, CIN, COUT, K, Stride, padding_size, dim_in):
    """kernel.cpp:268-295: x_lw [batch, dim_in, CIN, H, W], x_lb [batch, CIN, H, W], W [COUT, CIN, K, K]."""
    from ._lib import check, load
    dev = ops._chk(x_lb, x_ub, x_lw, x_uw, W, y_lb, y_ub, y_lw, y_uw)
    with torch.cuda.device(dev):
        check(load().fb_conv2d_f32(x_lw.data_ptr(), x_uw.data_ptr(), x_lb.data_ptr(), x_ub.data_ptr(), W.data_ptr(),
                                   None, y_lw.data_ptr(), y_uw.data_ptr(), y_lb.data_ptr(), y_ub.data_ptr(),
                                   batch_size, dim_in, CIN, Height, Width, COUT, K, K, Stride, padding_size,
                                   ops._stream()), "fb_conv2d_f32")
