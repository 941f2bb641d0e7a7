"""ctypes binding of libfaith_b200.so (the C ABI declared in include/faith_b200.h).

There is no CPU fallback: if the shared library is missing or a call fails, an exception is
raised.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfaith_b200.so")

FB_P1, FB_P2, FB_PINF = 1, 2, 3
FB_NATIVE, FB_TRANSPOSED = 0, 1
FB_RELU, FB_TANH, FB_EXP, FB_RECIPROCAL, FB_SQR, FB_SQRT = 0, 1, 2, 3, 4, 5
FB_INTERVAL = 8

_P = ctypes.c_void_p
_I = ctypes.c_int
_L = ctypes.c_int64
_F = ctypes.c_float


class EncoderLayer(ctypes.Structure):
    _fields_ = [(n, _P) for n in ("q_w", "q_b", "k_w", "k_b", "v_w", "v_b", "ao_w", "ao_b", "ln1_g", "ln1_b",
                                  "f1_w", "f1_b", "f2_w", "f2_b", "ln2_g", "ln2_b")]


class Encoder(ctypes.Structure):
    _fields_ = [("layers", _I), ("d_model", _I), ("heads", _I), ("ffn", _I), ("layer_norm", _I),
                ("emb_ln_g", _P), ("emb_ln_b", _P), ("layer", ctypes.POINTER(EncoderLayer)),
                ("pool_w", _P), ("pool_b", _P), ("cls_w", _P), ("cls_b", _P), ("first_token_only", _I), ("pooling", _I)]


class CnnLayer(ctypes.Structure):
    _fields_ = [("kind", _I), ("weight", _P), ("bias", _P), ("cout", _I), ("kh", _I), ("kw", _I), ("stride", _I),
                ("pad", _I), ("n_out", _I)]


class Cnn(ctypes.Structure):
    _fields_ = [("n_layers", _I), ("layer", ctypes.POINTER(CnnLayer)), ("cin", _I), ("h", _I), ("w", _I)]


FB_CNN_CONV, FB_CNN_RELU, FB_CNN_LINEAR = 0, 1, 2

# name -> argtypes; every function returns int (fb_status) unless listed in _OTHER_RESTYPE
SIGNATURES = {
    "fb_concretize_f32": [_P] * 6 + [_L, _I, _I, _I, _I, _F, _I, _P],
    "fb_relax_f32": [_I] + [_P] * 8 + [_L, _I, _I, _I, _I, _F, _I, _P, _P],
    "fb_norm_partials_f32": [_P] * 4 + [_L, _I, _I, _I, _P],
    "fb_relax_with_norms_f32": [_I] + [_P] * 10 + [_L, _I, _I, _I, _F, _P, _P],
    "fb_matmul_f32": [_P] * 10 + [_L, _I, _I, _I, _P],
    "fb_tc_error_flag": [ctypes.POINTER(_I)],
    "fb_tc_check": [],
    "fb_tc_selftest_timeout": [_P] * 5 + [_L, _I, _I, _I, _I, _P, _P],
    "fb_dot_product_f32": [_P] * 16 + [_I, _I, _I, _I, _I, _I, _I, _F, _F, _I, _P],
    "fb_matmul_heads_f32": [_P] * 10 + [_L, _I, _I, _I, _I, _I, _P],
    "fb_matmul_residual_f32": [_P] * 16 + [_L, _I, _I, _I, _P],
    "fb_matmul_residual_ln_f32": [_P] * 20 + [_L, _I, _I, _I, _P],
    "fb_matmul_heads_ranges_f32": [_P] * 13 + [_L, _I, _I, _I, _I, _I, _I, _I, _F, _P],
    "fb_relax_coef_f32": [_I] + [_P] * 8 + [_L, _I, _I, _I, _I, _F, _P, _P],
    "fb_relax_coef_given_f32": [_I] + [_P] * 8 + [_L, _I, _P, _P],
    "fb_matmul_coef_f32": [_P] * 12 + [_L, _I, _I, _I, _P],
    "fb_dot_product_heads_f32": [_P] * 16 + [_I, _I, _I, _I, _I, _I, _I, _F, _F, _I, _I, _P],
    "fb_dot_product_given_f32": [_P] * 16 + [_I, _I, _I, _I, _I, _I, _I, _F, _F, _I, _I, _I, _P],
    "fb_context_heads_f32": [_P] * 16 + [_I, _I, _I, _I, _I, _I, _I, _F, _F, _I, _P],
    "fb_context_given_f32": [_P] * 16 + [_I, _I, _I, _I, _I, _I, _I, _F, _F, _I, _I, _P],
    "fb_dot_product_noalloc_f32": [_P] * 12 + [_I, _I, _I, _I, _I, _I, _I, _F, _F, _I, _P],
    "fb_dot_product_noalloc_max_floats": [],
    "fb_mul_bounds_f32": [_P] * 12 + [_L, _I, _I, _I, _I, _F, _P],
    "fb_add_f32": [_P] * 12 + [_L, _I, _I, _P],
    "fb_scale_f32": [_P] * 8 + [_L, _I, _I, _F, _P],
    "fb_rowsum_f32": [_P] * 8 + [_L, _I, _I, _P],
    "fb_mul_features_f32": [_P] * 9 + [_L, _I, _I, _P],
    "fb_interval_mul_f32": [_P] * 6 + [_L, _P],
    "fb_interval_dot_f32": [_P] * 6 + [_I, _I, _I, _I, _P],
    "fb_softmax_f32": [_P] * 8 + [_L, _I, _I, _I, _I, _F, _P, _P],
    "fb_softmax_ranges_f32": [_P] * 10 + [_L, _I, _I, _I, _I, _F, _P, _P],
    "fb_layernorm_novar_f32": [_P] * 14 + [_L, _I, _I, _P],
    "fb_split_heads_f32": [_P] * 4 + [_I] * 6 + [_P],
    "fb_merge_heads_f32": [_P] * 4 + [_I] * 5 + [_P],
    "fb_conv2d_f32": [_P] * 10 + [_I] * 10 + [_P],
    "fb_conv2d_identity_relax_f32": [_I, _P, _P, _P, _P, _F] + [_P] * 5 + [_L, _L] + [_I] * 9 + [_F, _P, _P],
    "fb_conv2d_windowed_f32": [_P] * 5 + [_L, _L, _I, _I, _P, _I] + [_I] * 8 + [_P],
    "fb_cw_extent": [_I, _I, _P, _I, ctypes.POINTER(_I), ctypes.POINTER(_I)],
    "fb_cw_identity_relax_f32": [_I, _P, _P, _P, _P, _F] + [_P] * 5 + [_L, _L] + [_I] * 9 + [_F, _P, _P],
    "fb_cw_conv2d_f32": [_P] * 5 + [_L, _L, _I, _I, _P, _I] + [_I] * 8 + [_P],
    "fb_cw_norm_partials_f32": [_P] * 4 + [_L, _L, _I, _I, _I, _P, _I, _I, _I, _I, _I, _P],
    "fb_cw_relax_apply_f32": [_I] + [_P] * 11 + [_L, _L, _I, _I, _P, _I, _I, _I, _I, _I, _F, _P, _P],
    "fb_cw_linear_f32": [_P] * 6 + [_L, _L, _I, _I, _P, _I, _I, _I, _I, _I, _P],
    "fb_cw_expand_f32": [_P] * 4 + [_L, _L, _I, _I, _P, _I, _I, _I, _I, _P],
    "fb_cnn_workspace_bytes": [ctypes.POINTER(Cnn), _L],
    "fb_cnn_forward_f32": [ctypes.POINTER(Cnn), _P, _I, _F, _L, _L, _P, _I, _I, _P, _P, _P, _P, _L, _P],
    "fb_encoder_workspace_bytes": [ctypes.POINTER(Encoder), _I, _I, _I],
    "fb_encoder_forward_f32": [ctypes.POINTER(Encoder), _P, _I, _I, ctypes.POINTER(_I), _I, _I, _F, _P, _P, _P, _P, _L, _P],
    "fb_encoder_forward_instances_f32": [ctypes.POINTER(Encoder), _P, _I, _I, _P, _P, _I, _I, _P, _P, _P, _P, _L, _P],
    "fb_comm_unique_id": [_P],
    "fb_comm_create": [ctypes.POINTER(_P), _P, _I, _I, _L],
    "fb_comm_destroy": [_P],
    "fb_comm_abort": [_P],
    "fb_comm_info": [_P, ctypes.POINTER(_I), ctypes.POINTER(_I), ctypes.POINTER(_L)],
    "fb_comm_set_wait_ns": [_P, ctypes.c_uint64],
    "fb_comm_check": [_P, _I],
    "fb_comm_last_error": [],
    "fb_allreduce_f32": [_P, _P, _L, _I, _I, _P],
    "fb_relax_sharded_f32": [_P, _I, _I] + [_P] * 9 + [_L, _I, _I, _I, _I, _F, _P, _P],
    "fb_concretize_sharded_f32": [_P, _I] + [_P] * 7 + [_L, _I, _I, _I, _I, _F, _P],
    "fb_profile_enable": [_I],
    "fb_profile_read": [_I, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(_L), ctypes.POINTER(ctypes.c_double),
                        ctypes.POINTER(ctypes.c_double)],
    "fb_launch_count": [],
    "fb_bench_ffma": [_P, _I, ctypes.POINTER(ctypes.c_double), _P],
    "fb_bench_tf32": [_I, ctypes.POINTER(ctypes.c_double), _P],
    "fb_status_string": [_I],
    "fb_last_cuda_error": [],
    "fb_version": [],
}
_OTHER_RESTYPE = {"fb_comm_last_error": ctypes.c_char_p, "fb_status_string": ctypes.c_char_p, "fb_encoder_workspace_bytes": _L, "fb_cnn_workspace_bytes": _L, "fb_launch_count": _L,
                   "fb_dot_product_noalloc_max_floats": _L}

_lib = None


def load():
    """Loads the shared library (once) and declares the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError("libfaith_b200.so is not built (expected at %s); run `python -m faith_b200.build`. "
                           "There is no CPU fallback." % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is missing
        fn.argtypes = argtypes
        fn.restype = _OTHER_RESTYPE.get(name, _I)
    _lib = lib
    return lib


class FaithError(RuntimeError):
    pass


def check(status, what):
    if status != 0:
        lib = load()
        msg = lib.fb_status_string(status).decode()
        extra = ""
        if status == 4:
            extra = " (cudaError %d)" % lib.fb_last_cuda_error()
        if status == 7:
            extra = " (%s)" % lib.fb_comm_last_error().decode()
        raise FaithError("%s failed: %s%s" % (what, msg, extra))
