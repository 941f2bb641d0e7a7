"""The C-ABI library: loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    src = open(os.path.join(ROOT, "include", "faith_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(fb_[a-z0-9_]+)\s*\(", src)))


def test_library_builds_and_exports_header_symbols():
    from faith_b200 import build
    lib_path = build.build()
    lib = ctypes.CDLL(lib_path)
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), "symbol %s declared in include/faith_b200.h is not exported" % n


def test_ctypes_prototypes_cover_header():
    from faith_b200 import _lib
    assert set(declared_symbols()) == set(_lib.SIGNATURES)
    lib = _lib.load()
    assert lib.fb_version() >= 100
    assert lib.fb_status_string(0) == b"ok"


def test_argument_validation_without_gpu():
    """Bad arguments are rejected before any CUDA call is made."""
    from faith_b200 import _lib
    lib = _lib.load()
    assert lib.fb_relax_f32(0, None, None, None, None, None, None, None, None, 1, 4, 4, 1, 2, 0.1, 0, None, None) == 1
    assert lib.fb_concretize_f32(1, 1, 1, 1, 1, 1, 1, 4, 4, 1, 7, 0.1, 0, None) == 1  # unknown norm
    assert lib.fb_concretize_f32(1, 1, 1, 1, 1, 1, 1, 6, 4, 4, 2, 0.1, 0, None) == 2  # Di % words != 0
    # product + residual + layer norm: missing row sums of the residual, slopes given for one line only, result aliasing
    # the residual
    P = [256 * (k + 1) for k in range(20)]   # never dereferenced
    assert lib.fb_matmul_residual_ln_f32(*P[:12], None, *P[13:], 256, 128, 128, 128, None) == 1
    assert lib.fb_matmul_residual_ln_f32(*P[:4], P[4], None, *P[6:], 256, 128, 128, 128, None) == 1
    assert lib.fb_matmul_residual_ln_f32(*P[:15], P[8], *P[16:], 256, 128, 128, 128, None) == 1


def test_ops_refuse_cpu_tensors():
    import pytest
    import torch
    import faith_b200
    x = torch.zeros(1, 2, 4, 4)
    b = torch.zeros(1, 2, 4)
    with pytest.raises(faith_b200.FaithError):
        faith_b200.BoundsLite(2, 0.1, x, b, x, b).relu()


def declared_prototypes():
    """name -> list of parameter kinds ('p' pointer, 'i' int, 'l' 64-bit integer, 'f' float, 'd' double) read from the header."""
    src = open(os.path.join(ROOT, "include", "faith_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    src = re.sub(r"//[^\n]*", "", src)
    out = {}
    for name, args in re.findall(r"\b(fb_[a-z0-9_]+)\s*\(([^)]*)\)\s*;", src):
        kinds = []
        for a in (s.strip() for s in args.split(",")):
            if a in ("", "void"):
                continue
            if "*" in a:
                kinds.append("p")
            elif re.search(r"\b(u?int64_t|size_t)\b", a):
                kinds.append("l")
            elif re.search(r"\bdouble\b", a):
                kinds.append("d")
            elif re.search(r"\bfloat\b", a):
                kinds.append("f")
            else:
                kinds.append("i")
        out[name] = kinds
    return out


def test_ctypes_prototypes_match_the_header_parameter_by_parameter():
    """Every ctypes signature has the header's parameter count and, per parameter, the header's kind of type; a
    mismatch would otherwise only show as a TypeError (or a shifted argument) on the first call on a GPU."""
    from faith_b200 import _lib

    def kind(t):
        if t in (ctypes.c_int, ctypes.c_uint):
            return "i"
        if t in (ctypes.c_int64, ctypes.c_uint64, ctypes.c_size_t):
            return "l"
        if t is ctypes.c_float:
            return "f"
        if t is ctypes.c_double:
            return "d"
        return "p"

    protos = declared_prototypes()
    for name, argtypes in _lib.SIGNATURES.items():
        assert [kind(t) for t in argtypes] == protos[name], name


def test_cnn_driver_validates_the_network_without_gpu():
    """fb_cnn_workspace_bytes walks the layer records on the host: a network that does not start with a convolution, a
    convolution behind a linear layer or a feature map that shrinks to nothing is refused (-1); a well-formed one gets
    its arena size, which grows with the rows of the shard."""
    import ctypes
    from faith_b200 import _lib
    lib = _lib.load()
    dummy = ctypes.c_void_p(256)     # never dereferenced on the host

    def net(layers, cin=3, h=8, w=8):
        recs = (_lib.CnnLayer * len(layers))()
        for r, ly in zip(recs, layers):
            r.kind, r.weight, r.bias = ly[0], dummy, None
            if ly[0] == _lib.FB_CNN_CONV:
                r.cout, r.kh, r.kw, r.stride, r.pad = ly[1:]
            elif ly[0] == _lib.FB_CNN_LINEAR:
                r.n_out = ly[1]
        return _lib.Cnn(len(layers), recs, cin, h, w), recs

    conv = (_lib.FB_CNN_CONV, 4, 3, 3, 1, 1)
    good, keep = net([conv, (_lib.FB_CNN_RELU,), (_lib.FB_CNN_CONV, 6, 3, 3, 2, 1), (_lib.FB_CNN_RELU,), (_lib.FB_CNN_LINEAR, 5)])
    small = lib.fb_cnn_workspace_bytes(ctypes.byref(good), 10)
    large = lib.fb_cnn_workspace_bytes(ctypes.byref(good), 192)
    assert 0 < small < large
    for bad_layers in ([(_lib.FB_CNN_RELU,), conv], [(_lib.FB_CNN_LINEAR, 5)], [conv, (_lib.FB_CNN_LINEAR, 5), conv],
                       [(_lib.FB_CNN_CONV, 4, 9, 9, 1, 0), (_lib.FB_CNN_CONV, 4, 3, 3, 1, 0)], [(7,)]):
        bad, keep2 = net(bad_layers)
        assert lib.fb_cnn_workspace_bytes(ctypes.byref(bad), 10) == -1, bad_layers
    assert lib.fb_cnn_workspace_bytes(None, 10) == -1
    # the forward call refuses bad arguments before touching the device
    assert lib.fb_cnn_forward_f32(None, None, 3, 0.1, 0, 1, None, 0, 1, None, None, None, None, 0, None) == 1
    out = ctypes.c_void_p(512)
    assert lib.fb_cnn_forward_f32(ctypes.byref(good), dummy, 3, 0.1, 0, 10 ** 6, None, 0, 1, out, out, None, dummy, 1 << 40,
                                  None) == 1      # more rows than dim_in
    assert lib.fb_cnn_forward_f32(ctypes.byref(good), dummy, 3, 0.1, 0, 8, None, 0, 1, out, out, None, dummy, 16, None) == 5  # arena too small


def test_compact_window_extent_without_gpu():
    """fb_cw_extent is host arithmetic: the largest window a pixel reaches through a chain of convolutions."""
    import ctypes
    from faith_b200 import _lib
    lib = _lib.load()

    def extent(h, w, chain):
        flat = [v for c in chain for v in c]
        arr = (ctypes.c_int * max(1, len(flat)))(*flat)
        wh, ww = ctypes.c_int(0), ctypes.c_int(0)
        rc = lib.fb_cw_extent(h, w, arr, len(chain), ctypes.byref(wh), ctypes.byref(ww))
        return rc, wh.value, ww.value

    assert extent(32, 32, [(3, 3, 1, 1)]) == (0, 3, 3)
    assert extent(32, 32, [(3, 3, 1, 1), (3, 3, 2, 1)]) == (0, 3, 3)          # the benchmark CNN
    assert extent(32, 32, [(3, 3, 1, 1), (3, 3, 1, 1)]) == (0, 5, 5)
    assert extent(16, 8, [(5, 3, 1, 2)]) == (0, 5, 3)
    assert extent(9, 9, [(2, 2, 3, 0)]) == (0, 1, 1)
    assert extent(8, 8, [(3, 3, 0, 1)])[0] == 1                                # stride 0
    assert extent(4, 4, [(9, 9, 1, 0)])[0] == 2                                # feature map shrinks to nothing
    assert extent(8, 8, [(3, 3, 1, 1)] * 9)[0] == 2                            # more than eight convolutions


def test_encoder_arena_size_without_gpu():
    """fb_encoder_workspace_bytes is host arithmetic: four bound slots sized for the widest tensor of a block, the range
    scratch of the dot products, the column-norm scratch and the row sums of the layer input; it grows with the
    sentences, and a width that the heads do not divide is refused."""
    import ctypes
    from faith_b200 import _lib
    lib = _lib.load()

    def enc(d_model=128, heads=4, ffn=512, layers=3):
        e = _lib.Encoder()
        e.layers, e.d_model, e.heads, e.ffn, e.layer_norm = layers, d_model, heads, ffn, 1
        return e

    def up(v):
        return (v + 255) // 256 * 256
    S, L, words = 256, 32, 1
    D, F, H = 128, 512, 4
    Di = words * D
    got = lib.fb_encoder_workspace_bytes(ctypes.byref(enc()), S, L, words)
    slot = 2 * up(S * L * Di * F * 4) + 2 * up(S * L * F * 4)
    want = (4 * slot + 4 * up(S * H * L * L * 4) + up((D + 1) * 4) + up(2 * S * L * (words + 1) * F * 4) +
            up(8 * S * L * (Di + 1) * 4))
    assert got == want
    assert lib.fb_encoder_workspace_bytes(ctypes.byref(enc()), 8, L, words) < got
    assert lib.fb_encoder_workspace_bytes(ctypes.byref(enc()), S, L, 2) > got
    assert lib.fb_encoder_workspace_bytes(ctypes.byref(enc(d_model=130)), S, L, words) == -1
    assert lib.fb_encoder_workspace_bytes(None, S, L, words) == -1
