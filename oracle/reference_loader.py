"""Import the reference's own Python `Bounds` (Transformer_Verification_Code/Verifiers/Bounds.py)
unchanged, on CPU, for pinning the oracle and for generating golden vectors.

The reference module needs three things that this environment lacks, none of which
touches the arithmetic: the `tvm` package (imported at Bounds.py:8-10 but only used
by the TVM/Ansor back-ends), a JIT-compiled CUDA extension (Bounds.py:14-26, only used
when FLAG==1), and the module-global `ansor_model_lut` that `dense` reads
(Bounds.py:1025) without it being defined.  All three are stubbed here.

TEST AND BASELINE INFRASTRUCTURE ONLY: tests, the golden generator and the reference arm /
CPU-baseline leg of bench.py may use this file; the faith_b200 package never does.  The
reference files are looked up in the copy staged under oracle/_ref/ (oracle/stage_reference.py),
else in a checkout named by the environment variable FAITH_REFERENCE or lying beside this
repository.
"""
import importlib.util
import os
import sys
import types

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import stage_reference  # noqa: E402

REFERENCE_ROOT = stage_reference.staged_root() or stage_reference.find_checkout() or ""


def reference_available():
    return os.path.isfile(os.path.join(
        REFERENCE_ROOT, "Transformer_Verification_Code", "Verifiers", "Bounds.py"))


def _stub(name):
    if name not in sys.modules:
        m = types.ModuleType(name)
        m.__path__ = []  # let "from tvm import relay" style imports resolve
        sys.modules[name] = m
    return sys.modules[name]


_cache = {}


def load_reference_bounds():
    """Returns the reference module object of Verifiers/Bounds.py (class `Bounds` inside)."""
    if "bounds" in _cache:
        return _cache["bounds"]
    tvm = _stub("tvm")
    tvm.relay = _stub("tvm.relay")
    contrib = _stub("tvm.contrib")
    contrib.graph_executor = _stub("tvm.contrib.graph_executor")
    tvm.contrib = contrib
    import torch.utils.cpp_extension as cpp_ext
    saved = cpp_ext.load
    cpp_ext.load = lambda *a, **k: types.SimpleNamespace()
    try:
        path = os.path.join(REFERENCE_ROOT, "Transformer_Verification_Code", "Verifiers", "Bounds.py")
        spec = importlib.util.spec_from_file_location("faith_reference_bounds", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        cpp_ext.load = saved
    mod.ansor_model_lut = None
    _cache["bounds"] = mod
    return mod


def load_reference_kernel_test(c_bound=None):
    """Returns the module object of HandTunedKernels/kernel_test/transformer_forward_test_bound.py
    (its test-local `Bounds(p, eps, lw, lb, uw, ub)` class, the comparator and the *_test functions).
    The module builds its extension with torch.utils.cpp_extension.load at import (:24-31); that call is
    answered with `c_bound` (an object exposing the c_*_verification functions), so that the module's
    cuda_* methods run whatever the caller plugs in.  Without `c_bound` an empty stand-in is given."""
    key = "ktest" if c_bound is None else ("ktest", id(c_bound))
    if key in _cache:
        return _cache[key]
    import torch.utils.cpp_extension as cpp_ext
    saved = cpp_ext.load
    cpp_ext.load = lambda *a, **k: (c_bound if c_bound is not None else types.SimpleNamespace())
    saved_env = os.environ.get("CUDA_VISIBLE_DEVICES")
    try:
        path = os.path.join(REFERENCE_ROOT, "HandTunedKernels", "kernel_test",
                            "transformer_forward_test_bound.py")
        spec = importlib.util.spec_from_file_location(
            "faith_reference_kernel_test" if c_bound is None else "faith_reference_kernel_test_plugged", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        cpp_ext.load = saved
        if saved_env is None:
            os.environ.pop("CUDA_VISIBLE_DEVICES", None)
        else:
            os.environ["CUDA_VISIBLE_DEVICES"] = saved_env
    _cache[key] = mod
    return mod


def make_args(p=2.0, perturbed_words=1, method="forward", current_flag=0):
    """The attribute bag the reference `Bounds` constructor reads (Bounds.py:272-291)."""
    return types.SimpleNamespace(method=method, perturbed_words=perturbed_words,
                                 current_flag=current_flag, kernel_type=0, p=p)


def load_reference_verifier():
    """Returns the reference `VerifierForward` class (Verifiers/VerifierForward.py), imported
    unchanged.  `data_utils` (dataset loaders; needs nltk and creates a ./tmp directory on
    import) is replaced by an empty stub because the bound pass never calls it."""
    if "verifier" in _cache:
        return _cache["verifier"]
    load_reference_bounds()  # installs the tvm stubs
    du = _stub("data_utils")
    du.sample = lambda *a, **k: []
    du.get_batches = lambda *a, **k: []
    import torch.utils.cpp_extension as cpp_ext
    saved = cpp_ext.load
    cpp_ext.load = lambda *a, **k: types.SimpleNamespace()
    pkg_root = os.path.join(REFERENCE_ROOT, "Transformer_Verification_Code")
    sys.path.insert(0, pkg_root)
    try:
        import Verifiers  # noqa: the reference package; its __init__ rebinds submodule names to classes
        vf_mod = sys.modules["Verifiers.VerifierForward"]
        sys.modules["Verifiers.Bounds"].ansor_model_lut = None
    finally:
        cpp_ext.load = saved
        sys.path.remove(pkg_root)
    _cache["verifier"] = vf_mod.VerifierForward
    return vf_mod.VerifierForward


def build_reference_verifier(model, p, perturbed_words=1, device="cpu", method="forward"):
    """A reference VerifierForward wired to a stand-in encoder built from an oracle model
    dict (see oracle.bounds_oracle.make_encoder).  Only the attributes the forward bound
    pass reads are provided (Verifier.py:11-34, VerifierForward.py:15-20,199-204).
    `device`: where the weights live and where `_bound_input` creates its tensors."""
    import torch.nn as nn
    VF = load_reference_verifier()

    def lin(w, b):
        m = nn.Linear(w.shape[1], w.shape[0])
        m.weight.data, m.bias.data = w.clone().to(device), b.clone().to(device)
        return m

    def ln(g, b):
        return types.SimpleNamespace(weight=g.clone().to(device), bias=b.clone().to(device))

    heads = model["heads"]
    layers = []
    for ly in model["layers"]:
        d = ly["q_w"].shape[0]
        attn_self = types.SimpleNamespace(num_attention_heads=heads, attention_head_size=d // heads,
                                          query=lin(ly["q_w"], ly["q_b"]), key=lin(ly["k_w"], ly["k_b"]),
                                          value=lin(ly["v_w"], ly["v_b"]))
        attn_out = types.SimpleNamespace(dense=lin(ly["ao_w"], ly["ao_b"]), LayerNorm=ln(ly["ln1_g"], ly["ln1_b"]))
        layers.append(types.SimpleNamespace(
            attention=types.SimpleNamespace(self=attn_self, output=attn_out),
            intermediate=types.SimpleNamespace(dense=lin(ly["f1_w"], ly["f1_b"])),
            output=types.SimpleNamespace(dense=lin(ly["f2_w"], ly["f2_b"]), LayerNorm=ln(ly["ln2_g"], ly["ln2_b"]))))
    v = VF.__new__(VF)
    v.args = make_args(p=p, perturbed_words=perturbed_words, method=method)
    v.device = device
    v.p = p
    v.ibp = method == "ibp"
    v.debug = False
    v.verbose = False
    v.perturbed_words = perturbed_words
    v.tvm_model_lut = {}
    v.ansor_model_lut = {}
    v.current_flag = 0
    v.hidden_act = "relu"
    v.layer_norm = model["layer_norm"]
    v.embeddings = types.SimpleNamespace(LayerNorm=ln(model["emb_ln_g"], model["emb_ln_b"]))
    v.encoding_layers = layers
    v.pooler = types.SimpleNamespace(dense=lin(model["pool_w"], model["pool_b"]))
    v.classifier = lin(model["cls_w"], model["cls_b"])
    return v


def reference_encoder_pass(verifier, emb_one, index, eps, bounds_cls=None):
    """Runs the reference bound pass for one sentence (emb_one [1, L, D]) and returns the
    concretised (l, u) of logit0 - logit1 plus the stage bounds, following
    VerifierForward.verify_safety (VerifierForward.py:93-119) and _bound_classifier
    (:289-305) without the `check` calls (they need a concrete forward of the real model).
    `bounds_cls`: the class the verifier's module-level name `Bounds` is bound to for the duration of the
    pass (VerifierForward.py:7 imports it by name; _bound_input :153 and _bound_pooling :270 construct through
    it), i.e. the one place where another implementation of the operator API plugs in.  None = the reference's."""
    import copy
    import torch
    vf_mod = sys.modules["Verifiers.VerifierForward"]
    saved_cls = vf_mod.Bounds
    if bounds_cls is not None:
        vf_mod.Bounds = bounds_cls
    try:
        return _reference_encoder_pass(verifier, emb_one, index, eps)
    finally:
        vf_mod.Bounds = saved_cls


def _reference_encoder_pass(verifier, emb_one, index, eps):
    import copy
    import torch
    stages = []
    with torch.no_grad():
        b = verifier._bound_input(emb_one.clone(), index=index, eps=eps)
        stages.append(("embedding", b))
        for i, layer in enumerate(verifier.encoding_layers):
            scores, probs, b = verifier._bound_layer(b, layer)
            stages.append(("layer%d.scores" % i, scores))
            stages.append(("layer%d.probs" % i, probs))
            stages.append(("layer%d.output" % i, b))
        b = verifier._bound_pooling(b, verifier.pooler)
        stages.append(("pooled", b))
        cls = copy.deepcopy(verifier.classifier)
        cls.weight[0, :] -= cls.weight[1, :]
        cls.bias[0] -= cls.bias[1]
        b = b.dense(cls, verifier.tvm_model_lut, FLAG=0)
        l, u = b.concretize()
    return l[0][0][0], u[0][0][0], stages


def reference_epsilon_search(verifier, emb_one, label, max_eps, num_iters):
    """Runs the reference's own search loop, Verifier.verify (Verifier.py:62-208), unchanged for one sentence
    (emb_one [1, L, D]) and returns {position: eps}, or {(i1, i2): eps} when the verifier perturbs two words (its
    max_eps is then warmed up first, :150-157, and left in verifier.max_eps).  The loop asks its `target` for the
    embeddings, the tokens and the concrete activations (`std`) that `check` compares the bounds with; check
    never asserts (utils.py:30 is commented out), so the stand-in target hands out zeros of the right shapes."""
    import contextlib
    import io
    import torch
    L, D = emb_one.shape[1], emb_one.shape[2]
    n_layers = len(verifier.encoding_layers)
    heads = verifier.encoding_layers[0].attention.self.num_attention_heads if n_layers else 1
    dev = emb_one.device
    std = {
        "embedding_output": torch.zeros(1, L, D, device=dev),
        "attention_scores": [torch.zeros(1, heads, L, L, device=dev) for _ in range(n_layers)],
        "attention_probs": [torch.zeros(1, heads, L, L, device=dev) for _ in range(n_layers)],
        "encoded_layers": [torch.zeros(1, L, D, device=dev) for _ in range(n_layers)],
        "pooled_output": torch.zeros(1, D, device=dev),
    }
    tokens = ["[CLS]"] + ["w%d" % i for i in range(1, L - 1)] + ["[SEP]"]
    verifier.target = types.SimpleNamespace(get_embeddings=lambda examples: (emb_one.clone(), [tokens]),
                                            step=lambda examples: [std])
    verifier.logger = types.SimpleNamespace(write=lambda *a, **k: None)
    verifier.max_eps = max_eps
    verifier.warmed = False
    verifier.num_verify_iters = num_iters
    verifier.eps = max_eps
    verifier.debug_pos = 1
    verifier.method = "forward"
    verifier.res = os.devnull
    with contextlib.redirect_stdout(io.StringIO()):
        result, _avg, _min = verifier.verify({"label": label})
    def key(pos):
        return tuple(int(i) for i in pos) if isinstance(pos, (tuple, list)) else int(pos)
    return {key(b["position"]): float(b["eps"]) for b in result["bounds"]}
