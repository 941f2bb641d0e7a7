"""The C++ whole-model driver against the CPU oracle: per-stage noise budget, golden vectors and
sampled containment of concrete forward passes."""
import numpy as np
import pytest
import torch

import cases
import helpers
from oracle import bounds_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _small():
    c = cases.ENCODER_CASE
    model = O.make_encoder(c["seed"], c["layers"], c["d_model"], c["heads"], c["ffn"], c["std"])
    return c, model, cases.encoder_inputs(c)


def test_encoder_driver_matches_oracle_and_golden():
    import faith_b200
    c, model, emb = _small()
    l32, u32 = O.encoder_forward(model, emb, [c["index"]], c["p"], c["eps"])
    l64, u64 = O.encoder_forward(O.model_to(model, torch.float64), emb.double(), [c["index"]], c["p"], c["eps"])
    ver = faith_b200.EncoderVerifier(model, DEV)
    l, u, viol = ver.forward(emb.to(DEV), [c["index"]], c["p"], c["eps"])
    assert int(viol.item()) == 0
    helpers.assert_within_noise(l, l32, l64, "logit lower")
    helpers.assert_within_noise(u, u32, u64, "logit upper")
    g = helpers.load_golden("encoder.npz")
    helpers.assert_within_noise(l, g["l"], l64, "logit lower vs golden")
    helpers.assert_within_noise(u, g["u"], u64, "logit upper vs golden")


def test_encoder_stage_by_stage_with_bounds_class():
    """The same pass through the Python `Bounds` class (one C-ABI call per operator), compared
    stage by stage with the oracle trace."""
    import math
    import types
    import faith_b200
    c, model, emb = _small()
    trace, trace64 = [], []
    O.encoder_forward(model, emb, [c["index"]], c["p"], c["eps"], trace=trace)
    O.encoder_forward(O.model_to(model, torch.float64), emb.double(), [c["index"]], c["p"], c["eps"], trace=trace64)
    st32, st64 = dict(trace), dict(trace64)
    args = types.SimpleNamespace(method="forward", perturbed_words=1, current_flag=1)
    ib = O.input_bounds(emb, [c["index"]], c["p"], c["eps"])
    x = faith_b200.Bounds(args, c["p"], c["eps"], lw=ib.lw.to(DEV), lb=ib.lb.to(DEV), uw=ib.uw.to(DEV), ub=ib.ub.to(DEV))

    def lin(w, b):
        return types.SimpleNamespace(weight=w.to(DEV), bias=b.to(DEV))

    from faith_b200 import ops
    heads = model["heads"]

    def split(b, tr=False):
        o = ops.split_heads(b._t4(), heads, tr)
        return b._new(o[0], o[1], o[2], o[3])

    def check(name, b):
        gl, gu = b.concretize()
        l32, u32 = st32[name].concretize()
        l64, u64 = st64[name].concretize()
        helpers.assert_within_noise(gl, l32, l64, name + " l")
        helpers.assert_within_noise(gu, u32, u64, name + " u")

    x = x.layer_norm(lin(model["emb_ln_g"], model["emb_ln_b"]), "no_var")
    check("embedding", x)
    for i, ly in enumerate(model["layers"]):
        q = split(x.dense(lin(ly["q_w"], ly["q_b"])))
        k = split(x.dense(lin(ly["k_w"], ly["k_b"])))
        v = split(x.dense(lin(ly["v_w"], ly["v_b"])))
        scores = q.dot_product(k).multiply(1.0 / math.sqrt(q.lw.shape[-1]))
        check("layer%d.scores" % i, scores)
        probs = scores.softmax()
        check("layer%d.probs" % i, probs)
        ctx = probs.context(v)
        m = ops.merge_heads(ctx._t4(), heads)
        ctx = ctx._new(m[0], m[1], m[2], m[3])
        att = ctx.dense(lin(ly["ao_w"], ly["ao_b"])).add(x).layer_norm(lin(ly["ln1_g"], ly["ln1_b"]), "no_var")
        check("layer%d.attention" % i, att)
        inter = att.dense(lin(ly["f1_w"], ly["f1_b"])).relu()
        check("layer%d.intermediate" % i, inter)
        x = inter.dense(lin(ly["f2_w"], ly["f2_b"])).add(att).layer_norm(lin(ly["ln2_g"], ly["ln2_b"]), "no_var")
        check("layer%d.output" % i, x)


def test_encoder_bounds_contain_sampled_forward_passes():
    """10 000 concrete forward passes sampled in the eps-ball (half on vertices, half inside)
    must land inside the interval the driver returns."""
    import faith_b200
    c, model, emb = _small()
    ver = faith_b200.EncoderVerifier(model, DEV)
    l, u, _ = ver.forward(emb.to(DEV), [c["index"]], c["p"], c["eps"])
    l, u = l.cpu(), u.cpu()
    g = torch.Generator().manual_seed(9)
    n = 10000
    for s in range(emb.shape[0]):
        delta = (torch.randint(0, 2, (n, c["d_model"]), generator=g).float() * 2 - 1) * c["eps"]
        delta[: n // 2] *= torch.rand(n // 2, 1, generator=g)
        x = emb[s:s + 1].repeat(n, 1, 1)
        x[:, c["index"], :] += delta
        y = O.concrete_forward(model, x)
        assert float(y.min()) >= float(l[s]) - 1e-5, (float(y.min()), float(l[s]))
        assert float(y.max()) <= float(u[s]) + 1e-5, (float(y.max()), float(u[s]))


@pytest.mark.parametrize("p,words,positions", [(2.0, 2, [1, 2]), (1.0, 1, [3])])
def test_encoder_other_norms_and_two_words(p, words, positions):
    import faith_b200
    c, model, emb = _small()
    l32, u32 = O.encoder_forward(model, emb, positions, p, 5e-4)
    l64, u64 = O.encoder_forward(O.model_to(model, torch.float64), emb.double(), positions, p, 5e-4)
    ver = faith_b200.EncoderVerifier(model, DEV)
    l, u, viol = ver.forward(emb.to(DEV), positions, p, 5e-4)
    assert int(viol.item()) == 0
    helpers.assert_within_noise(l, l32, l64, "l")
    helpers.assert_within_noise(u, u32, u64, "u")


def test_encoder_full_size_config_properties():
    """Configuration of the headline benchmark (3 layers, d_model 128, 4 heads, FFN 512, L 32,
    one perturbed word, L-inf) on 8 sentences at eps = 1e-3: finite, ordered, contains the
    unperturbed forward pass, and agrees with the oracle within the fp32 noise budget."""
    import faith_b200
    model = O.make_encoder(4)
    emb = torch.randn(8, 32, 128, generator=torch.Generator().manual_seed(4))
    ver = faith_b200.EncoderVerifier(model, DEV)
    l, u, viol = ver.forward(emb.to(DEV), [1], float("inf"), 1e-3)
    assert ver.check_status(viol) == 0
    l, u = l.cpu(), u.cpu()
    assert bool(torch.isfinite(l).all()) and bool(torch.isfinite(u).all())
    y = O.concrete_forward(model, emb)
    assert bool((l <= y + 1e-5).all()) and bool((y <= u + 1e-5).all())
    l32, u32 = O.encoder_forward(model, emb[:2], [1], float("inf"), 1e-3)
    l64, u64 = O.encoder_forward(O.model_to(model, torch.float64), emb[:2].double(), [1], float("inf"), 1e-3)
    helpers.assert_within_noise(l[:2], l32, l64, "l")
    helpers.assert_within_noise(u[:2], u32, u64, "u")


def test_encoder_full_width_two_perturbed_words():
    """d_model 128 with two perturbed words (dim_in 256, L2): the paths that exist only for 128-wide
    models (input bounds fused with the embedding layer norm, ranges handed over by the GEMM epilogue
    with one word block per tile) with more than one word block."""
    import faith_b200
    model = O.make_encoder(4)
    emb = torch.randn(2, 32, 128, generator=torch.Generator().manual_seed(5))
    ver = faith_b200.EncoderVerifier(model, DEV)
    l, u, viol = ver.forward(emb.to(DEV), [1, 5], 2.0, 1e-3)
    assert int(viol.item()) == 0
    l32, u32 = O.encoder_forward(model, emb, [1, 5], 2.0, 1e-3)
    l64, u64 = O.encoder_forward(O.model_to(model, torch.float64), emb.double(), [1, 5], 2.0, 1e-3)
    helpers.assert_within_noise(l, l32, l64, "l")
    helpers.assert_within_noise(u, u32, u64, "u")
    y = O.concrete_forward(model, emb)
    assert bool((l.cpu() <= y + 1e-5).all()) and bool((y <= u.cpu() + 1e-5).all())


def test_encoder_without_layers():
    """An encoder with no layers (embedding layer norm, pooler, classifier): the driver's input stage must leave both
    lines of the bound written for the pooler (d_model 128 takes the fused input kernel)."""
    import faith_b200
    model = O.make_encoder(7, layers=0)
    emb = torch.randn(3, 8, 128, generator=torch.Generator().manual_seed(7))
    ver = faith_b200.EncoderVerifier(model, DEV)
    l, u, viol = ver.forward(emb.to(DEV), [2], float("inf"), 0.01)
    assert ver.check_status(viol) == 0
    l32, u32 = O.encoder_forward(model, emb, [2], float("inf"), 0.01)
    l64, u64 = O.encoder_forward(O.model_to(model, torch.float64), emb.double(), [2], float("inf"), 0.01)
    helpers.assert_within_noise(l, l32, l64, "l")
    helpers.assert_within_noise(u, u32, u64, "u")


def test_instances_entry_point_matches_one_call_per_radius():
    """fb_encoder_forward_instances_f32 (own positions and radius per instance, the radius folded into the input
    weights) against fb_encoder_forward_f32 called once per (position, radius): same bounds up to rounding."""
    import faith_b200
    c, model, emb = _small()
    ver = faith_b200.EncoderVerifier(model, DEV)
    combos = [(0, 1, 2e-4), (0, 5, 6e-4), (1, 3, 1e-4), (1, 6, 3e-4), (0, 2, 4e-4)]
    e = torch.stack([emb[s] for s, _, _ in combos]).to(DEV)
    pos = torch.tensor([[i] for _, i, _ in combos], dtype=torch.int32, device=DEV)
    eps = torch.tensor([r for _, _, r in combos], dtype=torch.float32, device=DEV)
    l, u, viol = ver.forward_instances(e, pos, c["p"], eps)
    assert ver.check_status(viol) == 0
    for k, (s, i, r) in enumerate(combos):
        l1, u1, v1 = ver.forward(emb[s:s + 1].to(DEV), [i], c["p"], r)
        l64, u64 = O.encoder_forward(O.model_to(model, torch.float64), emb[s:s + 1].double(), [i], c["p"], r)
        l32, u32 = O.encoder_forward(model, emb[s:s + 1], [i], c["p"], r)
        helpers.assert_within_noise(l[k:k + 1], l32, l64, "instance %d l" % k)
        helpers.assert_within_noise(u[k:k + 1], u32, u64, "instance %d u" % k)
        helpers.assert_within_noise(l[k:k + 1], l1, l64, "instance %d l vs single call" % k)
        helpers.assert_within_noise(u[k:k + 1], u1, u64, "instance %d u vs single call" % k)


def test_batched_search_reproduces_the_reference_radii():
    """The reference's search (Verifier.verify, run unchanged on CPU when the golden file was made) against the
    batched search: all (sentence, position) pairs of a bisection round are instances of one driver call.  A
    bisection step whose bound lands within rounding noise of zero may go the other way, which moves the answer by
    at most the width of the last steps (max_eps / 2^iters); most positions agree to the last bit."""
    import faith_b200
    from faith_b200.search import EpsilonSearch
    c = sc = cases.SEARCH_CASE
    model = O.make_encoder(c["seed"], c["layers"], c["d_model"], c["heads"], c["ffn"], c["std"])
    emb = cases.encoder_inputs(c)
    g = helpers.load_golden("search.npz")
    ver = faith_b200.EncoderVerifier(model, DEV)
    labels = torch.as_tensor(g["labels"])
    srch = EpsilonSearch(ver, c["p"], sc["max_eps"], sc["iters"], max_instances=8)
    got = srch.run(emb.to(DEV), labels)
    step = sc["max_eps"] / 2 ** sc["iters"]
    n, same = 0, 0
    for s in range(c["B"]):
        pos = [int(i) for i in g["s%d/positions" % s]]
        assert sorted(got[s]) == pos
        for i, e in zip(pos, g["s%d/eps" % s]):
            n += 1
            same += np.float32(got[s][i]) == np.float32(e)   # the reference keeps its answer in a float32 tensor
            assert abs(got[s][i] - float(e)) <= 2.001 * step, (s, i, got[s][i], float(e))
    assert same >= n - 1, "%d of %d radii differ from the reference" % (n - same, n)
    # 12 words x (1 + 8) probes = 108 verify_safety calls of the reference, here 9 rounds of 2 calls (8 instances each)
    assert srch.instances == n * (sc["iters"] + 1) and srch.passes == (sc["iters"] + 1) * 2


def test_batched_two_word_search_reproduces_the_reference_radii():
    """Two perturbed words (Verifier.py:149-201): warm-up of max_eps, then per pair doubling / halving and bisection,
    every pair with its own state machine and one driver call per round for all unfinished pairs."""
    import faith_b200
    from faith_b200.search import EpsilonSearch
    c = cases.SEARCH_CASE
    model = O.make_encoder(c["seed"], c["layers"], c["d_model"], c["heads"], c["ffn"], c["std"])
    emb = cases.encoder_inputs(c)
    g = helpers.load_golden("search.npz")
    ver = faith_b200.EncoderVerifier(model, DEV)
    step_floor = 2.0 ** -c["iters2"]
    for s in range(c["B"]):   # the reference warms max_eps up per verifier; the golden file used a fresh one per sentence
        srch = EpsilonSearch(ver, c["p"], c["max_eps"], c["iters2"], max_instances=16)
        got, warmed = srch.run_pairs(emb[s:s + 1].to(DEV), torch.as_tensor(g["labels"][s:s + 1]))
        assert warmed == float(g["s%d/warmed_max_eps" % s])
        pairs = [tuple(int(v) for v in q) for q in g["s%d/pairs" % s]]
        assert sorted(got[0]) == pairs
        diff = 0
        for q, e in zip(pairs, g["s%d/pair_eps" % s]):
            diff += np.float32(got[0][q]) != np.float32(e)
            assert abs(got[0][q] - float(e)) <= 2.001 * step_floor * max(float(e), warmed), (s, q, got[0][q], float(e))
        assert diff <= 1, "%d of %d radii differ from the reference" % (diff, len(pairs))


@pytest.mark.parametrize("words,positions,p", [(1, [1], float("inf")), (2, [3, 30], 2.0)])
def test_first_layer_projections_skip_zero_row_blocks_bit_for_bit(words, positions, p):
    """In the first layer only the weight rows of the perturbed positions are non-zero; the tensor-core GEMM is told so
    and stores zeros for the other row blocks without reading or multiplying them.  The pass must give the same bits
    as with the shortcut switched off (FB_ENCODER_NO_ZERO_SKIP), for one set of positions and for per-sentence ones."""
    import os
    import faith_b200
    model = O.make_encoder(4)
    emb = torch.randn(6, 32, 128, generator=torch.Generator().manual_seed(6)).to(DEV)
    ver = faith_b200.EncoderVerifier(model, DEV)
    inst = torch.tensor([[(q + 5 * s) % 32 for q in positions] for s in range(6)], dtype=torch.int32, device=DEV)
    eps_i = torch.full((6,), 1e-3, device=DEV)

    def run():
        a = ver.forward(emb, positions, p, 1e-3)
        b = ver.forward_instances(emb, inst, p, eps_i)
        return [t.clone() for t in (a[0], a[1], b[0], b[1])]

    assert "FB_ENCODER_NO_ZERO_SKIP" not in os.environ
    fast = run()
    os.environ["FB_ENCODER_NO_ZERO_SKIP"] = "1"
    try:
        plain = run()
    finally:
        del os.environ["FB_ENCODER_NO_ZERO_SKIP"]
    for x, y in zip(fast, plain):
        assert torch.equal(x, y)
    assert bool(torch.isfinite(fast[0]).all()) and bool((fast[0] <= fast[1]).all())


@pytest.mark.parametrize("full_size", [False, True])
def test_last_layer_for_the_first_token_only_gives_the_same_bounds(full_size):
    """The pooler reads token 0 of the last layer only; with first_token_only the driver forms the rest of that layer for
    token 0 alone.  Same bounds as the full pass up to the rounding of the other kernel shapes, and within the fp32
    noise of the fp64 oracle (which propagates every position, as the reference does)."""
    import faith_b200
    if full_size:
        model = O.make_encoder(4)
        emb = torch.randn(4, 32, 128, generator=torch.Generator().manual_seed(4))
        positions, p, eps = [1], float("inf"), 1e-3
    else:
        c, model, emb = _small()
        positions, p, eps = [c["index"]], c["p"], c["eps"]
    full = faith_b200.EncoderVerifier(model, DEV)
    pruned = faith_b200.EncoderVerifier(model, DEV, first_token_only=True)
    l0, u0, v0 = full.forward(emb.to(DEV), positions, p, eps)
    l1, u1, v1 = pruned.forward(emb.to(DEV), positions, p, eps)
    assert full.check_status(v0) == 0 and pruned.check_status(v1) == 0
    l32, u32 = O.encoder_forward(model, emb, positions, p, eps)
    l64, u64 = O.encoder_forward(O.model_to(model, torch.float64), emb.double(), positions, p, eps)
    helpers.assert_within_noise(l1, l32, l64, "l")
    helpers.assert_within_noise(u1, u32, u64, "u")
    width = float((u0 - l0).abs().max())
    assert float((l1 - l0).abs().max()) <= 1e-4 * max(width, 1.0) and float((u1 - u0).abs().max()) <= 1e-4 * max(width, 1.0)
    # per-sentence instances take the same route
    inst = torch.tensor([[positions[0]]] * emb.shape[0], dtype=torch.int32, device=DEV)
    l2, u2, _ = pruned.forward_instances(emb.to(DEV), inst, p, torch.full((emb.shape[0],), eps, device=DEV))
    helpers.assert_within_noise(l2, l32, l64, "l instances")
    helpers.assert_within_noise(u2, u32, u64, "u instances")


def test_mean_pooling_option():
    """pooling = "mean" (the pooling the benchmark description names; the reference pools the first token): mean over the
    positions -> dense -> tanh.  Against the oracle's restatement (no reference implementation exists: unpinned), and
    10 000 sampled concrete passes of the mean-pooled model inside [l, u]."""
    import faith_b200
    c, model, emb = _small()
    model = dict(model, pooling="mean")
    ver = faith_b200.EncoderVerifier(model, DEV)
    l, u, viol = ver.forward(emb.to(DEV), [c["index"]], c["p"], c["eps"])
    assert ver.check_status(viol) == 0
    l32, u32 = O.encoder_forward(model, emb, [c["index"]], c["p"], c["eps"])
    l64, u64 = O.encoder_forward(O.model_to(model, torch.float64), emb.double(), [c["index"]], c["p"], c["eps"])
    helpers.assert_within_noise(l, l32, l64, "l")
    helpers.assert_within_noise(u, u32, u64, "u")
    first = faith_b200.EncoderVerifier(dict(model, pooling="first"), DEV).forward(emb.to(DEV), [c["index"]], c["p"], c["eps"])
    assert float((first[0] - l).abs().max()) > 1e-4          # it is a different model
    l, u = l.cpu(), u.cpu()
    g = torch.Generator().manual_seed(12)
    n = 10000
    for s in range(emb.shape[0]):
        delta = (torch.randint(0, 2, (n, c["d_model"]), generator=g).float() * 2 - 1) * c["eps"]
        delta[: n // 2] *= torch.rand(n // 2, 1, generator=g)
        x = emb[s:s + 1].repeat(n, 1, 1)
        x[:, c["index"], :] += delta
        y = O.concrete_forward(model, x)
        assert float(y.min()) >= float(l[s]) - 1e-5 and float(y.max()) <= float(u[s]) + 1e-5


@pytest.mark.parametrize("words,positions,p,S", [(1, [1], float("inf"), 8), (2, [3, 30], 2.0, 8), (1, [2], float("inf"), 4)])
def test_layer_norms_applied_in_gemm_epilogues_give_the_same_bounds(words, positions, p, S):
    """With 128 features the first layer norm of every block is applied by the epilogue of the attention output product
    (row means of the product from the operand and the weight's column means, of the residual from the row sums its
    producer left behind).  FB_ENCODER_SEPARATE_LN=1 keeps the norm as a launch of its own; both routes stay within
    the noise budget of the fp64 oracle, the fused one is deterministic, and fewer than 256 rows (S = 4) take the
    separate launch either way."""
    import os
    import faith_b200
    from faith_b200 import _lib
    model = O.make_encoder(4)
    emb = torch.randn(S, 32, 128, generator=torch.Generator().manual_seed(8)).to(DEV)
    ver = faith_b200.EncoderVerifier(model, DEV)
    lib = _lib.load()

    def run():
        n0 = lib.fb_launch_count()
        a = ver.forward(emb, positions, p, 1e-3)
        torch.cuda.synchronize()
        return [t.clone() for t in a[:2]], lib.fb_launch_count() - n0

    assert "FB_ENCODER_SEPARATE_LN" not in os.environ
    fused, n_fused = run()
    os.environ["FB_ENCODER_SEPARATE_LN"] = "1"
    try:
        separate, n_separate = run()
    finally:
        del os.environ["FB_ENCODER_SEPARATE_LN"]
    layers = len(model["layers"])
    assert n_separate - n_fused == (layers if S * 32 >= 256 else 0)
    # Two fp32 evaluation orders of this pass differ by what the later layers make of their rounding (the oracle's own
    # fp32 run strays from its fp64 run by about 1e-2 of a bound here), so both routes are held against the fp64 oracle
    # with the noise budget of the other driver tests, on the first two sentences.
    l32, u32 = O.encoder_forward(model, emb[:2].cpu(), positions, p, 1e-3)
    l64, u64 = O.encoder_forward(O.model_to(model, torch.float64), emb[:2].cpu().double(), positions, p, 1e-3)
    for route, name in ((fused, "norm in the epilogue"), (separate, "norm as a launch")):
        assert bool(torch.isfinite(route[0]).all()) and bool(torch.isfinite(route[1]).all())
        helpers.assert_within_noise(route[0][:2], l32, l64, "lower, " + name)
        helpers.assert_within_noise(route[1][:2], u32, u64, "upper, " + name)
    again, _ = run()
    for x, y in zip(again, fused):
        assert torch.equal(x, y)
    assert lib.fb_tc_check() == 0


def test_run_and_record_gives_the_reference_result_file(tmp_path):
    """run_and_record on the real driver: the record's radii are those of the batched search (which the test above holds
    against the reference's own run), held in single precision with eps_normalized = eps / ||embedding||_p, the
    summary follows from them, and the file on disk is the record as the reference writes it."""
    import json
    import faith_b200
    from faith_b200.search import EpsilonSearch, run_and_record
    c = sc = cases.SEARCH_CASE
    model = O.make_encoder(c["seed"], c["layers"], c["d_model"], c["heads"], c["ffn"], c["std"])
    emb = cases.encoder_inputs(c).to(DEV)
    labels = torch.as_tensor(helpers.load_golden("search.npz")["labels"])
    ver = faith_b200.EncoderVerifier(model, DEV)
    plain = EpsilonSearch(ver, c["p"], sc["max_eps"], sc["iters"], max_instances=8).run(emb, labels)
    lines = []
    rec = run_and_record(EpsilonSearch(ver, c["p"], sc["max_eps"], sc["iters"], max_instances=8), emb, labels, None, 1,
                         tmp_path / "res.json", lines.append)
    assert len(rec["examples"]) == c["B"] and len(lines) == 3
    mins, avgs = [], []
    for s, ex in enumerate(rec["examples"]):
        assert [b["position"] for b in ex["bounds"]] == sorted(plain[s])
        for b in ex["bounds"]:
            e32 = torch.tensor(plain[s][b["position"]], dtype=torch.float32)
            assert b["eps"] == float(e32)
            assert b["eps_normalized"] == float(e32 / torch.norm(emb[s, b["position"]].cpu(), p=float(c["p"])))
        eps = [b["eps"] for b in ex["bounds"]]
        mins.append(min(eps))
        avgs.append(sum(eps) / len(eps))
    assert abs(rec["minimum"] - sum(mins) / len(mins)) < 1e-12 and abs(rec["average"] - sum(avgs) / len(avgs)) < 1e-12
    assert json.loads((tmp_path / "res.json").read_text()) == rec
