"""Generates tests/golden/*.npz from the reference's own Python implementation.

Run in a checkout that has the reference available (FAITH_REFERENCE, see ref_loader.py):

    python tests/golden/make_golden.py

For every case of cases.OP_CASES the reference `Bounds` operator
(Transformer_Verification_Code/Verifiers/Bounds.py) is run on the seeded inputs and its four
output tensors are stored; for the encoder case the reference `VerifierForward` pass
(Verifiers/VerifierForward.py:93-119) is run sentence by sentence and the concretised logit
bounds plus a few stage tensors are stored; for the search case the reference's `Verifier.verify`
(Verifiers/Verifier.py:62-147) is run and the radius it finds per position is stored.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import cases  # noqa: E402
import ref_loader  # noqa: E402


def run_reference_op(c):
    mod = ref_loader.load_reference_bounds()
    args = ref_loader.make_args(p=c["p"], perturbed_words=c["words"], method="ibp" if c.get("ibp") else "forward")
    (lw, lb, uw, ub), ex = cases.case_inputs(c)

    def mk(t):
        return mod.Bounds(args, c["p"], c["eps"], lw=t[0].clone(), lb=t[1].clone(), uw=t[2].clone(), ub=t[3].clone())

    x = mk((lw, lb, uw, ub))
    op = c["op"]
    if op == "concretize":
        l, u = x.concretize()
        return {"l": l, "u": u}
    if op == "relu":
        r = x.relu()
    elif op == "tanh":
        r = x.tanh()
    elif op == "exp":
        r = x.exp()
    elif op == "reciprocal":
        r = x.reciprocal()
    elif op == "matmul":
        r = x.matmul(ex["W"])
    elif op == "dense":
        import torch.nn as nn
        d = nn.Linear(ex["W"].shape[1], ex["W"].shape[0])
        d.weight.data, d.bias.data = ex["W"], ex["bias"]
        with torch.no_grad():
            r = x.dense(d)
    elif op == "dot":
        r = x.dot_product(mk(ex["y"]))
    elif op == "context":
        r = x.context(mk(ex["y"]))
    elif op == "mul_bounds":
        r = x.multiply(mk(ex["y"]))
    elif op == "softmax":
        r = x.softmax()
    elif op == "layer_norm":
        import types
        r = x.layer_norm(types.SimpleNamespace(weight=ex["W"], bias=ex["bias"]), "no_var")
    elif op == "layer_norm_std":
        import types
        r = x.layer_norm(types.SimpleNamespace(weight=ex["W"], bias=ex["bias"]), "standard")
    elif op == "mul_tensor":
        r = x.multiply(ex["W"])
    elif op == "sqr":
        r = x.sqr()
    elif op == "sqrt":
        r = x.sqrt()
    elif op == "scale":
        r = x.multiply(c["c"])
    elif op == "add":
        r = x.add(mk(ex["y"]))
    else:
        raise KeyError(op)
    return {"lw": r.lw, "lb": r.lb, "uw": r.uw, "ub": r.ub}


def main():
    if not ref_loader.reference_available():
        raise SystemExit("reference checkout not found at %s" % ref_loader.REFERENCE_ROOT)
    torch.set_num_threads(1)  # one summation order, whatever machine generates the files
    out = {}
    for name, c in cases.OP_CASES.items():
        if not c.get("golden", True):
            continue
        for k, v in run_reference_op(c).items():
            out["%s/%s" % (name, k)] = v.detach().contiguous().numpy().astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "ops.npz"), **out)

    from oracle import bounds_oracle as O
    c = cases.ENCODER_CASE
    model = O.make_encoder(c["seed"], c["layers"], c["d_model"], c["heads"], c["ffn"], c["std"])
    emb = cases.encoder_inputs(c)
    ver = ref_loader.build_reference_verifier(model, c["p"])
    enc = {}
    ls, us = [], []
    for s in range(c["B"]):
        l, u, stages = ref_loader.reference_encoder_pass(ver, emb[s:s + 1], c["index"], c["eps"])
        ls.append(float(l))
        us.append(float(u))
        for nm, b in stages:
            if nm in ("embedding", "layer0.scores", "layer0.probs", "layer0.output", "pooled"):
                bl, bu = b.concretize()
                enc["s%d/%s/l" % (s, nm)] = bl.numpy().astype(np.float32)
                enc["s%d/%s/u" % (s, nm)] = bu.numpy().astype(np.float32)
    enc["l"] = np.array(ls, dtype=np.float32)
    enc["u"] = np.array(us, dtype=np.float32)
    np.savez_compressed(os.path.join(HERE, "encoder.npz"), **enc)

    # the reference's own search loop (Verifier.verify, unchanged) on the same sentences
    sc = cases.SEARCH_CASE
    model = O.make_encoder(sc["seed"], sc["layers"], sc["d_model"], sc["heads"], sc["ffn"], sc["std"])
    emb = cases.encoder_inputs(sc)
    ver = ref_loader.build_reference_verifier(model, sc["p"])
    y = O.concrete_forward(model, emb)
    srch = {"labels": np.array([0 if float(y[s]) > 0 else 1 for s in range(sc["B"])], dtype=np.int64)}
    for s in range(sc["B"]):
        r = ref_loader.reference_epsilon_search(ver, emb[s:s + 1], int(srch["labels"][s]), sc["max_eps"], sc["iters"])
        srch["s%d/positions" % s] = np.array(sorted(r), dtype=np.int64)
        srch["s%d/eps" % s] = np.array([r[i] for i in sorted(r)], dtype=np.float64)
    # two perturbed words: warm-up of max_eps, doubling / halving, bisection (Verifier.py:149-201)
    ver2 = ref_loader.build_reference_verifier(model, sc["p"], perturbed_words=2)
    for s in range(sc["B"]):
        r = ref_loader.reference_epsilon_search(ver2, emb[s:s + 1], int(srch["labels"][s]), sc["max_eps"], sc["iters2"])
        keys = sorted(r)
        srch["s%d/pairs" % s] = np.array(keys, dtype=np.int64)
        srch["s%d/pair_eps" % s] = np.array([r[k] for k in keys], dtype=np.float64)
        srch["s%d/warmed_max_eps" % s] = np.array(ver2.max_eps, dtype=np.float64)
    np.savez_compressed(os.path.join(HERE, "search.npz"), **srch)
    print("wrote ops.npz (%d arrays), encoder.npz (%d arrays) and search.npz (%d arrays)" % (len(out), len(enc), len(srch)))


if __name__ == "__main__":
    main()
