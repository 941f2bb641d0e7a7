"""Host logic of the batched radius search against a plain-loop restatement of the reference's search
(Transformer_Verification_Code/Verifiers/Verifier.py:106-206), with a fake verifier on the CPU: a pair
(sentence, positions) certifies exactly when the radius is below a threshold the test chooses."""
import json

import torch

from faith_b200.search import EpsilonSearch, perturbable_positions, result_record, write_result


class FakeVerifier:
    """Certified iff eps < thr[sentence][first position] (* 0.5 with two positions); the sentence is recognised by
    the value its embedding carries in [0, 0]."""
    device = torch.device("cpu")

    def __init__(self, thr):
        self.thr = thr
        self.calls = 0

    def forward_instances(self, e, pos, p, eps):
        self.calls += 1
        n = e.shape[0]
        l = torch.empty(n)
        for j in range(n):
            s = int(e[j, 0, 0])
            t = self.thr[s][int(pos[j, 0])] * (0.5 if pos.shape[1] == 2 else 1.0)
            l[j] = 1.0 if float(eps[j]) < t else -1.0
        return l, l.clone(), torch.zeros(1, dtype=torch.int32)

    def check_status(self, viol):
        return 0


def _inputs(N=3, L=8, D=4, seed=0):
    g = torch.Generator().manual_seed(seed)
    emb = torch.randn(N, L, D, generator=g)
    emb[:, 0, 0] = torch.arange(N, dtype=torch.float32)
    thr = (torch.rand(N, L, generator=g) * 0.08 + 0.001).tolist()
    labels = torch.zeros(N, dtype=torch.int64)
    return emb, labels, thr


def _reference_one_word(thr_row, L, max_eps, iters):
    out = {}
    for i in range(1, L - 1):
        l, r = 0, max_eps
        for _ in range(iters):
            m = (l + r) / 2
            if float(torch.tensor(m, dtype=torch.float32)) < thr_row[i]:
                l = m
            else:
                r = m
        out[i] = l
    return out


def test_one_word_search_follows_the_reference_bisection():
    emb, labels, thr = _inputs()
    fake = FakeVerifier(thr)
    search = EpsilonSearch(fake, p=2, max_eps=0.1, num_verify_iters=10, max_instances=7)
    got = search.run(emb, labels)
    for s in range(emb.shape[0]):
        assert got[s] == _reference_one_word(thr[s], emb.shape[1], 0.1, 10)
    n = emb.shape[0] * (emb.shape[1] - 2)
    assert search.instances == n * 11            # the unused probe at max_eps and ten bisection steps
    assert search.passes == 11 * -(-n // 7)


def test_label_one_certifies_on_the_upper_bound():
    emb, labels, thr = _inputs(N=2)
    labels[:] = 1

    class Flipped(FakeVerifier):
        def forward_instances(self, e, pos, p, eps):
            l, u, v = super().forward_instances(e, pos, p, eps)
            return -l, -l, v                     # certified now means u < 0
    got = EpsilonSearch(Flipped(thr), 2, 0.1).run(emb, labels)
    assert got[1] == _reference_one_word(thr[1], emb.shape[1], 0.1, 10)


def test_softmax_violation_means_not_certified():
    emb, labels, thr = _inputs(N=1)

    class Failing(FakeVerifier):
        def check_status(self, viol):
            return 1
    got = EpsilonSearch(Failing(thr), 2, 0.1).run(emb, labels)
    assert all(v == 0 for v in got[0].values())


def _reference_pairs(thr_row, L, max_eps, iters):
    def safe(i1, e):
        return float(torch.tensor(e, dtype=torch.float32)) < thr_row[i1] * 0.5
    while not safe(1, max_eps):
        max_eps /= 2
    while safe(1, max_eps):
        max_eps *= 2
    out = {}
    for i1 in range(1, L - 1):
        for i2 in range(i1 + 1, L - 1):
            l, r = 0, max_eps
            ok = safe(i1, r)
            while ok:
                l = r
                r *= 2
                ok = safe(i1, r)
            if l == 0:
                while not ok:
                    r /= 2
                    ok = safe(i1, r)
                l, r = r, r * 2
            for _ in range(iters):
                m = (l + r) / 2
                if safe(i1, m):
                    l = m
                else:
                    r = m
            out[(i1, i2)] = l
    return out, max_eps


def test_two_word_search_follows_the_reference_state_machine():
    emb, labels, thr = _inputs(N=1, L=7)
    search = EpsilonSearch(FakeVerifier(thr), p=2, max_eps=0.5, num_verify_iters=6, max_instances=5)
    got, max_eps = search.run_pairs(emb, labels)
    want, want_max = _reference_pairs(thr[0], 7, 0.5, 6)
    assert max_eps == want_max
    assert got[0] == want


def test_word_pieces_are_skipped():
    tokens = ["[CLS]", "un", "##believ", "##able", "film", "[SEP]"]
    assert perturbable_positions(6) == [1, 2, 3, 4]
    assert perturbable_positions(6, tokens) == [4]


def test_result_record_has_the_reference_layout(tmp_path):
    emb, labels, thr = _inputs(N=2, L=6)
    labels[1] = 1
    found = [{1: 0.0125, 3: 0.05}, {2: 0.03125}]
    rec = result_record(found, emb, labels, p=2, tokens=[["a"] * 6, ["b"] * 6], seconds=[1.5, 2.5])
    assert list(rec) == ["examples", "minimum", "average"]
    ex = rec["examples"][0]
    assert list(ex) == ["tokens", "label", "bounds", "time"]
    assert ex["label"] == 0.0 and rec["examples"][1]["label"] == 1.0 and ex["time"] == 1.5
    b = ex["bounds"][0]
    e32 = torch.tensor(0.0125, dtype=torch.float32)
    assert b == {"position": 1, "eps": float(e32), "eps_normalized": float(e32 / torch.norm(emb[0, 1], p=2))}
    avg0 = (float(e32) + float(torch.tensor(0.05, dtype=torch.float32))) / 2
    assert rec["average"] == (avg0 + 0.03125) / 2
    assert rec["minimum"] == (float(e32) + 0.03125) / 2
    lines = []
    write_result(tmp_path / "res.json", rec, log=lines.append)
    assert json.loads((tmp_path / "res.json").read_text()) == rec
    assert (tmp_path / "res.json").read_text() == json.dumps(rec, indent=4)
    assert lines == ["2 valid examples", "Minimum: %.5f" % rec["minimum"], "Average: %.5f" % rec["average"]]


def test_result_record_two_words_and_empty_sentence():
    emb, labels, _ = _inputs(N=1, L=6)
    rec = result_record([{(1, 2): 0.25, (1, 3): 0.125}], emb, labels, p=1)
    assert rec["examples"][0]["bounds"] == [{"position": (1, 2), "eps": 0.25}, {"position": (1, 3), "eps": 0.125}]
    assert rec["minimum"] == 0.125 and rec["average"] == 0.1875
    try:
        result_record([{}], emb, labels, p=1)
    except ValueError as e:
        assert "no searched position" in str(e)
    else:
        raise AssertionError("an empty sentence must be rejected")


def test_run_and_record_mirrors_the_reference_run(tmp_path):
    """One word: word pieces are skipped, every other position is searched, the record has the reference's layout and is
    written with its summary lines; two words: every pair of the remaining positions; three words are refused as the
    reference refuses them."""
    from faith_b200.search import run_and_record
    emb, labels, thr = _inputs(N=2, L=7)
    tokens = [["[CLS]", "a", "b", "##c", "d", "e", "[SEP]"], ["[CLS]", "f", "g", "h", "i", "j", "[SEP]"]]
    search = EpsilonSearch(FakeVerifier(thr), p=2, max_eps=0.1, num_verify_iters=6, max_instances=64)
    lines = []
    rec = run_and_record(search, emb, labels, tokens, 1, tmp_path / "res.json", lines.append)
    assert [b["position"] for b in rec["examples"][0]["bounds"]] == [1, 4, 5]     # 2 precedes a word piece, 3 is one
    assert [b["position"] for b in rec["examples"][1]["bounds"]] == [1, 2, 3, 4, 5]
    want = _reference_one_word(thr[0], 7, 0.1, 6)
    for b in rec["examples"][0]["bounds"]:
        assert b["eps"] == float(torch.tensor(want[b["position"]], dtype=torch.float32))
    assert rec["examples"][0]["tokens"] == tokens[0]
    assert json.loads((tmp_path / "res.json").read_text()) == rec
    assert lines[0] == "2 valid examples" and lines[1].startswith("Minimum: ") and lines[2].startswith("Average: ")
    pairs = run_and_record(EpsilonSearch(FakeVerifier(thr), 2, 0.5, 4), emb[:1], labels[:1], tokens[:1], 2)
    assert [tuple(b["position"]) for b in pairs["examples"][0]["bounds"]] == [(1, 4), (1, 5), (4, 5)]
    try:
        run_and_record(search, emb, labels, tokens, 3)
    except NotImplementedError:
        pass
    else:
        raise AssertionError("three perturbed words must be refused")
