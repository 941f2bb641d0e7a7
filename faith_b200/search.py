"""The reference's search for the largest certified perturbation radius, with the probes batched.

Reference: Verifier.verify (Transformer_Verification_Code/Verifiers/Verifier.py:106-147, one perturbed word): for every
perturbable position i of a sentence, one probe at max_eps (whose answer the reference does not use, :116) and then
num_verify_iters bisection steps on [0, max_eps], each step a full bound pass (verify_safety) at m = (l + r) / 2 that
moves l up when the sentence is certified (logit0 - logit1 > 0 for label 0, < 0 for label 1,
VerifierForward.py:306-312) and r down otherwise; the answer is l.  Sentences, positions and probes of different words are
independent given the radius, so here every round is ONE call of the whole-model driver over all (sentence, position)
pairs, each instance with its own radius (fb_encoder_forward_instances_f32).

With two perturbed words (Verifier.py:149-201) the reference first warms max_eps up on the pair (1, 2), then for every
pair of positions doubles or halves the radius until the answer flips and bisects from there: the number of probes
differs from pair to pair, so here every pair carries its own small state machine and a round evaluates the current
probe of every pair that is not finished.
"""
import numpy as np
import torch


def perturbable_positions(length, tokens=None):
    """Positions the reference perturbs: 1 .. length-2 ([CLS] and [SEP] stay, Verifier.py:107), minus word pieces
    (a token starting with '#' at i or i+1, :109-110) when the tokens are known."""
    out = []
    for i in range(1, length - 1):
        if tokens is not None and (tokens[i][0] == "#" or tokens[i + 1][0] == "#"):
            continue
        out.append(i)
    return out


class EpsilonSearch:
    """verifier: a faith_b200.EncoderVerifier.  max_instances bounds the instances of one driver call (the driver's
    arena grows with it: about 68 MB per instance for the 128-wide, 32-token model)."""

    def __init__(self, verifier, p, max_eps, num_verify_iters=10, max_instances=256, probe_max_eps=True):
        self.ver = verifier
        self.p = p
        self.max_eps = float(max_eps)
        self.iters = int(num_verify_iters)
        self.max_instances = int(max_instances)
        self.probe_max_eps = probe_max_eps
        self.passes = 0          # driver calls made
        self.instances = 0       # instances propagated (the reference would have made this many verify_safety calls)

    def _safe(self, emb, sent, pos, labels, eps):
        """One round: certified[j] for instance j = (sentence sent[j], position pos[j]) at radius eps[j]."""
        dev = self.ver.device
        n = sent.numel()
        safe = torch.empty(n, dtype=torch.bool, device=dev)
        for a in range(0, n, self.max_instances):
            b = min(n, a + self.max_instances)
            e = emb.index_select(0, sent[a:b])
            l, u, viol = self.ver.forward_instances(e, pos[a:b].reshape(b - a, -1).contiguous(), self.p, eps[a:b].contiguous())
            status = self.ver.check_status(viol)
            # bit 0 (a softmax denominator not provably positive) is the reference's failed assertion, which
            # verify_safety turns into "not certified" (VerifierForward.py:120-125); the flag is per call, so the
            # whole chunk is treated that way
            ok = torch.where(labels.index_select(0, sent[a:b]) == 0, l > 0, u < 0)
            safe[a:b] = ok if status == 0 else torch.zeros_like(ok)
            self.passes += 1
            self.instances += b - a
        return safe

    def run(self, emb, labels, positions=None):
        """emb [N, L, D] and labels [N] on the device; positions: per sentence the list of positions to search (default:
        all perturbable ones).  Returns a list of dicts {position: eps} per sentence, eps being the reference's `l`
        after the last bisection step."""
        dev = self.ver.device
        N, L, _ = emb.shape
        if positions is None:
            positions = [perturbable_positions(L)] * N
        sent = torch.tensor([s for s in range(N) for _ in positions[s]], dtype=torch.int64, device=dev)
        pos = torch.tensor([i for s in range(N) for i in positions[s]], dtype=torch.int32, device=dev)
        labels = labels.to(dev)
        lo = torch.zeros(sent.numel(), dtype=torch.float64, device=dev)
        hi = torch.full_like(lo, self.max_eps)
        if self.probe_max_eps:
            self._safe(emb, sent, pos, labels, hi.float())   # the reference's first probe; its answer is not used
        for _ in range(self.iters):
            mid = (lo + hi) / 2          # the reference bisects in Python floats (double precision)
            safe = self._safe(emb, sent, pos, labels, mid.float())
            lo = torch.where(safe, mid, lo)
            hi = torch.where(safe, hi, mid)
        lo = lo.cpu().tolist()
        out, k = [], 0
        for s in range(N):
            out.append({int(i): lo[k + j] for j, i in enumerate(positions[s])})
            k += len(positions[s])
        return out

    def run_pairs(self, emb, labels, pairs=None, warm_up=True):
        """Two perturbed words.  emb [N, L, D], labels [N]; pairs: per sentence the list of (i1, i2) to search (default:
        all i1 < i2 among the perturbable positions).  Returns (list of dicts {(i1, i2): eps} per sentence, max_eps after
        the warm-up).  The warm-up is the reference's (Verifier.py:150-157): on the first sentence and the pair (1, 2),
        halve max_eps until it certifies, then double it until it does not."""
        dev = self.ver.device
        N, L, _ = emb.shape
        labels = labels.to(dev)
        if pairs is None:
            pp = perturbable_positions(L)
            pairs = [[(a, b) for k, a in enumerate(pp) for b in pp[k + 1:]]] * N
        max_eps = self.max_eps
        if warm_up:
            s0 = torch.zeros(1, dtype=torch.int64, device=dev)
            p0 = torch.tensor([[1, 2]], dtype=torch.int32, device=dev)

            def probe(e):
                return bool(self._safe(emb, s0, p0, labels, torch.tensor([e], dtype=torch.float32, device=dev))[0])
            while not probe(max_eps):
                max_eps /= 2
            while probe(max_eps):
                max_eps *= 2
        sent = torch.tensor([s for s in range(N) for _ in pairs[s]], dtype=torch.int64, device=dev)
        pos = torch.tensor([list(q) for s in range(N) for q in pairs[s]], dtype=torch.int32, device=dev).reshape(-1, 2)
        n = sent.numel()
        lo, hi = np.zeros(n), np.full(n, max_eps)     # the reference's l, r (Python floats)
        phase = np.zeros(n, dtype=np.int64)           # 0 first probe, 1 doubling, 2 halving, 3 bisecting, 4 done
        step = np.zeros(n, dtype=np.int64)
        cur = hi.copy()
        while (phase != 4).any():
            act = np.nonzero(phase != 4)[0]
            idx = torch.as_tensor(act, device=dev)
            safe = self._safe(emb, sent[idx], pos[idx], labels,
                              torch.as_tensor(cur[act], dtype=torch.float32, device=dev)).cpu().numpy()
            for k, ok in zip(act, safe):
                ph = phase[k]
                if ph in (0, 1):
                    if ok:                       # while safe: l = r; r *= 2
                        lo[k] = hi[k]
                        hi[k] *= 2
                        cur[k] = hi[k]
                        phase[k] = 1
                        continue
                    if ph == 0:                  # never certified: halve until it is
                        hi[k] /= 2
                        cur[k] = hi[k]
                        phase[k] = 2
                        continue
                    phase[k] = 3                 # doubling ended: bisect [l, r]
                elif ph == 2:
                    if not ok:
                        hi[k] /= 2
                        cur[k] = hi[k]
                        continue
                    lo[k], hi[k] = hi[k], hi[k] * 2
                    phase[k] = 3
                else:                            # one bisection step
                    if ok:
                        lo[k] = cur[k]
                    else:
                        hi[k] = cur[k]
                    step[k] += 1
                if phase[k] == 3:
                    if step[k] >= self.iters:
                        phase[k] = 4
                    else:
                        cur[k] = (lo[k] + hi[k]) / 2
        out, k = [], 0
        for s in range(N):
            out.append({tuple(q): float(lo[k + j]) for j, q in enumerate(pairs[s])})
            k += len(pairs[s])
        return out, max_eps


def run_and_record(search, emb, labels, tokens=None, perturbed_words=1, path=None, log=None):
    """The reference's Verifier.run (Verifiers/Verifier.py:36-60) on a batch of sentences: search every perturbable
    position (one word) or pair of positions (two words) of every sentence, word pieces skipped where the tokens are
    given (:109-110, :159-163), and return the reference's result record; with `path` the record is also written as the
    reference writes it, with `log` (a callable taking one string) its summary lines are logged.  search: an
    EpsilonSearch; emb [N, L, D] and labels [N] on the verifier's device."""
    N, L, _ = emb.shape
    positions = [perturbable_positions(L, tokens[s] if tokens is not None else None) for s in range(N)]
    if perturbed_words == 1:
        found = search.run(emb, labels, positions)
    elif perturbed_words == 2:
        pairs = [[(a, b) for k, a in enumerate(pp) for b in pp[k + 1:]] for pp in positions]
        found, _ = search.run_pairs(emb, labels, pairs)
    else:
        raise NotImplementedError("perturbed_words = %r (the reference supports 1 and 2, Verifier.py:203-204)" % (perturbed_words,))
    record = result_record(found, emb, labels, search.p, tokens)
    if path is not None:
        write_result(path, record, log)
    elif log is not None:
        log("{} valid examples".format(len(record["examples"])))
        log("Minimum: {:.5f}".format(record["minimum"]))
        log("Average: {:.5f}".format(record["average"]))
    return record


def result_record(per_sentence, emb, labels, p, tokens=None, seconds=None):
    """The reference's result file for one run of the search, as a dict ready for json.dumps(indent=4).

    Reference: Verifier.run and Verifier.verify (Transformer_Verification_Code/Verifiers/Verifier.py:40-60, :76-80,
    :139-147, :197-206).  per_sentence is what run() or run_pairs() returned: one dict {position: eps} or
    {(i1, i2): eps} per sentence.  Each sentence becomes {"tokens", "label", "bounds": [...], "time"}; a one-word
    bound is {"position", "eps", "eps_normalized"} with eps held in single precision, as the reference keeps it in a
    float tensor (:98, :137), and eps_normalized = eps / ||embedding of that position||_p in single precision (:143-146);
    a two-word bound is {"position": (i1, i2), "eps"} in double precision (:194-200).  "average" is the mean over
    sentences of the per-sentence mean radius and "minimum" the mean over sentences of the per-sentence smallest radius
    (:45-47, :52-58).  A sentence with nothing to search has no mean radius (the reference divides by zero there,
    :206) and is rejected.  tokens: per sentence the list of token strings (default: the position numbers as strings);
    seconds: per sentence the time the reference would have logged (default: 0.0, the batched search has no
    per-sentence time)."""
    emb = emb.detach().float().cpu()
    labels = [float(v) for v in labels.tolist()] if hasattr(labels, "tolist") else [float(v) for v in labels]
    N, L, _ = emb.shape
    if len(per_sentence) != N or len(labels) != N:
        raise ValueError("result_record: one entry per sentence is needed")
    examples, sum_avg, sum_min = [], 0.0, 0.0
    for s, found in enumerate(per_sentence):
        if not found:
            raise ValueError("result_record: sentence %d has no searched position" % s)
        bounds, sum_eps, min_eps = [], 0.0, 1e30
        for position, eps in found.items():
            if isinstance(position, tuple):
                value = float(eps)
                bounds.append({"position": (int(position[0]), int(position[1])), "eps": value})
            else:
                e32 = torch.tensor(float(eps), dtype=torch.float32)
                norm = torch.norm(emb[s, int(position), :], p=float(p))
                value = float(e32)
                bounds.append({"position": int(position), "eps": value, "eps_normalized": float(e32 / norm)})
            sum_eps += value
            min_eps = min(min_eps, value)
        examples.append({
            "tokens": list(tokens[s]) if tokens is not None else [str(i) for i in range(L)],
            "label": labels[s],
            "bounds": bounds,
            "time": float(seconds[s]) if seconds is not None else 0.0,
        })
        sum_avg += sum_eps / len(found)
        sum_min += min_eps
    return {"examples": examples, "minimum": sum_min / N, "average": sum_avg / N}


def write_result(path, record, log=None):
    """Writes the record the way the reference does (Verifier.py:59-60: json.dumps(result, indent=4)) and, when log
    is a callable taking one string, the three summary lines the reference logs (:49-51)."""
    import json
    with open(path, "w") as f:
        f.write(json.dumps(record, indent=4))
    if log is not None:
        log("{} valid examples".format(len(record["examples"])))
        log("Minimum: {:.5f}".format(record["minimum"]))
        log("Average: {:.5f}".format(record["average"]))
