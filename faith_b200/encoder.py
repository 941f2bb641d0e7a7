"""Python handle of the C++ whole-model driver (fb_encoder_forward_f32)."""
import ctypes

import torch

from . import _lib, ops
from ._lib import Encoder, EncoderLayer, check, load

_LAYER_KEYS = ("q_w", "q_b", "k_w", "k_b", "v_w", "v_b", "ao_w", "ao_b", "ln1_g", "ln1_b",
               "f1_w", "f1_b", "f2_w", "f2_b", "ln2_g", "ln2_b")


class EncoderVerifier:
    """Forward bound pass of a BERT-style encoder for a batch of sentences.

    `model` is a dict of float32 tensors: emb_ln_g, emb_ln_b, layers (list of dicts with the
    keys of _LAYER_KEYS, nn.Linear layout), pool_w, pool_b, cls_w [2, D], cls_b [2], heads,
    layer_norm ("no_var" or "no"), optionally pooling ("first": the reference's first-token pooler, the default; "mean":
    mean over the positions).  Weights are copied to `device` once.

    first_token_only: the reference propagates every layer at every position (VerifierForward.py:93-119) although its
    pooler reads token 0 of the last layer only (:269-287).  With this flag the last layer forms keys and values at every
    position but the query, the attention row and everything behind them for token 0 alone: the same bounds up to the
    rounding of other kernel shapes, about a quarter less work for three layers.  Off by default, so that a pass does the
    work the reference does.
    """

    def __init__(self, model, device, first_token_only=False):
        self.device = torch.device(device)
        self.heads = int(model["heads"])
        self.ln = {"no": 0, "no_var": 1}[model["layer_norm"]]
        keep = []

        def dev(t):
            t = t.detach().to(self.device, torch.float32).contiguous()
            keep.append(t)
            return t.data_ptr()

        self.d_model = model["pool_w"].shape[0]
        self.ffn = model["layers"][0]["f1_w"].shape[0] if model["layers"] else self.d_model
        n = len(model["layers"])
        self._layers = (EncoderLayer * max(n, 1))()
        for i, ly in enumerate(model["layers"]):
            for k in _LAYER_KEYS:
                setattr(self._layers[i], k, dev(ly[k]))
        self._enc = Encoder(n, self.d_model, self.heads, self.ffn, self.ln, dev(model["emb_ln_g"]),
                            dev(model["emb_ln_b"]), ctypes.cast(self._layers, ctypes.POINTER(EncoderLayer)),
                            dev(model["pool_w"]), dev(model["pool_b"]), dev(model["cls_w"]), dev(model["cls_b"]),
                            1 if first_token_only else 0, {"first": 0, "mean": 1}[model.get("pooling", "first")])
        self._keep = keep
        self._ws = None

    def workspace_bytes(self, S, L, words=1):
        n = load().fb_encoder_workspace_bytes(ctypes.byref(self._enc), S, L, words)
        if n < 0:
            raise _lib.FaithError("invalid encoder configuration")
        return n

    @staticmethod
    def check_status(violation):
        """Reads the status word of a pass (synchronises) and raises if the bounds must not be used: bit 2 = a
        bounded wait inside a tensor-core kernel expired, so l / u are partly written.  Returns the word;
        bits 0 and 1 (softmax denominator not provably positive, inverted hidden range) are left to the caller
        as in the reference, which asserts on the first (Bounds.py:1147)."""
        v = int(violation.item())
        if v & 4:
            raise _lib.FaithError("a bounded wait inside a tensor-core kernel expired during the bound pass; "
                                  "the returned bounds are not valid (status word %d)" % v)
        return v

    def forward(self, emb, positions, p, eps, out=None):
        """emb [S, L, D] on the device; positions: perturbed token indices.  Returns (l, u, violation):
        concretised bounds of logit0 - logit1 per sentence and the device status word of the pass (see
        check_status; any non-zero value means the bounds are no proof)."""
        ops._chk(emb)
        S, L, D = emb.shape
        words = len(positions)
        need = self.workspace_bytes(S, L, words)
        if self._ws is None or self._ws.numel() < need:
            self._ws = None
            self._ws = torch.empty(need, dtype=torch.uint8, device=self.device)
        if out is None:
            out = (torch.empty(S, device=self.device), torch.empty(S, device=self.device),
                   torch.empty(1, dtype=torch.int32, device=self.device))
        l, u, viol = out
        pos = (ctypes.c_int * words)(*positions)
        with torch.cuda.device(self.device):
            check(load().fb_encoder_forward_f32(ctypes.byref(self._enc), emb.data_ptr(), S, L, pos, words,
                                                ops.norm_code(p), float(eps), l.data_ptr(), u.data_ptr(),
                                                viol.data_ptr(), self._ws.data_ptr(), need,
                                                torch.cuda.current_stream().cuda_stream), "fb_encoder_forward_f32")
        return l, u, viol

    def forward_instances(self, emb, positions, p, eps, out=None):
        """The pass for S independent verification instances: emb [S, L, D], positions [S, words] (int32) and
        eps [S] (float32), all on the device.  Returns (l, u, violation) like forward()."""
        ops._chk(emb, eps)
        S, L, D = emb.shape
        if positions.dtype != torch.int32 or not positions.is_cuda or not positions.is_contiguous() or positions.dim() != 2 \
                or positions.shape[0] != S or eps.shape != (S,):
            raise ValueError("positions must be a contiguous int32 CUDA tensor [S, words] and eps a float32 tensor [S]")
        words = positions.shape[1]
        need = self.workspace_bytes(S, L, words)
        if self._ws is None or self._ws.numel() < need:
            self._ws = None
            self._ws = torch.empty(need, dtype=torch.uint8, device=self.device)
        if out is None:
            out = (torch.empty(S, device=self.device), torch.empty(S, device=self.device),
                   torch.empty(1, dtype=torch.int32, device=self.device))
        l, u, viol = out
        with torch.cuda.device(self.device):
            check(load().fb_encoder_forward_instances_f32(ctypes.byref(self._enc), emb.data_ptr(), S, L, positions.data_ptr(),
                                                          eps.data_ptr(), words, ops.norm_code(p), l.data_ptr(), u.data_ptr(),
                                                          viol.data_ptr(), self._ws.data_ptr(), need,
                                                          torch.cuda.current_stream().cuda_stream),
                  "fb_encoder_forward_instances_f32")
        return l, u, viol
