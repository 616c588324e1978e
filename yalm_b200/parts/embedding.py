"""Token embedding (x = float(E[token]), infer.cpp:454-475) and the output
head (logits = Wcls x, the embedding matrix when tied, model.cpp:389-398).

``hashed_pair_embedding`` adds a row of a second table chosen by a hash of the previous
and the current token, x = E[tok] + P[(prev * mul_prev + tok * mul_cur) mod buckets], with
the table's last row (number ``buckets``) for a sequence's first token.  The previous
token of a step's first token is part of the sequence's state: the part declares a cache
need of one int32 per sequence, which its kernel reads and keeps up to date.

An embedding's ``forward(batch, view=None, keep_copy=False)`` returns the residual
stream's start x, or (x, a second buffer with the same values) when a later run entry
adds the embedding output again.  The head takes an optional ``softcap``:
logits <- cap * tanh(logits / cap)."""
from __future__ import annotations

import torch

from ..cache import CacheNeed
from ..csrc import ops
from ..weights import TensorNeed
from .base import register_embedding, register_head
from .linear import matmul_store


@register_embedding("embedding")
class Embedding:
    def __init__(self, params: dict, rt):
        self.rt = rt
        self.vocab = int(params["vocab_size"])
        self.size = int(params["size"])
        self.scale = float(params.get("scale") or 1.0)       # x = E[token] * scale
        # "norm" = {"eps": e}: the looked-up row is RMS-normed with a weight ("norm") before it
        # starts the residual stream
        self.norm = params.get("norm") or None
        self.table = None
        self.norm_weight = None

    def tensor_needs(self):
        needs = {"weight": TensorNeed((self.vocab, self.size))}
        if self.norm:
            needs["norm"] = TensorNeed((self.size,), init="ones")
        return needs

    def bind(self, tensors) -> None:
        self.table = self.rt.matrix(tensors["weight"], share=True)
        if self.norm:
            self.norm_weight = self.rt.vector(tensors["norm"])

    def cache_need(self):
        return None

    def forward(self, batch, view=None, keep_copy: bool = False):
        x = self.rt.buffer("residual", (batch.n_tokens, self.size), torch.float32)
        ops.embed(batch.tokens, self.table, x, self.rt.status, scale=self.scale)
        if self.norm:
            ops.sum_norm(x, 1.0, [], self.norm_weight, float(self.norm["eps"]))    # x <- n(x) w, in place
        if keep_copy:
            copy = self.rt.buffer("embedding_output", (batch.n_tokens, self.size), torch.float32)
            copy.copy_(x)
            return x, copy
        return x


@register_embedding("hashed_pair_embedding")
class HashedPairEmbedding:
    def __init__(self, params: dict, rt):
        self.rt = rt
        self.vocab = int(params["vocab_size"])
        self.size = int(params["size"])
        self.buckets = int(params["buckets"])
        self.mul_prev = int(params["mul_prev"])
        self.mul_cur = int(params["mul_cur"])
        if self.buckets <= 0:
            raise ValueError(f"a hashed table needs at least one bucket, got {self.buckets}")
        self.table = None
        self.pair = None

    def tensor_needs(self):
        return {"weight": TensorNeed((self.vocab, self.size)),
                "pair": TensorNeed((self.buckets + 1, self.size))}

    def bind(self, tensors) -> None:
        both = [tensors["weight"], tensors["pair"]]
        if any(t.dtype == torch.float32 for t in both):
            both = [t.to(torch.float32) for t in both]
        self.table = self.rt.matrix(both[0], share=True)
        self.pair = self.rt.matrix(both[1])

    def cache_need(self) -> CacheNeed:
        """The last token the sequence has been given: one int32 per sequence."""
        return CacheNeed("state", state_shape=(1,), state_dtype=torch.int32)

    def forward(self, batch, view=None, keep_copy: bool = False):
        if view is None:
            raise RuntimeError("the hashed embedding needs its per-sequence state from the cache")
        x = self.rt.buffer("residual", (batch.n_tokens, self.size), torch.float32)
        copy = self.rt.buffer("embedding_output", (batch.n_tokens, self.size), torch.float32) \
            if keep_copy else None
        ops.embed_pair(batch, self.table, self.pair, view.state, view.slot_pos, x, copy,
                       self.mul_prev, self.mul_cur, self.rt.status)
        return (x, copy) if keep_copy else x


@register_head("linear_head")
class LinearHead:
    def __init__(self, params: dict, rt):
        self.rt = rt
        self.vocab = int(params["vocab_size"])
        self.size = int(params["size"])
        cap = params.get("softcap")
        self.softcap = None if not cap else float(cap)
        self.weight = None

    def tensor_needs(self):
        return {"weight": TensorNeed((self.vocab, self.size))}

    def bind(self, tensors) -> None:
        self.weight = self.rt.matrix(tensors["weight"], share=True)

    def flops(self, q_lens, past) -> float:
        return 2.0 * sum(q_lens) * self.vocab * self.size

    def forward(self, h: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        matmul_store(self.rt, h, self.weight, out)
        if self.softcap:
            ops.softcap(out, self.softcap)
        return out
