"""Attention over a cached latent (multi-head latent attention).  A token's keys and values of
all heads are functions of one small row, which is all the cache keeps:

    [c' | kr] = Wdkv h;   c = c' / sqrt(mean(c'^2) + eps) * w_c  [rank];   kr rotated  [rot_dim]
    head i:   key = [Wuk_i c | kr],   value = Wuv_i c,   query = [qa_i | rot(qr_i)] = Wq h
    score = scale (qa_i . Wuk_i c + qr_i . kr),  causal softmax,  o_i = sum_j p_j Wuv_i c_j

The rotation turns neighbouring pairs (2i, 2i+1) by position * base^(-2i/rot_dim).  The
concatenated heads are multiplied by sigmoid(Wg h) and projected by Wo.  Since
qa_i . Wuk_i c = (Wuk_i^T qa_i) . c and sum_j p_j Wuv_i c_j = Wuv_i sum_j p_j c_j, the attention
kernels run with ONE key/value head whose rows are the cached rows [c | kr] themselves, as keys
and as values (a cache need with ``values=False``): queries are moved into the latent space
before, the mixed latent is expanded by Wuv after.  ``shared``: the layer has no Wdkv and reads
the rows that another run entry cached (and that entry's rows of this step).

Scores, softmax weights and the weighted sum are 32-bit (the library's exact attention kernels);
the cache rows, q' and the mixed latent are in the compute type.
"""
from __future__ import annotations

import torch

from ..cache import CacheNeed
from ..csrc import ops
from ..weights import TensorNeed
from .attention import exact_attention
from .base import register_mixer
from .linear import matmul_partials


@register_mixer("latent_attention")
class LatentAttention:
    def __init__(self, params: dict, rt):
        self.rt = rt
        self.D = int(params["hidden_size"])
        self.H = int(params["num_heads"])
        self.dim = int(params["head_dim"])            # unrotated query/key features per head
        self.rd = int(params["rot_dim"])              # rotated features, shared by the heads' keys
        self.vdim = int(params["value_dim"])
        self.rank = int(params["kv_rank"])
        self.scale = float(params["scale"])
        self.base = float(params["rot_base"])
        self.eps = float(params["eps"])
        self.owns_latent = bool(params.get("owns_latent", True))
        if min(self.H, self.dim, self.vdim, self.rank) <= 0 or self.rd < 0 or self.rd % 2:
            raise ValueError("latent_attention: heads, sizes and rank must be positive, rot_dim even")
        # the one head size of the attention kernels: a cached row, padded
        self.hd = -(-(self.rank + self.rd) // 16) * 16
        if self.hd > 256:
            raise ValueError(f"latent_attention: kv_rank + rot_dim = {self.rank + self.rd} exceeds the attention "
                             f"kernels' largest head size (256)")
        if self.dim + self.rd > 1024 or self.rank > 1024:
            raise ValueError("latent_attention: dim + rot_dim and kv_rank up to 1,024")
        f = [self.base ** (-2.0 * i / self.rd) for i in range(self.rd // 2)] or [0.0]
        self.freq = torch.tensor(f, dtype=torch.float64).to(torch.float32).to(rt.device)
        self.w_q = self.w_dkv = self.c_norm = self.w_uk = self.w_uv = self.w_g = self.w_o = None

    def tensor_needs(self):
        H, D = self.H, self.D
        needs = {"q": TensorNeed((H * (self.dim + self.rd), D)), "uk": TensorNeed((H * self.dim, self.rank)),
                 "uv": TensorNeed((H * self.vdim, self.rank)), "g": TensorNeed((H * self.vdim, D)),
                 "o": TensorNeed((D, H * self.vdim))}
        if self.owns_latent:
            needs["dkv"] = TensorNeed((self.rank + self.rd, D))
            needs["dkv.norm"] = TensorNeed((self.rank,), init="ones")
        return needs

    def bind(self, tensors) -> None:
        rt = self.rt
        self.w_q = rt.matrix(tensors["q"])
        self.w_g = rt.matrix(tensors["g"])
        self.w_o = rt.matrix(tensors["o"])
        # [H, dim, rank] as stored; the value expansion transposed to [H, rank, vdim]
        self.w_uk = rt.matrix(tensors["uk"])
        self.w_uv = rt.matrix(tensors["uv"].view(self.H, self.vdim, self.rank).transpose(1, 2).contiguous())
        if self.owns_latent:
            self.w_dkv = rt.matrix(tensors["dkv"])
            self.c_norm = rt.vector(tensors["dkv.norm"])

    def cache_need(self):
        return CacheNeed("kv", kv_heads=1, head_dim=self.hd, window=None, values=False) if self.owns_latent else None

    prefers_longest_first = True

    def cache_read_bytes(self, contexts, element_size: int) -> int:
        return sum(contexts) * self.hd * element_size

    def flops(self, q_lens, past) -> float:
        n = sum(q_lens)
        H, D = self.H, self.D
        lin = 2.0 * n * (H * (self.dim + self.rd) * D + 2 * H * self.vdim * D
                         + ((self.rank + self.rd) * D if self.owns_latent else 0)
                         + H * self.dim * self.rank + H * self.vdim * self.rank)
        pairs = sum(q * p + q * (q + 1) // 2 for q, p in zip(q_lens, past))
        return lin + 2.0 * H * (2 * self.rank + self.rd) * pairs

    def forward(self, h, batch, stream, view, shared: bool = False):
        rt, H, hd = self.rt, self.H, self.hd
        n = batch.n_tokens
        if shared != (not self.owns_latent):
            raise RuntimeError("latent_attention: a layer without a down projection reads another run's cache")
        q, qS = matmul_partials(rt, h, self.w_q, "latent_q")
        gate, gS = matmul_partials(rt, h, self.w_g, "latent_gate")
        kv_step = view.kv_step if getattr(view, "kv_step", None) is not None else \
            rt.buffer("latent_step", (n, 2, 1, hd), rt.dtype)
        if not shared:
            dkv, dS = matmul_partials(rt, h, self.w_dkv, "latent_dkv")
            ops.latent_store(dkv, dS, self.c_norm, self.eps, self.freq, batch, view.slot_pos, kv_step, view.k,
                             self.rank, self.rd, hd, view.capacity, pages=view.pages)
        q_lat = rt.buffer("latent_q_abs", (n, H * hd), rt.dtype)
        ops.latent_absorb_q(q, qS, self.w_uk, self.freq, batch, view.slot_pos, q_lat, H, self.dim, self.rd,
                            self.rank, hd)
        o_lat = rt.buffer("latent_mixed", (n, H * hd), rt.dtype)
        exact_attention(rt, q_lat, kv_step, view.k, view.k, batch, view.slot_pos, o_lat, H, 1, hd,
                        view.capacity, None, view.pages, self.scale)
        o = rt.buffer("attn_out", (n, H * self.vdim), rt.dtype)
        ops.latent_expand(o_lat, self.w_uv, gate, gS, o, H, self.rank, self.vdim, hd)
        stream.add_linear(o, self.w_o)
        return None
