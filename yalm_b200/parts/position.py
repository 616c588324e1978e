"""Position encodings.  A mixer owns one and calls
``rotate_and_store(qkv, n_partials, batch, view, q_out, kv_step, H, G, write_cache)``
after its q/k/v projection: the encoding rotates q and k, and the fused kernel
writes k and v into the cache on the way.

``rope``: pairs (i, i + head_dim/2) of each head are rotated by the angle
pos * inv_freq[i], computed in 32 bits inside the kernel.  The reference rotates
interleaved pairs of weights whose rows its packer permuted (infer.cpp:202-215,
convert.py:145-158); on unpermuted checkpoints that is this half-split pairing.
inv_freq[i] = theta^(-2i/head_dim), optionally rescaled by the llama3 rule
(long wavelengths divided by ``factor``, short ones kept, a linear blend
between), which the reference does not read.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..csrc import ops
from .base import register_position


def llama3_inv_freq(head_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    out = []
    for i in range(0, head_dim, 2):
        f = 1.0 / (float(theta) ** (i / head_dim))
        if scaling is not None:
            factor = float(scaling["factor"])
            low = float(scaling["low_freq_factor"])
            high = float(scaling["high_freq_factor"])
            orig = float(scaling["original_max_position_embeddings"])
            wavelen = 2.0 * math.pi / f
            if wavelen > orig / low:
                f = f / factor
            elif wavelen >= orig / high:
                s = (orig / wavelen - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64).to(torch.float32)


@register_position("none")
class NoPosition:
    """No position encoding: q and k stay as projected.  It runs the rotary kernels with every
    frequency zero (cos 1, sin 0: each rotated pair is exactly the pair that went in), so the
    same fused paths -- the q/k/v product that stores in its epilogue, the decode attention
    that sums the product's slices and writes the cache row -- serve a mixer without
    positions."""

    def __init__(self, params: dict, rt):
        self.rt = rt
        self.head_dim = int(params["head_dim"])
        if self.head_dim % 2:
            raise ValueError(f"the store kernels take an even head size, got {self.head_dim}")
        self.inv_freq = torch.zeros(self.head_dim // 2, dtype=torch.float32, device=rt.device)
        self._table_key = "rope_table_identity_%d" % self.head_dim

    step_table = None              # set below: the same table logic as Rope's

    def rotate_and_store(self, qkv, n_partials, batch, view, q_out, kv_step, H, G,
                         write_cache=True) -> None:
        ops.rope_store(qkv, n_partials, self.inv_freq, batch, q_out, kv_step, view.k, view.v,
                       view.slot_pos, H, G, self.head_dim, view.capacity, write_cache,
                       pages=view.pages)


@register_position("rope")
class Rope:
    def __init__(self, params: dict, rt):
        self.rt = rt
        self.head_dim = int(params["head_dim"])
        if self.head_dim % 2:
            raise ValueError(f"rope needs an even head size, got {self.head_dim}")
        self.inv_freq = llama3_inv_freq(self.head_dim, float(params["theta"]),
                                        params.get("scaling")).to(rt.device)
        scaling = params.get("scaling")
        self._table_key = "rope_table_%d_%r_%r" % (
            self.head_dim, float(params["theta"]),
            None if scaling is None else tuple(sorted((k, str(v)) for k, v in scaling.items())))

    def step_table(self, batch, slot_pos) -> torch.Tensor:
        """(cos, sin) of every token's angle for every pair, float32 [tokens, head_dim/2, 2]:
        made once per step and shared by the layers whose encoding has the same constants,
        for a q/k/v product that rotates and stores in its own epilogue (an encoding
        without this method always gets ``rotate_and_store``)."""
        table = batch.notes.get(self._table_key)
        if table is None:
            table = self.rt.buffer(self._table_key, (batch.n_tokens, self.head_dim // 2, 2),
                                   torch.float32)
            ops.rope_table(self.inv_freq, batch, slot_pos, table)
            batch.notes[self._table_key] = table
        return table

    def rotate_and_store(self, qkv, n_partials, batch, view, q_out, kv_step, H, G,
                         write_cache=True) -> None:
        ops.rope_store(qkv, n_partials, self.inv_freq, batch, q_out, kv_step, view.k, view.v,
                       view.slot_pos, H, G, self.head_dim, view.capacity, write_cache,
                       pages=view.pages)


NoPosition.step_table = Rope.step_table


def yarn_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """Angle per position of the dims/2 rotated pairs, f_i = base^(-2i/dims), and the factor on
    cos and sin.  With ``scaling`` = {factor, original, fast, slow} (YaRN): pairs that turn fewer
    than ``slow`` times over ``original`` positions are slowed down by ``factor``, pairs that
    turn more than ``fast`` times stay, a linear ramp over the pair index between them, and cos
    and sin are multiplied by 0.1 ln(factor) + 1."""
    f = [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]
    mult = 1.0
    if scaling:
        factor, orig = float(scaling["factor"]), float(scaling["original"])
        where = lambda turns: dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))
        lo = max(math.floor(where(float(scaling["fast"]))), 0)
        hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
        for i in range(dims // 2):
            ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
            f[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp)
        mult = 0.1 * math.log(factor) + 1.0
    return torch.tensor(f, dtype=torch.float64).to(torch.float32), mult


@register_position("rope_partial")
class PartialRope:
    """Rotation of the first ``dims`` features of every head (the rest pass unchanged), in pairs
    (i, i + dims/2) (``layout`` "halves") or (2i, 2i + 1) ("neighbours"), by pos * f_i with
    optional YaRN scaling; the angle is formed in 32 bits inside the kernel.  ``scaling`` with
    ``"kind": "llama3"`` (``factor``, ``low_freq_factor``, ``high_freq_factor``,
    ``original_max_position_embeddings``) rescales the frequencies by wavelength bands instead, as the
    ``rope`` encoding does.  Its kernel also
    norms q and k over their whole projections first when the mixer hands it the weights
    (``norms``), takes the values from the keys as projected when the product has no v
    rows (``has_v`` False), and with ``head_norm`` = (eps, size) divides every head of q and k by its
    root mean square after the rotation.  It has no per-step table: the mixer's products stay apart
    from it."""

    def __init__(self, params: dict, rt):
        self.rt = rt
        self.head_dim = int(params["head_dim"])
        self.dims = int(params.get("dims", self.head_dim))
        self.neighbours = params.get("layout", "halves") == "neighbours"
        if params.get("layout", "halves") not in ("halves", "neighbours"):
            raise ValueError(f"rope_partial: layout {params.get('layout')!r} (halves or neighbours)")
        if self.dims % 2 or not 0 <= self.dims <= self.head_dim:
            raise ValueError(f"rope_partial: {self.dims} rotated features of a head of {self.head_dim}")
        scaling = params.get("scaling") or None
        if self.dims and scaling and scaling.get("kind") == "llama3":
            freq, self.mult = llama3_inv_freq(self.dims, float(params["base"]), scaling), 1.0
        elif self.dims:
            freq, self.mult = yarn_frequencies(self.dims, float(params["base"]), scaling)
        else:
            freq, self.mult = torch.zeros(1), 1.0
        self.freq = freq.to(rt.device)

    def rotate_and_store(self, qkv, n_partials, batch, view, q_out, kv_step, H, G, write_cache=True,
                         norms=None, has_v=True, bias=None, head_norm=None) -> None:
        qn, kn, n_q, n_k, eps = norms if norms is not None else (None, None, 1, 1, 0.0)
        ops.qk_norm_rope_store(qkv, n_partials, qn, kn, n_q, n_k, eps, self.freq, self.dims,
                               self.neighbours, self.mult, batch, q_out, kv_step, view.k, view.v,
                               view.slot_pos, H, G, self.head_dim, has_v, view.capacity, write_cache,
                               pages=view.pages, bias=bias, head_norm=head_norm)
