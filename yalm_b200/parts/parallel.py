"""Mixers side by side: every branch is a mixer of its own kind that reads the same input;
the result is ``scale`` times the sum of the branches' outputs, each first normed over the
model width (n(y, w) = y / sqrt(mean(y^2) + eps) * w) with a weight of its own.

The branches' norms are not launches of their own: each branch leaves the slices of its
output product with its weight on the residual stream (``ResidualStream.add_branches``), and
the norm of the block that holds the sum (``sum_rmsnorm``) norms, scales and adds them while it
forms the residual sum.  The block must therefore be one that norms after the sum.

params: ``hidden_size``, ``eps``, ``scale``, ``branches`` = [(name, PartSpec), ...]; a branch's
tensors are the keys of its own part prefixed with "<name>.", and its norm weight is
"<name>.out".  Cache needs of the branches are passed through under "<name>.<need name>".

``branch_norm`` False: the branches are not normed; the result is sum_b scales[b] * branch_b
(``scales``: one factor per branch, default ``scale`` for each), left on the stream for a block
whose own norm takes the sum (``sum_rmsnorm``, or the output norm of a ``prepost_norm`` block).
"""
from __future__ import annotations

from ..cache.storage import normalise_needs
from ..weights import TensorNeed
from .base import MIXERS, make_part, register_mixer
from .linear import matmul_partials


class _BranchStream:
    """What a branch's mixer sees in place of the residual stream: its output product is kept
    apart, as slices in a buffer of the branch's own."""

    def __init__(self, rt, name: str):
        self.rt, self.name = rt, name
        self.slices, self.n = None, 0

    def add_linear(self, a, w) -> None:
        if self.n:
            raise RuntimeError(f"branch {self.name!r} added a second output")
        self.slices, self.n = matmul_partials(self.rt, a, w, f"branch_out_{self.name}")


@register_mixer("parallel_branches")
class ParallelBranches:
    def __init__(self, params: dict, rt):
        self.rt = rt
        self.D = int(params["hidden_size"])
        self.eps = float(params["eps"])
        self.scale = float(params.get("scale", 1.0))
        self.branch_norm = bool(params.get("branch_norm", True))
        self.names = [name for name, _ in params["branches"]]
        self.scales = [float(v) for v in (params.get("scales") or [self.scale] * len(self.names))]
        if len(self.scales) != len(self.names):
            raise ValueError("parallel_branches: one scale per branch")
        if len(self.names) != 2 or len(set(self.names)) != 2:
            raise ValueError("parallel_branches takes two branches with different names")
        self.branches = {name: make_part(MIXERS, spec, rt) for name, spec in params["branches"]}
        self.out_norm = {}

    def tensor_needs(self):
        needs = {}
        for name, part in self.branches.items():
            for key, need in part.tensor_needs().items():
                needs[f"{name}.{key}"] = need
            if self.branch_norm:
                needs[f"{name}.out"] = TensorNeed((self.D,), init="ones")
        return needs

    def bind(self, tensors) -> None:
        for name, part in self.branches.items():
            part.bind({key: tensors[f"{name}.{key}"] for key in part.tensor_needs()})
            self.out_norm[name] = self.rt.vector(tensors[f"{name}.out"]) if self.branch_norm else None

    def cache_need(self):
        needs = {}
        for name, part in self.branches.items():
            for nname, need in normalise_needs(part.cache_need()).items():
                needs[f"{name}.{nname}"] = need
        return needs or None

    @property
    def prefers_longest_first(self) -> bool:
        return any(getattr(p, "prefers_longest_first", False) for p in self.branches.values())

    def cache_read_bytes(self, contexts, element_size: int) -> int:
        return sum(p.cache_read_bytes(contexts, element_size) for p in self.branches.values()
                   if hasattr(p, "cache_read_bytes"))

    def flops(self, q_lens, past) -> float:
        return sum(p.flops(q_lens, past) for p in self.branches.values() if hasattr(p, "flops"))

    def _view_of(self, name: str, part, view):
        """The branch's own view(s) out of this mixer's: one view for a single need, a dict for several."""
        needs = normalise_needs(part.cache_need())
        if not needs:
            return None
        views = view if isinstance(view, dict) else {"cache": view}
        got = {nname: views[f"{name}.{nname}"] for nname in needs}
        return got["cache"] if list(got) == ["cache"] else got

    def forward(self, h, batch, stream, view, shared: bool = False):
        outs, later = [], []
        for name, scale in zip(self.names, self.scales):
            part = self.branches[name]
            bs = _BranchStream(self.rt, name)
            w = part.forward(h, batch, bs, self._view_of(name, part, view), shared=shared)
            if w is not None:
                later.append(w)
            if not bs.n:
                raise RuntimeError(f"branch {name!r} left no output")
            outs.append((bs.slices, bs.n, self.out_norm[name], scale))
        stream.add_branches(outs, self.eps)
        if later:
            return lambda: [w() for w in later]
        return None
