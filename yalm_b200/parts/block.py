"""Arrangements of a layer's parts.  ``prenorm``: x += mixer(norm(x)); then
x += ffn(norm(x)) -- the reference's block order (infer.cpp:257-386).

A block arrangement is a class with ``__init__(layer_spec, rt)`` (it builds the
parts it names from ``layer_spec.parts``), ``parts()`` (the built parts with
their specs, for weight binding), ``mixers()`` (the parts that may ask for cache,
by name) and ``forward(stream, batch, views, shared)``.  ``views`` maps a mixer's
name to what that mixer sees of the cache: one :class:`CacheView`, a dict of them
by need name when the mixer declared several needs, or None.
"""
from __future__ import annotations

from .base import FEED_FORWARDS, MIXERS, NORMS, make_part, register_block


@register_block("prenorm")
class PreNormBlock:
    def __init__(self, layer_spec, rt):
        self.spec = layer_spec
        self.mixer_norm = make_part(NORMS, layer_spec.part("mixer_norm"), rt)
        self.mixer = make_part(MIXERS, layer_spec.part("mixer"), rt)
        # a layer may have no feed-forward: then it is x += mixer(norm(x)) alone
        self.ffn = self.ffn_norm = None
        if "feed_forward" in layer_spec.parts:
            self.ffn_norm = make_part(NORMS, layer_spec.part("feed_forward_norm"), rt)
            self.ffn = make_part(FEED_FORWARDS, layer_spec.part("feed_forward"), rt)

    def parts(self):
        """(part, its PartSpec) pairs, for weight binding."""
        s = self.spec
        out = [(self.mixer_norm, s.part("mixer_norm")), (self.mixer, s.part("mixer"))]
        if self.ffn is not None:
            out += [(self.ffn_norm, s.part("feed_forward_norm")), (self.ffn, s.part("feed_forward"))]
        return out

    def mixers(self):
        """name -> mixer, for the cache's needs."""
        return {"mixer": self.mixer}

    def forward(self, stream, batch, views, shared: bool = False):
        """Returns what the mixer returned: None, or a cache write that the model makes
        once every run entry that reads this entry's cache has run."""
        h = self.mixer_norm(stream)
        later = self.mixer.forward(h, batch, stream, views["mixer"], shared=shared)
        if self.ffn is not None:
            h = self.ffn_norm(stream)
            self.ffn.forward(h, batch, stream)
        return later


@register_block("postnorm")
class PostNormBlock:
    """Norm after the sum: x <- norm1(a x + mixer(x)); x <- norm2(a x + ffn(x)).  The sublayers
    read x itself (in the compute type); the norms are of kind ``sum_rmsnorm``, which own the
    factor a.  The feed-forward and its norm may be absent."""

    def __init__(self, layer_spec, rt):
        self.spec = layer_spec
        self.mixer = make_part(MIXERS, layer_spec.part("mixer"), rt)
        self.mixer_norm = make_part(NORMS, layer_spec.part("mixer_norm"), rt)
        self.ffn = self.ffn_norm = None
        if "feed_forward" in layer_spec.parts:
            self.ffn = make_part(FEED_FORWARDS, layer_spec.part("feed_forward"), rt)
            self.ffn_norm = make_part(NORMS, layer_spec.part("feed_forward_norm"), rt)
        for n in (self.mixer_norm, self.ffn_norm):
            if n is not None and not hasattr(n, "apply"):
                raise TypeError("a postnorm block needs norms that form the sum themselves (sum_rmsnorm)")

    def parts(self):
        s = self.spec
        out = [(self.mixer, s.part("mixer")), (self.mixer_norm, s.part("mixer_norm"))]
        if self.ffn is not None:
            out += [(self.ffn, s.part("feed_forward")), (self.ffn_norm, s.part("feed_forward_norm"))]
        return out

    def mixers(self):
        return {"mixer": self.mixer}

    def forward(self, stream, batch, views, shared: bool = False):
        stream.resolve()
        stream.hold = True
        try:
            later = self.mixer.forward(stream.as_input(), batch, stream, views["mixer"], shared=shared)
            self.mixer_norm.apply(stream)
            if self.ffn is not None:
                self.ffn.forward(stream.as_input(), batch, stream)
                self.ffn_norm.apply(stream)
        finally:
            stream.hold = False
        return later


@register_block("hyper_prenorm")
class HyperPreNormBlock:
    """Pre-norm sublayers over several residual copies: each sublayer reads one mixture of the
    copies through its norm and writes its output into all of them (``hyper_rmsnorm`` owns both).
    The feed-forward and its norm may be absent.  The stream holds the products apart (``hold``)
    so that the write gets them as they are."""

    def __init__(self, layer_spec, rt):
        self.spec = layer_spec
        self.mixer_norm = make_part(NORMS, layer_spec.part("mixer_norm"), rt)
        self.mixer = make_part(MIXERS, layer_spec.part("mixer"), rt)
        self.ffn = self.ffn_norm = None
        if "feed_forward" in layer_spec.parts:
            self.ffn_norm = make_part(NORMS, layer_spec.part("feed_forward_norm"), rt)
            self.ffn = make_part(FEED_FORWARDS, layer_spec.part("feed_forward"), rt)
        for n in (self.mixer_norm, self.ffn_norm):
            if n is not None and not (hasattr(n, "read") and hasattr(n, "write")):
                raise TypeError("a hyper_prenorm block needs norms that read and write the copies (hyper_rmsnorm)")

    def parts(self):
        s = self.spec
        out = [(self.mixer_norm, s.part("mixer_norm")), (self.mixer, s.part("mixer"))]
        if self.ffn is not None:
            out += [(self.ffn_norm, s.part("feed_forward_norm")), (self.ffn, s.part("feed_forward"))]
        return out

    def mixers(self):
        return {"mixer": self.mixer}

    def forward(self, stream, batch, views, shared: bool = False):
        stream.hold = True
        try:
            h = self.mixer_norm.read(stream)
            later = self.mixer.forward(h, batch, stream, views["mixer"], shared=shared)
            self.mixer_norm.write(stream)
            if self.ffn is not None:
                h = self.ffn_norm.read(stream)
                self.ffn.forward(h, batch, stream)
                self.ffn_norm.write(stream)
        finally:
            stream.hold = False
        return later
