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


@register_block("prepost_norm")
class PrePostNormBlock:
    """Every sublayer is normed before AND after: x <- x + post(f(pre(x))), for the mixer, then the
    feed-forward (optional), then an optional third sublayer ``extra`` that reads x itself (no norm
    before it) and is normed after.  The norms after a sublayer hand their form to the stream
    (``ResidualStream.post_norm``), which performs the write together with the next read; the parts
    are ``mixer_norm``, ``mixer``, ``mixer_post_norm``, ``feed_forward_norm``, ``feed_forward``,
    ``feed_forward_post_norm``, ``extra``, ``extra_post_norm``."""

    def __init__(self, layer_spec, rt):
        self.spec = layer_spec
        self.rt = rt
        self.mixer_norm = make_part(NORMS, layer_spec.part("mixer_norm"), rt)
        self.mixer = make_part(MIXERS, layer_spec.part("mixer"), rt)
        self.mixer_post = make_part(NORMS, layer_spec.part("mixer_post_norm"), rt)
        self.ffn = self.ffn_norm = self.ffn_post = self.extra = self.extra_post = None
        if "feed_forward" in layer_spec.parts:
            self.ffn_norm = make_part(NORMS, layer_spec.part("feed_forward_norm"), rt)
            self.ffn = make_part(FEED_FORWARDS, layer_spec.part("feed_forward"), rt)
            self.ffn_post = make_part(NORMS, layer_spec.part("feed_forward_post_norm"), rt)
        if "extra" in layer_spec.parts:
            self.extra = make_part(FEED_FORWARDS, layer_spec.part("extra"), rt)
            self.extra_post = make_part(NORMS, layer_spec.part("extra_post_norm"), rt)
        for n in (self.mixer_post, self.ffn_post, self.extra_post):
            if n is not None and not hasattr(n, "form"):
                raise TypeError("a prepost_norm block needs output norms that give their form (dynamic_tanh, rmsnorm)")

    def parts(self):
        s = self.spec
        names = ["mixer_norm", "mixer", "mixer_post_norm"]
        if self.ffn is not None:
            names += ["feed_forward_norm", "feed_forward", "feed_forward_post_norm"]
        if self.extra is not None:
            names += ["extra", "extra_post_norm"]
        built = {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "mixer_post_norm": self.mixer_post,
                 "feed_forward_norm": self.ffn_norm, "feed_forward": self.ffn,
                 "feed_forward_post_norm": self.ffn_post, "extra": self.extra, "extra_post_norm": self.extra_post}
        return [(built[n], s.part(n)) for n in names]

    def mixers(self):
        return {"mixer": self.mixer}

    def forward(self, stream, batch, views, shared: bool = False):
        from ..csrc import ops
        stream.hold = True
        try:
            h = self.mixer_norm(stream)
            later = self.mixer.forward(h, batch, stream, views["mixer"], shared=shared)
            stream.post_norm(self.mixer_post.form())
            if self.ffn is not None:
                h = self.ffn_norm(stream)
                self.ffn.forward(h, batch, stream)
                stream.post_norm(self.ffn_post.form())
            if self.extra is not None:
                # the third sublayer reads the stream as it is, in the compute type
                h = self.rt.buffer("stream_input", tuple(stream.x.shape), self.rt.dtype)
                stream.read_norm((ops.NORM_NONE, None, None, 0.0, 0.0), h)
                self.extra.forward(h, batch, stream)
                stream.post_norm(self.extra_post.form())
        finally:
            stream.hold = False
        return later
