"""How a layer's parts are arranged around the residual stream.

``PreNormBlock``: ``x1 = x + mixer(norm1(x))``, ``x2 = x1 + feed_forward(norm2(x1))``
(engine/engine.py:665-736).  Every residual sum is followed at once by a norm, so
the two are one kernel: a block takes ``(residual, pending)``, where ``pending``
is the previous block's output not yet added, and returns the same pair
(engine/engine.py:669-673).  The model's final norm closes the chain the same way.
A block does not know its neighbours or the model it is in.

A mixer or feed-forward that sets ``adds_to_stream = True`` is called with ``add_to=residual``: it
may add its output onto that tensor itself (in the epilogue of its last product) and return
``ops.ADDED`` instead of the output; the norm that follows then only norms.

An arrangement says which parts it is made of: ``FAMILIES`` maps each part's name inside the layer
to the family its spec is looked up in.  The model builds exactly those parts from the layer spec
and hands them over by name; ``mixer`` names the part that owns the layer's cache entry.
"""

from __future__ import annotations

from dataclasses import dataclass

from .. import ops


class PreNormBlock:
    FAMILIES = {"mixer": "mixer", "feed_forward": "feed_forward", "norm1": "norm", "norm2": "norm"}

    def __init__(self, parts: dict):
        self._parts = dict(parts)
        self.mixer = parts["mixer"]
        self.feed_forward = parts["feed_forward"]
        self.norm1 = parts["norm1"]
        self.norm2 = parts["norm2"]

    def parts(self) -> dict:
        return dict(self._parts)

    def __call__(self, residual, pending, ctx, entry, writes_cache=True):
        n = self.norm1.add(residual, pending)
        if getattr(self.mixer, "adds_to_stream", False):
            a = self.mixer(n, ctx, entry, writes_cache, add_to=residual)
        else:
            a = self.mixer(n, ctx, entry, writes_cache)
        m = self.norm2.add(residual, a)
        if getattr(self.feed_forward, "adds_to_stream", False):
            return residual, self.feed_forward(m, ctx, add_to=residual)
        return residual, self.feed_forward(m, ctx)


@dataclass
class Summand:
    """A sublayer's output not yet added onto a float32 residual stream (it is added as it is)."""

    value: object
    eps: float = 0.0

    def for_kernel(self):
        return self.value, None, None, self.eps


class PreNorm32Block:
    """The same layer around a residual stream that is a 32-bit sum whatever the working type: ``x <- x +
    mixer(norm1(x))``, then ``x <- x + feed_forward(norm2(x))``.  The sum that closes one sublayer and the norm
    that opens the next are one kernel (``ops.residual_norm``): a sublayer's output stays a ``Summand`` until the
    next sublayer, or the model's end, takes it."""

    FAMILIES = {"mixer": "mixer", "feed_forward": "feed_forward", "norm1": "norm", "norm2": "norm"}
    #: what the model makes the residual stream of: float32 rows from ``ops.embedding32``
    residual_kind = "float32"

    def __init__(self, parts: dict):
        self._parts = dict(parts)
        self.mixer = parts["mixer"]
        self.feed_forward = parts.get("feed_forward")
        self.norm1, self.norm2 = parts["norm1"], parts.get("norm2")
        for norm in (self.norm1, self.norm2):
            if norm is not None and getattr(norm.spec, "kind", None) != "rmsnorm":
                raise ValueError("the 32-bit pre-norm arrangement fuses RMS norms; got " + repr(norm.spec))
            if norm is not None and not (norm.spec.gain_32bit or norm.spec.unit_offset):
                raise ValueError("the 32-bit pre-norm arrangement needs norms whose gains are held in float32")

    def parts(self) -> dict:
        return dict(self._parts)

    def _open(self, residual, pending, norm):
        return ops.residual_norm(residual, self.mixer.dtype, norm.spec.eps,
                                 pending.for_kernel() if pending is not None else None, norm.weight)

    def __call__(self, residual, pending, ctx, entry, writes_cache=True):
        n = self._open(residual, pending, self.norm1)
        pending = Summand(self.mixer(n, ctx, entry, writes_cache))
        if self.feed_forward is None:
            return residual, pending
        m = self._open(residual, pending, self.norm2)
        return residual, Summand(self.feed_forward(m, ctx))


class PreNorm32MixerOnlyBlock(PreNorm32Block):
    """The same layer without a feed-forward (and so without the second norm)."""

    FAMILIES = {"mixer": "mixer", "norm1": "norm"}
