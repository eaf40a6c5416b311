"""Pre-norm layers around a float32 residual stream that is joined over depth.

Level 0 of the history is the token embedding (``X_0``); layer ``i`` files its result as level ``i + 1``:

    x1 = x + m * mixer(norm1(x)),   X_(i+1) = x1 + m * feed_forward(norm2(x1)),   x <- sum_(j <= i+1) a_i[j] X_j

where ``m`` is a constant of the model and ``a_i`` the layer's ``i + 2`` learnt weights.  The layer results
live in one buffer ``[levels, tokens, width]`` (``DepthStream.history``).  What touches a row between two
sublayers is one kernel (``ops.depth_step``): the sum that closes a sublayer, at a layer's end the filing of
the result and the weighted sum over depth, and the norm that opens the next sublayer.  So a sublayer's
output stays ``Open`` until the next sublayer, or the model's end, takes it.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops
from .base import ParamSpec, Part, bytes_of


class DepthAverage(Part):
    """The ``levels`` weights of one layer's sum over depth and the constant its sublayers' outputs are
    multiplied by (family ``connection``)."""

    def param_specs(self):
        return {"weights": ParamSpec((self.spec.levels,), "stream_weight")}

    def set_params(self, params):
        self.weights = params["weights"].float().contiguous()

    def weight_bytes(self):
        return bytes_of(self.weights)


@dataclass
class DepthStream:
    """The residual stream of one step: ``history[j]`` holds ``X_j`` for all tokens, ``x`` the rows the next
    sublayer reads and adds onto (``history[0]`` before the first layer, then one of the two spare buffers)."""

    history: torch.Tensor      # float32 [levels, T, H]
    x: torch.Tensor            # float32 [T, H]
    spare: list                # two float32 [T, H] buffers; the one that is not ``x`` is free

    def free(self):
        return self.spare[1] if self.x.data_ptr() == self.spare[0].data_ptr() else self.spare[0]


@dataclass
class Open:
    """A sublayer's output not yet added onto the stream: ``value * mult`` is to be added to ``stream.x``; with
    ``mix`` the sum closes a layer (it is filed as the layer's result and the stream is summed over depth)."""

    value: object
    mult: float
    mix: object = None


def open_stream(tokens, table, levels, status):
    """The stream at a step's start: the embedding output as ``history[0]`` (the step's fence)."""
    n, hidden = tokens.shape[0], table.shape[1]
    history = torch.empty((levels, n, hidden), dtype=torch.float32, device=table.device)
    ops.embedding32(tokens, table, 1.0, status, fence=True, out=history[0])
    spare = [torch.empty((n, hidden), dtype=torch.float32, device=table.device) for _ in range(2)]
    return DepthStream(history, history[0], spare)


def open_sublayer(stream, pending, norm, dtype):
    """Take ``pending`` (an ``Open`` or None) into the stream and return ``norm`` of the new rows in ``dtype``."""
    if pending is None:
        return ops.depth_step(stream.x, dtype, norm=norm.for_kernel())
    dst = stream.free()
    out = ops.depth_step(stream.x, dtype, pending.value, pending.mult, stream.history, pending.mix, dst,
                         norm.for_kernel())
    stream.x = dst
    return out


def close_rows_depth(stream, pending, rows, norm, dtype):
    """The model's end for the rows asked for: the last open sum (and sum over depth) and the final norm; the
    stream is left as it was."""
    if pending is None:
        return ops.depth_step(stream.x, dtype, norm=norm.for_kernel(), rows=rows)
    return ops.depth_step(stream.x, dtype, pending.value, pending.mult, stream.history, pending.mix, None,
                          norm.for_kernel(), rows=rows)


class DepthPreNormBlock:
    FAMILIES = {"mixer": "mixer", "feed_forward": "feed_forward", "norm1": "norm", "norm2": "norm",
                "connection": "connection"}
    #: what the model makes the residual stream of: a ``DepthStream`` from ``open_stream``
    residual_kind = "depth"

    def __init__(self, parts: dict):
        self._parts = dict(parts)
        self.mixer = parts["mixer"]
        self.feed_forward = parts.get("feed_forward")
        self.norm1, self.norm2 = parts["norm1"], parts.get("norm2")
        self.connection = parts["connection"]
        for norm in (self.norm1, self.norm2):
            if norm is not None and not hasattr(norm, "for_kernel"):
                raise ValueError("the depth arrangement fuses norms that state (kind, gain, eps); got " + repr(norm.spec))

    def parts(self) -> dict:
        return dict(self._parts)

    @property
    def levels(self) -> int:
        return self.connection.spec.levels

    def __call__(self, stream, pending, ctx, entry, writes_cache=True):
        dtype = self.mixer.dtype
        mult = self.connection.spec.multiplier
        if stream.history.shape[0] < self.levels:
            raise ValueError(f"this layer sums over {self.levels} levels; the stream holds {stream.history.shape[0]}")
        n = open_sublayer(stream, pending, self.norm1, dtype)
        a = self.mixer(n, ctx, entry, writes_cache)
        if self.feed_forward is None:
            return stream, Open(a, mult, self.connection.weights)
        m = open_sublayer(stream, Open(a, mult), self.norm2, dtype)
        return stream, Open(self.feed_forward(m, ctx), mult, self.connection.weights)


class DepthMixerOnlyBlock(DepthPreNormBlock):
    """The same layer without a feed-forward (and so without the second norm)."""

    FAMILIES = {"mixer": "mixer", "norm1": "norm", "connection": "connection"}
