"""Two mixers side by side that read the same input: the result is half the sum of their outputs, each first
RMS-normed over the model width with a plain gain of its own (``ops.norm_pair_mean``).

The two sides are built from their own specs through the registry, so any mixer can stand on either side.  The
layer's cache entry serves both: at most one side may keep keys and values, at most one a per-sequence state.
"""

from __future__ import annotations

from .. import ops
from .base import ParamSpec, Part, bytes_of


class ParallelMixer(Part):
    SIDES = ("left", "right")

    def __init__(self, spec, dtype, position=None):
        super().__init__(spec, dtype)
        from .registry import lookup

        self.sides = {}
        for name in self.SIDES:
            side = getattr(spec, name)
            wants = getattr(side, "position", None) is not None
            self.sides[name] = lookup("mixer", side.kind)(side, dtype, position if wants else None)
        if sum(m.kv_need() is not None for m in self.sides.values()) > 1:
            raise ValueError("both sides of a parallel mixer keep keys and values; a layer has one cache entry")
        if sum(m.state_need() is not None for m in self.sides.values()) > 1:
            raise ValueError("both sides of a parallel mixer keep a per-sequence state; a layer has one")

    def kv_need(self):
        return next((n for n in (m.kv_need() for m in self.sides.values()) if n is not None), None)

    def state_need(self):
        return next((n for n in (m.state_need() for m in self.sides.values()) if n is not None), None)

    def param_specs(self):
        out = {}
        for name, mixer in self.sides.items():
            out.update({f"{name}.{k}": v for k, v in mixer.param_specs().items()})
            out[f"{name}_out"] = ParamSpec((self.spec.hidden_size,), "gain32")
        return out

    def set_params(self, params):
        for name, mixer in self.sides.items():
            mixer.set_params({k[len(name) + 1:]: v for k, v in params.items() if k.startswith(name + ".")})
        self.gains = {name: params[f"{name}_out"].float().contiguous() for name in self.sides}

    def prepare(self, max_position: int) -> bool:
        moved = False
        for mixer in self.sides.values():
            moved = bool(mixer.prepare(max_position)) or moved
        return moved

    def __call__(self, x, ctx, entry, writes_cache=True):
        left, right = (self.sides[n](x, ctx, entry, writes_cache) for n in self.SIDES)
        return ops.norm_pair_mean(left, right, self.gains["left"], self.gains["right"], self.spec.norm_eps)

    def weight_bytes(self):
        return sum(m.weight_bytes() for m in self.sides.values()) + bytes_of(*self.gains.values())
