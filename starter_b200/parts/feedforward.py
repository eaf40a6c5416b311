"""Dense gated feed-forward: ``down(round(act(gate(x))) * up(x))`` with silu or tanh-approximated gelu,
no biases, no routing."""

from __future__ import annotations

import torch

from .. import ops
from .base import ParamSpec, Part, bytes_of


class GatedFeedForward(Part):
    """gate and up are stored stacked as one ``[2 * I, H]`` matrix so one product feeds both
    (engine/engine.py:163, 464-468, 735)."""

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        if spec.activation not in ops.ACTIVATIONS:
            raise ValueError(f"the gated feed-forward kernels implement {', '.join(ops.ACTIVATIONS)}, "
                             f"not {spec.activation!r}")

    def param_specs(self):
        h, i = self.spec.hidden_size, self.spec.intermediate_size
        return {"gate": ParamSpec((i, h)), "up": ParamSpec((i, h)), "down": ParamSpec((h, i))}

    def set_params(self, params):
        self.gate_up = torch.cat([params["gate"], params["up"]], dim=0).contiguous()
        self.down = params["down"].contiguous()

    adds_to_stream = True

    def __call__(self, x, ctx=None, add_to=None):
        status = ctx.status if ctx is not None else None
        act = ops.linear(x, self.gate_up, gated=self.spec.activation, status=status)
        return ops.linear(act, self.down, status=status, add_to=add_to)

    def weight_bytes(self):
        return bytes_of(self.gate_up, self.down)


class ClampedGatedFeedForward(Part):
    """``down(g * sigmoid(1.702 g) * (u + 1))`` with ``g = min(gate(x), limit)``, ``u = clamp(up(x), -limit,
    limit)``; gate and up are stored stacked so that one product feeds both."""

    def param_specs(self):
        h, i = self.spec.hidden_size, self.spec.intermediate_size
        return {"gate": ParamSpec((i, h)), "up": ParamSpec((i, h)), "down": ParamSpec((h, i))}

    def set_params(self, params):
        self.gate_up = torch.cat([params["gate"], params["up"]], dim=0).contiguous()
        self.down = params["down"].contiguous()

    def __call__(self, x, ctx=None):
        status = ctx.status if ctx is not None else None
        act = ops.linear_gated_clamped(x, self.gate_up, self.spec.limit, status=status)
        return ops.linear(act, self.down, status=status)

    def weight_bytes(self):
        return bytes_of(self.gate_up, self.down)


class BiasedFeedForward(Part):
    """``down(act(up(x) + b_up)) + b_down`` with the activation of the spec (``relu2``: the square of relu).
    The down bias can be left to whoever writes the output to the residual stream (``defer_bias``)."""

    can_defer_bias = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        if spec.activation not in ops.BIAS_ACTIVATIONS:
            raise ValueError(f"the biased feed-forward implements relu2 and tanh, not {spec.activation!r}")
        self.deferred_bias = None

    def param_specs(self):
        h, i = self.spec.hidden_size, self.spec.intermediate_size
        if not getattr(self.spec, "bias", True):
            return {"up": ParamSpec((i, h)), "down": ParamSpec((h, i))}
        return {"up": ParamSpec((i, h)), "up_bias": ParamSpec((i,), "bias32"),
                "down": ParamSpec((h, i)), "down_bias": ParamSpec((h,), "bias32")}

    def set_params(self, params):
        self.up, self.down = params["up"].contiguous(), params["down"].contiguous()
        self.up_bias = self.deferred_bias = None
        if getattr(self.spec, "bias", True):
            self.up_bias = params["up_bias"].float().contiguous()
            self.deferred_bias = params["down_bias"].float().contiguous()

    def __call__(self, x, ctx=None, defer_bias=False):
        status = ctx.status if ctx is not None else None
        act = ops.bias_act(ops.linear(x, self.up, status=status), self.up_bias, self.spec.activation)
        y = ops.linear(act, self.down, status=status)
        return y if defer_bias or self.deferred_bias is None else ops.bias_act(y, self.deferred_bias, None)

    def weight_bytes(self):
        return bytes_of(self.up, self.up_bias, self.down, self.deferred_bias)


class RoutedExperts(Part):
    """A mixture of small experts: the router's logits in 32-bit, the ``top`` largest, their weights by the
    spec's ``scoring``; the chosen experts of all tokens run as tiles grouped by expert (``ops.moe_experts``),
    without a word from the host, so the part also runs inside a captured step.  The experts are gated and
    clamped, or (``expert = "relu2"``) an up and a down projection around a squared relu."""

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        if spec.top > spec.experts + getattr(spec, "identity_experts", 0):
            raise ValueError(f"{spec.top} choices among {spec.experts} experts")
        if spec.expert not in ops.MOE_EXPERTS or spec.scoring not in ops.MOE_SCORINGS:
            raise ValueError(f"no routed experts of kind {spec.expert!r} with scoring {spec.scoring!r}")
        self.gated = spec.expert in ("gated_clamped", "gated_silu")
        self.all_scores = spec.scoring == "softmax_all"
        if not self.all_scores and (spec.correction or spec.group_count != 1 or spec.identity_experts):
            raise ValueError("a correction, groups and identity experts belong to the router that scores by the softmax "
                             "over all its outputs")
        if self.all_scores and spec.router_bias:
            raise ValueError("the router that scores by the softmax over all its outputs has no bias")
        self.outputs = spec.experts + spec.identity_experts
        if self.outputs % spec.group_count or spec.group_keep > spec.group_count:
            raise ValueError(f"{self.outputs} router outputs do not form {spec.group_count} equal groups of which "
                             f"{spec.group_keep} are kept")
        #: the experts chosen in the latest call (int32 ``[T, top]``, on the device), for whoever wants to
        #: look at the routing
        self.last_ids = None

    def param_specs(self):
        s = self.spec
        out = {"router": ParamSpec((self.outputs, s.hidden_size), "matrix32")}
        if s.router_bias:
            out["router_bias"] = ParamSpec((s.experts,), "bias32")
        if s.correction:
            out["correction"] = ParamSpec((self.outputs,), "bias32")
        if s.shared_size:
            out["shared_gate"] = ParamSpec((s.shared_size, s.hidden_size))
            out["shared_up"] = ParamSpec((s.shared_size, s.hidden_size))
            out["shared_down"] = ParamSpec((s.hidden_size, s.shared_size))
            out["shared_sg"] = ParamSpec((1, s.hidden_size), "matrix32")
        for e in range(s.experts):
            if self.gated:
                out[f"e{e}_gate"] = ParamSpec((s.intermediate_size, s.hidden_size))
            out[f"e{e}_up"] = ParamSpec((s.intermediate_size, s.hidden_size))
            out[f"e{e}_down"] = ParamSpec((s.hidden_size, s.intermediate_size))
        return out

    def set_params(self, params):
        s = self.spec
        self.router = params["router"].float().contiguous()
        self.router_bias = params["router_bias"].float().contiguous() if s.router_bias else None
        if self.gated:
            self.gate_up = torch.stack([torch.cat([params[f"e{e}_gate"], params[f"e{e}_up"]], dim=0)
                                        for e in range(s.experts)]).contiguous()
        else:
            self.gate_up = torch.stack([params[f"e{e}_up"] for e in range(s.experts)]).contiguous()
        self.down = torch.stack([params[f"e{e}_down"] for e in range(s.experts)]).contiguous()
        self.correction = params["correction"].float().contiguous() if s.correction else None
        self.shared_gate_up = self.shared_down = None
        if s.shared_size:
            # the shared expert's gate vector rides along as one more row of the router
            self.router = torch.cat([self.router, params["shared_sg"].float().reshape(1, -1)], dim=0).contiguous()
            self.shared_gate_up = torch.cat([params["shared_gate"], params["shared_up"]], dim=0).contiguous()
            self.shared_down = params["shared_down"].contiguous()

    def __call__(self, x, ctx=None):
        s = self.spec
        status = ctx.status if ctx is not None else None
        if not self.all_scores:
            ids, weights = ops.moe_route(x, self.router, self.router_bias, s.top, s.scoring, s.weight_scale)
            self.last_ids = ids
            return ops.moe_experts(x, ids, weights, self.gate_up, self.down, s.limit, s.expert, status=status)
        routed = ops.moe_route_all(x, self.router, self.correction, s.top, s.group_count, s.group_keep, s.weight_scale,
                                   shared_gate=bool(s.shared_size))
        ids, weights = routed[0], routed[1]
        self.last_ids = ids
        shared = None
        if s.shared_size:
            act = ops.linear(x, self.shared_gate_up, gated="silu", status=status)
            shared = ops.linear(act, self.shared_down, status=status)
        return ops.moe_experts(x, ids, weights, self.gate_up, self.down, s.limit, s.expert, status=status,
                               identity=bool(s.identity_experts), shared=shared,
                               shared_gate=routed[2] if s.shared_size else None)

    def weight_bytes(self):
        """What a step reads at most: the router and every expert (a step of few tokens reads only the
        experts they choose)."""
        return bytes_of(self.router, self.router_bias, self.gate_up, self.down, self.correction, self.shared_gate_up,
                        self.shared_down)
