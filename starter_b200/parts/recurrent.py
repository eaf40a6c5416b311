"""Recurrent mixers whose state lives in the cache's per-sequence slots, each behind a short causal convolution
whose last inputs are part of that state:

* ``GatedLinearRecurrence``: a gated branch times a real-gated linear recurrent unit per channel
  (``ops.short_conv``, a block-diagonal product for the two gates, ``ops.glru_scan``);
* ``StateSpaceMixer``: a selective state-space recurrence with a matrix state per head (``ops.short_conv``,
  ``ops.state_scan`` in its ``state_space`` form, ``ops.group_norm_gate``);
* ``GatedDeltaMixer``: the gated delta rule on unit queries and keys (the same three kernels, the scan in its
  ``gated_delta`` form).

A whole prompt, a later portion and a single token are the same code, and a step captured in a CUDA graph too:
the kernels work from the step's device arrays and the slots.  A slot's floats: the convolution's last ``taps -
1`` inputs of every convolved channel, then the recurrence's state; zero when a sequence opens.
"""

from __future__ import annotations

import torch

from .. import ops
from ..cache.layout import StateNeed
from .base import ParamSpec, Part, bytes_of


def _padded_rows(rows, width):
    """The matrices stacked by rows, with rows of zeros up to a multiple of 8: a token's projections then start
    on a 16-byte boundary whatever the sizes."""
    pad = -sum(r.shape[0] for r in rows) % 8
    if pad:
        rows = list(rows) + [torch.zeros((pad, width), dtype=rows[0].dtype, device=rows[0].device)]
    return torch.cat(list(rows), dim=0).contiguous()


class _Recurrent(Part):
    def __init__(self, spec, dtype, position=None):
        super().__init__(spec, dtype)
        if position is not None:
            raise ValueError(f"{type(self).__name__} takes no position part")

    def kv_need(self):
        return None

    def prepare(self, max_position: int) -> bool:
        return False

    def _state(self, ctx, entry, writes_cache):
        state = ctx.cache.entry_state(entry)
        if state is None or not writes_cache:
            raise ValueError(f"{type(self).__name__} needs a state of its own in the cache")
        return state


class GatedLinearRecurrence(_Recurrent):
    def __init__(self, spec, dtype, position=None):
        super().__init__(spec, dtype, position)
        if spec.width % spec.blocks:
            raise ValueError(f"{spec.width} channels do not split into {spec.blocks} equal blocks")
        self.block = spec.width // spec.blocks

    def state_need(self):
        return StateNeed((self.spec.conv * self.spec.width,), "float32")

    def param_specs(self):
        s, c, b = self.spec, self.spec.width, self.block
        return {
            "y": ParamSpec((c, s.hidden_size)), "y_bias": ParamSpec((c,), "bias32"),
            "x": ParamSpec((c, s.hidden_size)), "x_bias": ParamSpec((c,), "bias32"),
            "conv": ParamSpec((c, s.conv), "vector32"), "conv_bias": ParamSpec((c,), "bias32"),
            "ra": ParamSpec((s.blocks, b, b)), "ra_bias": ParamSpec((s.blocks, b), "bias32"),
            "ri": ParamSpec((s.blocks, b, b)), "ri_bias": ParamSpec((s.blocks, b), "bias32"),
            "lam": ParamSpec((c,), "vector32"),
            "o": ParamSpec((s.hidden_size, c)),
        }

    def set_params(self, params):
        self.yx = torch.cat([params["y"], params["x"]], dim=0).contiguous()
        self.y_bias, self.x_bias = params["y_bias"].float().contiguous(), params["x_bias"].float().contiguous()
        self.conv, self.conv_bias = params["conv"].float().contiguous(), params["conv_bias"].float().contiguous()
        # a block's two gate matrices side by side and transposed: one batched product gives [zr | zi] a block
        self.gates = torch.cat([params["ra"].transpose(1, 2), params["ri"].transpose(1, 2)], dim=2).contiguous()
        self.ra_bias = params["ra_bias"].float().reshape(-1).contiguous()
        self.ri_bias = params["ri_bias"].float().reshape(-1).contiguous()
        self.lam = params["lam"].float().contiguous()
        self.o = params["o"].contiguous()

    def __call__(self, x, ctx, entry, writes_cache=True):
        s, c = self.spec, self.spec.width
        state = self._state(ctx, entry, writes_cache)
        seqs = (ctx.seq_slot, ctx.seq_q_start, ctx.seq_q_len, ctx.max_q_len)
        proj = ops.linear(x, self.yx, status=ctx.status)                      # [y | x]
        u = ops.short_conv(proj, c, c, self.conv, self.conv_bias, self.x_bias, state, 0, *seqs)
        parts = u.view(u.shape[0], s.blocks, self.block).transpose(0, 1)
        # the gates' logits stay 32-bit (a library product, as the head-wise products of the latent attention are)
        if u.dtype == torch.float32:
            logits = torch.bmm(parts, self.gates)
        else:
            logits = torch.bmm(parts, self.gates, out_dtype=torch.float32)
        out = ops.glru_scan(u, logits, self.ra_bias, self.ri_bias, self.lam, s.decay_scale, proj, 0, self.y_bias,
                            state, (s.conv - 1) * c, *seqs)
        return ops.linear(out, self.o, status=ctx.status)

    def weight_bytes(self):
        return bytes_of(self.yx, self.y_bias, self.x_bias, self.conv, self.conv_bias, self.gates, self.ra_bias,
                        self.ri_bias, self.lam, self.o)


class StateSpaceMixer(_Recurrent):
    def __init__(self, spec, dtype, position=None):
        super().__init__(spec, dtype, position)
        if spec.num_heads % spec.groups:
            raise ValueError(f"{spec.num_heads} heads cannot share {spec.groups} groups")
        self.inner = spec.num_heads * spec.head_dim
        self.bc = spec.groups * spec.state
        self.convolved = self.inner + 2 * self.bc
        if self.inner % spec.norm_groups:
            raise ValueError(f"{self.inner} entries do not split into {spec.norm_groups} norm groups")

    def state_need(self):
        s = self.spec
        return StateNeed(((s.conv - 1) * self.convolved + s.num_heads * s.state * s.head_dim,), "float32")

    def param_specs(self):
        s = self.spec
        return {
            "in": ParamSpec((2 * self.inner + 2 * self.bc + s.num_heads, s.hidden_size)),
            "conv": ParamSpec((self.convolved, s.conv), "vector32"), "conv_bias": ParamSpec((self.convolved,), "bias32"),
            "dt_bias": ParamSpec((s.num_heads,), "vector32"), "A_log": ParamSpec((s.num_heads,), "vector32"),
            "D": ParamSpec((s.num_heads,), "vector32"), "norm": ParamSpec((self.inner,), "gain32"),
            "o": ParamSpec((s.hidden_size, self.inner)),
        }

    def set_params(self, params):
        self.w_in = _padded_rows([params["in"]], self.spec.hidden_size)       # [z | x | B | C | dt]
        self.conv, self.conv_bias = params["conv"].float().contiguous(), params["conv_bias"].float().contiguous()
        self.dt_bias, self.A_log, self.D = (params[n].float().contiguous() for n in ("dt_bias", "A_log", "D"))
        self.gain = params["norm"].float().contiguous()
        self.o = params["o"].contiguous()

    def __call__(self, x, ctx, entry, writes_cache=True):
        s = self.spec
        state = self._state(ctx, entry, writes_cache)
        seqs = (ctx.seq_slot, ctx.seq_q_start, ctx.seq_q_len)
        proj = ops.linear(x, self.w_in, status=ctx.status)
        xbc = ops.short_conv(proj, self.inner, self.convolved, self.conv, self.conv_bias, None, state, 0, *seqs,
                             ctx.max_q_len, "silu")
        y = ops.state_scan("state_space", (xbc, self.inner + self.bc), (xbc, self.inner), (xbc, 0),
                           (proj, self.inner + self.convolved), None, self.A_log, self.dt_bias, self.D, state,
                           (s.conv - 1) * self.convolved, *seqs, s.num_heads, s.groups, s.state, s.head_dim)
        y = ops.group_norm_gate(y, proj, 0, self.gain, s.norm_groups, s.norm_eps, True, x.dtype)
        return ops.linear(y, self.o, status=ctx.status)

    def weight_bytes(self):
        return bytes_of(self.w_in, self.conv, self.conv_bias, self.dt_bias, self.A_log, self.D, self.gain, self.o)


class GatedDeltaMixer(_Recurrent):
    def __init__(self, spec, dtype, position=None):
        super().__init__(spec, dtype, position)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} heads cannot share {spec.num_kv_heads} query/key heads")
        self.qk = spec.num_kv_heads * spec.head_dim
        self.inner = spec.num_heads * spec.value_dim
        self.convolved = 2 * self.qk + self.inner

    def state_need(self):
        s = self.spec
        return StateNeed(((s.conv - 1) * self.convolved + s.num_heads * s.head_dim * s.value_dim,), "float32")

    def param_specs(self):
        s = self.spec
        return {
            "q": ParamSpec((self.qk, s.hidden_size)), "q_conv": ParamSpec((self.qk, s.conv), "vector32"),
            "k": ParamSpec((self.qk, s.hidden_size)), "k_conv": ParamSpec((self.qk, s.conv), "vector32"),
            "v": ParamSpec((self.inner, s.hidden_size)), "v_conv": ParamSpec((self.inner, s.conv), "vector32"),
            "b": ParamSpec((s.num_heads, s.hidden_size)), "a": ParamSpec((s.num_heads, s.hidden_size)),
            "A_log": ParamSpec((s.num_heads,), "vector32"), "dt_bias": ParamSpec((s.num_heads,), "vector32"),
            "norm": ParamSpec((s.value_dim,), "gain32"),
            "g": ParamSpec((self.inner, s.hidden_size)), "o": ParamSpec((s.hidden_size, self.inner)),
        }

    def set_params(self, params):
        # one product for [q | k | v | g | b | a]
        self.stacked = _padded_rows([params[n] for n in ("q", "k", "v", "g", "b", "a")], self.spec.hidden_size)
        self.conv = torch.cat([params[n].float() for n in ("q_conv", "k_conv", "v_conv")], dim=0).contiguous()
        self.A_log, self.dt_bias = params["A_log"].float().contiguous(), params["dt_bias"].float().contiguous()
        self.gain = params["norm"].float().contiguous()
        self.o = params["o"].contiguous()

    def __call__(self, x, ctx, entry, writes_cache=True):
        s = self.spec
        state = self._state(ctx, entry, writes_cache)
        seqs = (ctx.seq_slot, ctx.seq_q_start, ctx.seq_q_len)
        proj = ops.linear(x, self.stacked, status=ctx.status)
        qkv = ops.short_conv(proj, 0, self.convolved, self.conv, None, None, state, 0, *seqs, ctx.max_q_len, "silu")
        gate_at = self.convolved
        beta_at = gate_at + self.inner
        o = ops.state_scan("gated_delta", (qkv, 0), (qkv, self.qk), (qkv, 2 * self.qk), (proj, beta_at + s.num_heads),
                           (proj, beta_at), self.A_log, self.dt_bias, None, state, (s.conv - 1) * self.convolved, *seqs,
                           s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim)
        y = ops.group_norm_gate(o, proj, gate_at, self.gain, s.num_heads, s.norm_eps, False, x.dtype)
        return ops.linear(y, self.o, status=ctx.status)

    def weight_bytes(self):
        return bytes_of(self.stacked, self.conv, self.A_log, self.dt_bias, self.gain, self.o)
