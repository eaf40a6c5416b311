"""Grouped-query attention whose positions enter through the scores and the mask: a logarithmic distance
penalty per head, chunks of the sequence, a window, a sink in the softmax (learnt per head, or a fixed number), a
sigmoid gate per head (each optional, see ``SinkAttentionSpec``); optionally with rotary positions on the leading
entries of queries and keys, and with the keys as projected standing in for values.

One step of it: one stacked product gives ``[q | k | v | g]``; ``ops.sink_prepare`` files keys and values
at each token's own position and forms the gates; the attention kernel reads the queries from the stacked
rows, the keys and values from the cache, and applies the gate; the output projection follows.  A whole
prompt, a later portion and a single token are the same code: every query is told its absolute position,
and chunks are counted from the sequence's start.
"""

from __future__ import annotations

import torch

from .. import ops
from ..cache.layout import KVNeed
from .base import ParamSpec, Part, bytes_of


class SinkAttention(Part):
    def __init__(self, spec, dtype, position=None):
        super().__init__(spec, dtype)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} query heads cannot share {spec.num_kv_heads} key/value heads")
        if (position is None) != (spec.position is None):
            raise ValueError("the attention's spec and the position part it is handed do not agree")
        if (position is not None or spec.values_from_keys) and spec.head_gate:
            raise ValueError("head gates are formed by the kernel that files keys and values without a rotation")
        if spec.values_from_keys and spec.value_dim != spec.head_dim:
            raise ValueError(f"values taken from the keys have their size: {spec.head_dim}, not {spec.value_dim}")
        if spec.fixed_sink is not None and spec.sink:
            raise ValueError("a sink is either learnt per head or a fixed number")
        self.position = position
        if max(spec.head_dim, spec.value_dim) > 256:
            raise ValueError(f"head sizes {spec.head_dim} / {spec.value_dim} exceed the 256 entries the kernels take")
        self.q_size = spec.num_heads * spec.head_dim
        self.kv_size = spec.num_kv_heads * (spec.head_dim + (0 if spec.values_from_keys else spec.value_dim))
        self.penalty = self.sink = None

    def kv_need(self):
        s = self.spec
        # every key stays: a later query of the same chunk may still read it (chunks bound what is read)
        return KVNeed(s.num_kv_heads, s.head_dim, s.window, s.value_dim)

    def state_need(self):
        return None

    def param_specs(self):
        s = self.spec
        out = {
            "q": ParamSpec((self.q_size, s.hidden_size)),
            "k": ParamSpec((s.num_kv_heads * s.head_dim, s.hidden_size)),
            "v": ParamSpec((s.num_kv_heads * s.value_dim, s.hidden_size)),
            "o": ParamSpec((s.hidden_size, s.num_heads * s.value_dim)),
        }
        if s.values_from_keys:
            del out["v"]
        if s.distance_penalty:
            out["r1"] = ParamSpec((s.num_heads,), "vector32")
            out["r2"] = ParamSpec((s.num_heads,), "slope")
        if s.sink:
            out["sink"] = ParamSpec((s.num_heads,), "vector32")
        if s.head_gate:
            out["g"] = ParamSpec((s.num_heads, s.hidden_size))
        return out

    def set_params(self, params):
        s = self.spec
        def stacked(rows):
            # rows of zeros bring the product's width to a multiple of 8, so that every token's queries
            # start on a 16-byte boundary for the kernels that copy them in 16-byte pieces
            pad = -sum(r.shape[0] for r in rows) % 8
            if pad:
                rows = rows + [torch.zeros((pad, s.hidden_size), dtype=rows[0].dtype, device=rows[0].device)]
            return torch.cat(rows, dim=0).contiguous()

        own_values = [] if s.values_from_keys else [params["v"]]
        self.qkvg = stacked([params["q"], params["k"]] + own_values + ([params["g"]] if s.head_gate else []))
        # the rows a layer that only reads another layer's cache needs: queries and gates
        self.qg = stacked([params["q"]] + ([params["g"]] if s.head_gate else []))
        self.o = params["o"].contiguous()
        if s.distance_penalty:
            self.penalty = (params["r1"].float().contiguous(), params["r2"].float().contiguous())
        if s.sink:
            self.sink = params["sink"].float().contiguous()
        elif s.fixed_sink is not None:
            self.sink = torch.full((s.num_heads,), float(s.fixed_sink), dtype=torch.float32, device=self.o.device)

    def prepare(self, max_position: int) -> bool:
        """Host-side growth before a step; True if device tables were reallocated."""
        if self.position is not None:
            return bool(self.position.ensure(max_position + 1))
        return False

    def __call__(self, x, ctx, entry, writes_cache=True):
        s = self.spec
        cache = ctx.cache
        keys, values = cache.entry_pages(entry)
        weight = self.qkvg if writes_cache else self.qg
        proj = ops.linear(x, weight, status=ctx.status)
        if self.position is not None or s.values_from_keys:
            # queries turned in place, keys turned on their way into the cache, values as projected
            cos, sin, dims = ops.sink_tables(self.position.rotation() if self.position is not None else None, s.head_dim)
            ops.sink_prepare_rot(proj, s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim, ctx.tok_pos, ctx.tok_slot,
                                 cache.block_table, keys, values, cos, sin, dims, values_from_keys=s.values_from_keys,
                                 write_cache=writes_cache)
            a = ops.sink_attention_step(proj, keys, values, cache.block_table, ctx, s.num_heads, s.num_kv_heads,
                                        s.head_dim, s.value_dim, s.scale, self.penalty, self.sink, None, s.chunk, s.window)
            return ops.linear(a, self.o, status=ctx.status)
        gate = ops.sink_prepare(proj, s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim, ctx.tok_pos, ctx.tok_slot,
                                cache.block_table, keys, values, gated=s.head_gate, write_cache=writes_cache)
        a = ops.sink_attention_step(proj, keys, values, cache.block_table, ctx, s.num_heads, s.num_kv_heads,
                                    s.head_dim, s.value_dim, s.scale, self.penalty, self.sink, gate, s.chunk, s.window)
        return ops.linear(a, self.o, status=ctx.status)

    def weight_bytes(self):
        return bytes_of(self.qkvg, self.o, self.sink, *(self.penalty or ()))
