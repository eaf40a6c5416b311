"""Attention over a cached low-rank latent with a rotated key part that all heads share, and a window.

One step of it: one stacked product gives ``[query latent | key/value latent | shared key part]``;
``ops.latent_prepare`` norms the two latents, turns the shared part by the token's position and files
latent and shared part in the token's cache row; the query up-projection follows.  The key
up-projection is not applied to the cache: it is folded into the query, head by head (``q' = W_uk^T
q_plain``), so the attention kernel scores ``q' . c + q_rot . shared`` against the cache rows as they
are and sums the latents; the value up-projection is applied to that sum, head by head, and the output
projection follows.  A whole prompt, a later portion and a single token are the same code: every query
is told its absolute position.

A layer whose spec says ``own_kv = False`` has no key/value down-projection: the run order gives it the
cache entry of the layer whose latent it reads (``writes_cache`` false).
"""

from __future__ import annotations

import torch

from .. import ops
from ..cache.layout import KVNeed
from .base import ParamSpec, Part, bytes_of


class LatentAttention(Part):
    def __init__(self, spec, dtype, position=None):
        super().__init__(spec, dtype)
        if spec.kv_rank + spec.rot_dim > 640:
            raise ValueError(f"kv_rank + rot_dim = {spec.kv_rank + spec.rot_dim} exceeds the 640 entries a cache "
                             "row of the latent-attention kernels holds")
        if position is None:
            raise ValueError("latent attention needs its position part")
        self.position = position
        self.row = spec.kv_rank + spec.rot_dim

    # what this mixer keeps per token: one row for all heads, and no separate values
    def kv_need(self):
        if not self.spec.own_kv:
            return None
        return KVNeed(1, self.row, self.spec.window, 0)

    def state_need(self):
        return None

    def param_specs(self):
        s = self.spec
        out = {
            "dq": ParamSpec((s.q_rank, s.hidden_size)),
            "dq_norm": ParamSpec((s.q_rank,), "gain32"),
            "uq": ParamSpec((s.num_heads * (s.head_dim + s.rot_dim), s.q_rank)),
            "uk": ParamSpec((s.num_heads * s.head_dim, s.kv_rank)),
            "uv": ParamSpec((s.num_heads * s.value_dim, s.kv_rank)),
            "o": ParamSpec((s.hidden_size, s.num_heads * s.value_dim)),
        }
        if s.own_kv:
            out["dkv"] = ParamSpec((s.kv_rank + s.rot_dim, s.hidden_size))
            out["dkv_norm"] = ParamSpec((s.kv_rank,), "gain32")
        return out

    def set_params(self, params):
        s = self.spec
        rows = [params["dq"]] + ([params["dkv"]] if s.own_kv else [])
        self.down = torch.cat(rows, dim=0).contiguous()
        self.q_gain = params["dq_norm"].float().contiguous()
        self.kv_gain = params["dkv_norm"].float().contiguous() if s.own_kv else None
        self.uq = params["uq"].contiguous()
        # per head: [dim, kv_rank] (folded into the query) and [kv_rank, vdim] (applied to the summed latents)
        self.uk = params["uk"].contiguous().view(s.num_heads, s.head_dim, s.kv_rank)
        self.uv = params["uv"].contiguous().view(s.num_heads, s.value_dim, s.kv_rank).transpose(1, 2)
        self.o = params["o"].contiguous()

    def prepare(self, max_position: int) -> bool:
        return bool(self.position.ensure(max_position + 1))

    def __call__(self, x, ctx, entry, writes_cache=True):
        s = self.spec
        if writes_cache and not s.own_kv:
            raise ValueError("a latent attention without a key/value down-projection cannot fill a cache entry")
        cache = ctx.cache
        store, _ = cache.entry_pages(entry)
        weight = self.down if writes_cache else self.down[: s.q_rank]
        proj = ops.linear(x, weight, status=ctx.status)
        rotation = self.position.rotation()
        cos, sin = ops.latent_tables(rotation, s.position.dims)
        cq = ops.latent_prepare(proj, self.q_gain, self.kv_gain, s.norm_eps, cos, sin, ctx.tok_pos, ctx.tok_slot,
                                cache.block_table, store, s.q_rank, s.kv_rank, s.rot_dim, s.position.dims,
                                write_cache=writes_cache, layout=rotation.layout)
        q = ops.linear(cq, self.uq, status=ctx.status)
        n = q.shape[0]
        qa = torch.empty((n, s.num_heads, self.row), dtype=q.dtype, device=q.device)
        q3 = q.view(n, s.num_heads, s.head_dim + s.rot_dim)
        torch.bmm(q3[:, :, : s.head_dim].transpose(0, 1), self.uk, out=qa[:, :, : s.kv_rank].transpose(0, 1))
        ops.latent_rotate_q(q, qa, cos, sin, ctx.tok_pos, s.num_heads, s.head_dim, s.rot_dim, s.position.dims,
                            s.kv_rank, layout=rotation.layout)
        summed = ops.latent_attention_step(qa, store, cache.block_table, ctx, s.num_heads, s.kv_rank, s.rot_dim,
                                           s.scale, s.window)
        a = torch.empty((n, s.num_heads, s.value_dim), dtype=q.dtype, device=q.device)
        torch.bmm(summed.transpose(0, 1), self.uv, out=a.transpose(0, 1))
        return ops.linear(a.view(n, s.num_heads * s.value_dim), self.o, status=ctx.status)

    def weight_bytes(self):
        return bytes_of(self.down, self.q_gain, self.kv_gain, self.uq, self.uk, self.uv, self.o)
